"""gs.jit.compile on the GPU: the rewritten graph returns what the eager function returns (same seed sequence)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def graphsage(A, seeds, fanouts):
    input_node, blocks = seeds, []
    for fanout in fanouts:
        subA = A[:, seeds].columnwise_sampling(fanout, False)
        seeds = subA.all_indices()
        blocks.append(subA)
    return input_node, seeds, blocks


def ladies_layer(A, seeds, k):
    sub = A[:, seeds]
    p = sub.sum(1, 2)
    rows = sub.row_ids(False)
    return sub, p, rows


def test_compiled_graphsage_equals_eager(cfg1_graph):
    import graph_sampling_b200.gs as gs
    indptr, indices = cfg1_graph
    m = gs.Matrix().load_csc(dev(indptr), dev(indices))
    seeds = dev(np.random.default_rng(0).choice(len(indptr) - 1, 1024, replace=False).astype(np.int64))
    compiled = gs.jit.compile(graphsage, (m, seeds, [10, 5]))
    assert compiled.targets().count("_CAPI_fused_columnwise_slicing_sampling") == 2
    gs.set_seed(42)
    _, f_eager, b_eager = graphsage(m, seeds, [10, 5])
    gs.set_seed(42)
    inp, f_comp, b_comp = compiled(m, seeds, [10, 5])
    assert torch.equal(inp, seeds) and torch.equal(f_eager, f_comp)
    for e, c in zip(b_eager, b_comp):
        assert isinstance(c, gs.Matrix)
        assert torch.equal(e.row_indices(), c.row_indices())
        be, bc = e.to_block(), c.to_block()
        assert torch.equal(be.src_ids, bc.src_ids) and be.num_src == bc.num_src and be.num_dst == bc.num_dst
        assert (be.format, bc.format) == ("coo", "csc")       # same block, handed over in the fused operator's format
        assert torch.equal(be.tensor1, bc.tensor2)            # coo rows == csc indices
    # a different batch through the same compiled object
    seeds2 = seeds.flip(0)[:512].contiguous()
    gs.set_seed(7)
    want = graphsage(m, seeds2, [10, 5])[1]
    gs.set_seed(7)
    assert torch.equal(compiled(m, seeds2, [10, 5])[1], want)


def test_compiled_deterministic_pipeline_and_torchscript_handle(cfg1_graph):
    import graph_sampling_b200.gs as gs
    from graph_sampling_b200 import build as b
    indptr, indices = cfg1_graph
    w = torch.rand(len(indices), device="cuda")
    m = gs.Matrix().load_csc(dev(indptr), dev(indices), w)
    seeds = torch.arange(0, 3000, 7, device="cuda")
    compiled = gs.jit.compile(ladies_layer, (m, seeds, 64))
    sub_e, p_e, rows_e = ladies_layer(m, seeds, 64)
    sub_c, p_c, rows_c = compiled(m, seeds, 64)
    assert torch.equal(p_e, p_c) and torch.equal(rows_e, rows_c)
    assert torch.equal(sub_e.row_indices(), sub_c.row_indices())
    # the same compiled graph drives a TorchScript graph object (methods are looked up by name)
    torch.classes.load_library(b.build_glue())
    g = torch.classes.gs_classes.Graph(False)
    g._CAPI_load_csc(dev(indptr), dev(indices))
    g._CAPI_set_data(w)
    sub_t, p_t, rows_t = compiled(gs.Matrix(g), seeds, 64)
    assert torch.allclose(p_e, p_t) and torch.equal(rows_e, rows_t)
