"""gs.jit.compile: tracing and graph rewrites (no GPU: tracing runs no kernel); execution equality is in the GPU test."""
import pytest
import torch


@pytest.fixture(scope="module")
def gs():
    import graph_sampling_b200.gs as m
    return m


def graphsage(A, seeds, fanouts):
    input_node, ret = seeds, []
    for fanout in fanouts:
        subA = A[:, seeds]
        subA = subA.columnwise_sampling(fanout, False)
        seeds = subA.all_indices()
        ret.append(subA)
    return input_node, seeds, ret


def test_slicing_sampling_fusion_and_static_fanouts(gs):
    m = gs.Matrix(gs.Graph(False))
    c = gs.jit.compile(graphsage, (m, torch.arange(4), [25, 15]))
    t = c.targets()
    assert t.count("_CAPI_fused_columnwise_slicing_sampling") == 2
    assert "_CAPI_slicing" not in t and "_CAPI_sampling" not in t
    assert "25" in c.gm.code and "15" in c.gm.code          # fanouts are constants of the graph
    c = gs.jit.compile(graphsage, (m, torch.arange(4), [25, 15]), fuse_slicing_sampling=False)
    assert c.targets().count("_CAPI_slicing") == 2 and c.targets().count("_CAPI_sampling") == 2


def test_fusion_is_skipped_when_the_slice_or_sample_is_used_elsewhere(gs):
    def keeps_slice(A, seeds):
        sl = A[:, seeds]
        return sl.columnwise_sampling(5, False), sl.sum(0)

    def format_dependent_user(A, seeds):
        s = A[:, seeds].columnwise_sampling(5, False)
        return s._graph._CAPI_get_coo(), s.all_indices()

    m = gs.Matrix(gs.Graph(False))
    assert "_CAPI_fused_columnwise_slicing_sampling" not in gs.jit.compile(keeps_slice, (m, torch.arange(3))).targets()
    assert "_CAPI_fused_columnwise_slicing_sampling" not in gs.jit.compile(format_dependent_user,
                                                                           (m, torch.arange(3))).targets()


def test_relabel_and_all_indices_share_one_call(gs):
    def hop(A, seeds):
        sub = A[:, seeds].columnwise_sampling(5, False)
        frontier = sub.all_indices()
        r = sub._graph._CAPI_relabel()
        return frontier, r[0], r[3], r[4]

    c = gs.jit.compile(hop, (gs.Matrix(gs.Graph(False)), torch.arange(3)))
    t = c.targets()
    assert t.count("_CAPI_relabel") == 1 and "_CAPI_all_valid_node" not in t


def test_cse_keeps_two_samples_and_merges_two_getters_and_dce_keeps_side_effects(gs):
    def f(A, seeds, w):
        sub = A[:, seeds]
        a = sub.columnwise_sampling(5, False)
        b = sub.columnwise_sampling(5, False)          # a second, independent sample
        r1, r2 = sub.row_ids(False), sub.row_ids(False)
        unused = sub.sum(0)                            # dead
        sub.set_data(w)                                # side effect: must stay
        return a, b, r1, r2

    c = gs.jit.compile(f, (gs.Matrix(gs.Graph(False)), torch.arange(3), torch.ones(3)))
    t = c.targets()
    assert t.count("_CAPI_sampling") == 2
    assert t.count("_CAPI_get_rows") == 1
    assert "_CAPI_sum" not in t and "_CAPI_set_data" in t


def test_call_checks_arity(gs):
    c = gs.jit.compile(graphsage, (gs.Matrix(gs.Graph(False)), torch.arange(4), [3]))
    with pytest.raises(TypeError):
        c(torch.arange(4))
