"""Graphs whose arrays stay in pinned host memory (the reference's large-graph mode: src/graph_ops.cc:144,226,
src/cuda/slicing.cu:128, examples/fastgcn/unbatching_training.py:48-51).  The kernels read the pinned arrays in place,
so every result must equal, bit for bit, the one computed from a device copy of the same graph with the same seed."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

_COO, _CSC, _CSR = 1, 2, 4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def pin(a):
    return torch.from_numpy(np.ascontiguousarray(a)).pin_memory()


class _PythonFace:
    def __init__(self):
        import graph_sampling_b200.gs as gs
        self.Graph, self.ops = gs.Graph, gs.gs_ops


class _TorchScriptFace:
    def __init__(self):
        from graph_sampling_b200 import build as b
        torch.classes.load_library(b.build_glue())
        self.Graph, self.ops = torch.classes.gs_classes.Graph, torch.ops.gs_ops


@pytest.fixture(scope="module", params=["python", "torchscript"])
def face(request):
    return _PythonFace() if request.param == "python" else _TorchScriptFace()


def both(face, small_graph, weights=None):
    indptr, indices = small_graph
    out = []
    for put in (dev, pin):
        g = face.Graph(False)
        g._CAPI_LoadCSC(put(indptr), put(indices))
        if weights is not None:
            g._CAPI_SetData(put(weights))
        out.append(g)
    return out


def same_graph(a, b):
    ca, cb = a._CAPI_GetCOO(), b._CAPI_GetCOO()
    assert ca[0].is_cuda and cb[0].is_cuda
    assert torch.equal(ca[0], cb[0]) and torch.equal(ca[1], cb[1])
    da, db = a._CAPI_GetData("default"), b._CAPI_GetData("default")
    assert (da is None) == (db is None)
    if da is not None:
        assert db.is_cuda and torch.equal(da, db)


def test_pinned_graph_matches_device_graph(face, small_graph):
    indptr, indices = small_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(3)
    w = rng.random(len(indices)).astype(np.float32)
    seeds = dev(rng.choice(n, 300, replace=False).astype(np.int64))
    rows = dev(rng.choice(n, n // 2, replace=False).astype(np.int64))
    on_dev, on_host = both(face, small_graph, w)
    same_graph(on_dev._CAPI_Slicing(seeds, 0, _CSC, _COO, False), on_host._CAPI_Slicing(seeds, 0, _CSC, _COO, False))
    same_graph(on_dev._CAPI_FusionSlicing(seeds, rows), on_host._CAPI_FusionSlicing(seeds, rows))
    for fanout, replace in ((5, False), (3, True), (1, True)):
        face.ops._CAPI_SetSeed(11)
        a = on_dev._CAPI_FusedColumnwiseSlicingSampling(seeds, fanout, replace)
        face.ops._CAPI_SetSeed(11)
        b = on_host._CAPI_FusedColumnwiseSlicingSampling(seeds, fanout, replace)
        same_graph(a, b)
    face.ops._CAPI_SetSeed(5)
    a = on_dev._CAPI_RandomWalk(seeds, 6)
    face.ops._CAPI_SetSeed(5)
    b = on_host._CAPI_RandomWalk(seeds, 6)
    assert b.is_cuda and torch.equal(a, b)
    # a sampled subgraph of a pinned graph is an ordinary device graph: everything downstream works on it
    sub = on_host._CAPI_FusedColumnwiseSlicingSampling(seeds, 5, False)
    frontier = sub._CAPI_AllValidNode()
    assert frontier.is_cuda and torch.equal(frontier[:seeds.numel()], seeds)
    assert sub._CAPI_Sum(0, 1, _CSC).is_cuda


def test_pageable_host_graph_is_rejected(face, small_graph):
    indptr, indices = small_graph
    g = face.Graph(False)
    with pytest.raises((TypeError, RuntimeError), match="pinned"):                  # neither device nor pinned
        g._CAPI_LoadCSC(torch.from_numpy(indptr), torch.from_numpy(indices))
        g._CAPI_Slicing(dev(np.array([1, 2], dtype=np.int64)), 0, _CSC, _COO, False)


def test_multi_hop_sampler_over_pinned_graph(small_graph):
    from graph_sampling_b200 import ops
    indptr, indices = small_graph
    n = len(indptr) - 1
    seeds = dev(np.random.default_rng(8).choice(n, 4 * 64, replace=False).astype(np.int64))
    seeds_ptr = dev(np.arange(0, 4 * 64 + 1, 64, dtype=np.int64))
    a = ops.sage_sample_batches(dev(indptr), dev(indices), seeds, seeds_ptr, [4, 3], seed=21)
    b = ops.sage_sample_batches(pin(indptr), pin(indices), seeds, seeds_ptr, [4, 3], seed=21)
    assert len(a) == len(b) == 2
    for ha, hb in zip(a, b):
        assert ha.keys() == hb.keys()
        for key in ha:
            if isinstance(ha[key], torch.Tensor):
                assert hb[key].is_cuda and torch.equal(ha[key], hb[key]), key
