"""Doubly compressed formats (DCSC / DCSR: offsets only over the columns / rows that have edges): the reference's
own unit tests for them, and the invariant that every operator gives the same answer on the compact form as on
the plain one."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
_COO, _CSC, _CSR, _DCSC, _DCSR = 1, 2, 4, 8, 16


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


class _PythonFace:
    def __init__(self):
        import graph_sampling_b200.gs as gs
        self.Graph = gs.Graph


class _TorchScriptFace:
    def __init__(self):
        from graph_sampling_b200 import build as b
        torch.classes.load_library(b.build_glue())
        self.Graph = torch.classes.gs_classes.Graph


@pytest.fixture(scope="module", params=["python", "torchscript"])
def face(request):
    return _PythonFace() if request.param == "python" else _TorchScriptFace()


def toy(face):
    """tests/test_rowwise_slicing.cc:22-40: 12 columns, only the last two have edges (rows 5 and 6 each)."""
    g = face.Graph(False)
    indptr = torch.cat([torch.zeros(10, dtype=torch.int64), torch.arange(0, 3) * 2]).cuda()
    indices = torch.arange(5, 7).repeat(2).cuda()
    g._CAPI_LoadCSC(indptr, indices)
    return g


def test_reference_unit_tests_on_dcsr(face):
    # tests/test_rowwise_slicing.cc:22-40
    sub = toy(face)._CAPI_Slicing(torch.arange(5, 6).cuda(), 1, _DCSR, _CSR, False)
    c = sub._CAPI_Metadata() if False else None
    coo_rows, coo_cols = sub._CAPI_GetCOORows(False), sub._CAPI_GetCooCols(False)
    assert host(coo_cols).tolist() == [10, 11] and host(coo_rows).tolist() == [0, 0]
    # tests/test_relabel.cc:28-51: the same slice with relabelling of the columns
    g = toy(face)
    sub = g._CAPI_Slicing(torch.arange(5, 6).cuda(), 1, _DCSR, _CSR, True)
    assert (g._CAPI_GetNumCols(), g._CAPI_GetNumRows()) == (12, 12)
    assert (sub._CAPI_GetNumCols(), sub._CAPI_GetNumRows()) == (2, 1)
    assert host(sub._CAPI_GetCooCols(False)).tolist() == [0, 1]
    assert host(sub._CAPI_GetCols()).tolist() == [10, 11]


def _graph(face, small_graph, with_data=True):
    indptr, indices = small_graph
    g = face.Graph(False)
    g._CAPI_LoadCSC(dev(indptr), dev(indices))
    if with_data:
        w = np.random.default_rng(0).random(len(indices)).astype(np.float32) + 0.25
        g._CAPI_SetData(dev(w))
    return g


def test_compact_forms_agree_with_plain_forms(face, small_graph):
    indptr, indices = small_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(1)
    # a column-sliced graph has many empty rows: its DCSR is much shorter than its CSR
    seeds = dev(rng.choice(n, 150, replace=False).astype(np.int64))
    rows = dev(rng.choice(n, 400, replace=False).astype(np.int64))

    def sliced():
        return _graph(face, small_graph)._CAPI_Slicing(seeds, 0, _CSC, _CSC + _COO, False)

    plain, compact = sliced(), sliced()
    a = plain._CAPI_Slicing(rows, 1, _CSR, _CSR + _COO, False)
    b = compact._CAPI_Slicing(rows, 1, _DCSR, _CSR + _COO, False)
    assert torch.equal(a._CAPI_GetCOORows(False), b._CAPI_GetCOORows(False))
    assert torch.equal(a._CAPI_GetCooCols(False), b._CAPI_GetCooCols(False))
    assert torch.equal(a._CAPI_GetData("default"), b._CAPI_GetData("default"))
    assert a._CAPI_GetNumEdges() == b._CAPI_GetNumEdges() > 0
    # sums, normalisation and division per row on the compact form
    assert torch.allclose(plain._CAPI_Sum(1, 2, _CSR), compact._CAPI_Sum(1, 2, _DCSR), rtol=1e-5, atol=1e-6)
    div = torch.rand(n, device="cuda") + 0.5
    assert torch.equal(plain._CAPI_Divide(div, 1, _CSR)._CAPI_GetData("default"),
                       compact._CAPI_Divide(div, 1, _DCSR)._CAPI_GetData("default"))
    assert torch.allclose(plain._CAPI_Normalize(1, _CSR)._CAPI_GetData("default"),
                          compact._CAPI_Normalize(1, _DCSR)._CAPI_GetData("default"), rtol=1e-5, atol=1e-7)
    # valid rows come straight from the compact form
    assert torch.equal(torch.sort(plain._CAPI_GetValidRows())[0], torch.sort(compact._CAPI_GetValidRows())[0])
    # SDDMM (u . v) on the compact form
    F = 16
    xs, xd = torch.randn(n, F, device="cuda"), torch.randn(seeds.numel(), F, device="cuda")
    E = plain._CAPI_GetNumEdges()
    o1, o2 = torch.zeros(E, 1, device="cuda"), torch.zeros(E, 1, device="cuda")
    plain._CAPI_SDDMM("dot", xs, xd, o1, 0, 2, _COO)
    compact._CAPI_SDDMM("dot", xs, xd, o2, 0, 2, _DCSR)
    assert torch.allclose(o1, o2, rtol=1e-5, atol=1e-5)


def test_dcsc_from_csr_and_format_errors(face, small_graph):
    g = _graph(face, small_graph, with_data=False)
    rows = torch.arange(0, 300, 3).cuda()
    rs = g._CAPI_Slicing(rows, 1, _CSR, _CSR, False)               # CSR only
    n_cols = rs._CAPI_GetNumCols()
    cols = torch.arange(0, n_cols, 7).cuda()
    a = rs._CAPI_Slicing(cols, 0, _DCSC, _CSC + _COO, False)       # CSR -> COO -> DCSC, then a compact column slice
    rs2 = g._CAPI_Slicing(rows, 1, _CSR, _CSR, False)
    b = rs2._CAPI_Slicing(cols, 0, _CSC, _CSC + _COO, False)
    assert torch.equal(a._CAPI_GetCOORows(False), b._CAPI_GetCOORows(False))
    assert torch.equal(a._CAPI_GetCooCols(False), b._CAPI_GetCooCols(False))
    with pytest.raises(RuntimeError):
        rs._CAPI_Slicing(cols, 0, _CSC, _CSC, False)               # holds a DCSC now: "Require CSC, get DCSC instead"
    with pytest.raises(RuntimeError):
        rs2._CAPI_Slicing(cols, 0, _DCSC, _CSC, False)             # and the other way round
