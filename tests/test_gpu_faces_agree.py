"""The two host layers over the C ABI — the Python `Graph` (graph_sampling_b200/graph.py) and the TorchScript class
of lib/libgs.so (csrc/glue/gs_glue.cc) — restate the same gs::Graph bookkeeping (src/graph.cc) separately.  This test
keeps them from drifting: it enumerates EVERY method name the TorchScript class registers, requires the Python face
to answer to the same name, and runs a recipe for each name on both faces from the same state, comparing every
returned tensor, number and child graph (stochastic methods included: both faces derive their per-call seeds the
same way from a base seed).  A name that is registered without a recipe fails the test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
_COO, _CSC, _CSR = 1, 2, 4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def faces():
    import graph_sampling_b200.gs as pygs
    from graph_sampling_b200 import build as b, ops
    torch.classes.load_library(b.build_glue())
    return {"python": (pygs.Graph, lambda s: ops.set_seed(s)),
            "torchscript": (torch.classes.gs_classes.Graph, lambda s: torch.ops.gs_ops._CAPI_SetSeed(s))}


def is_graph(x):
    return hasattr(x, "_CAPI_GetNumEdges") or (hasattr(x, "_method_names") and "_CAPI_GetNumEdges" in x._method_names())


def snapshot(x):
    """Everything observable of a result, as nested lists of numpy arrays / numbers / strings."""
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    if isinstance(x, (int, float, str, bool)):
        return x
    if isinstance(x, (list, tuple)):
        return [snapshot(v) for v in x]
    if is_graph(x):
        out = ["graph", int(x._CAPI_GetNumRows()), int(x._CAPI_GetNumCols()), int(x._CAPI_GetNumEdges())]
        out.append(snapshot(list(x._CAPI_CSCMetadata())))
        out.append(snapshot(list(x._CAPI_COOMetadata())))
        return out
    raise TypeError(type(x))


def same(a, b, path=""):
    if isinstance(a, list):
        assert isinstance(b, list) and len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            same(x, y, f"{path}[{i}]")
    elif isinstance(a, np.ndarray):
        assert isinstance(b, np.ndarray) and a.shape == b.shape and a.dtype == b.dtype, path
        if a.dtype.kind == "f":
            assert np.allclose(a, b, rtol=1e-6, atol=1e-7), path
        else:
            assert np.array_equal(a, b), path
    else:
        assert a == b, (path, a, b)


@pytest.fixture(scope="module")
def inputs(small_graph):
    indptr, indices = small_graph
    rng = np.random.default_rng(3)
    n = len(indptr) - 1
    return {"indptr": dev(indptr), "indices": dev(indices), "n": n,
            "w": dev((rng.random(len(indices)) + 0.25).astype(np.float32)),
            "seeds": dev(rng.choice(n, 96, replace=False).astype(np.int64)),
            "rows": dev(rng.choice(n, 700, replace=False).astype(np.int64)),
            "x": dev(rng.standard_normal((n, 8)).astype(np.float32))}


def base(Graph, I):
    g = Graph(False)
    g._CAPI_LoadCSC(I["indptr"], I["indices"])
    g._CAPI_SetData(I["w"])
    return g


def sliced(Graph, I, fmt=_CSC + _COO):
    return base(Graph, I)._CAPI_Slicing(I["seeds"], 0, _CSC, fmt, False)


def batch_ptrs(I):
    return dev(np.array([0, 32, 64, 96], dtype=np.int64)), dev(np.array([0, 200, 450, 700], dtype=np.int64))


def r_sddmm(G, I):
    s = sliced(G, I)
    out = torch.zeros(int(s._CAPI_GetNumEdges()), 1, device="cuda")
    s._CAPI_SDDMM("dot", I["x"], I["x"][I["seeds"]], out, 0, 2, _COO)
    return out


def r_set_coo(G, I):
    s = sliced(G, I)
    row, col, e = s._CAPI_GetCOO()
    g = G(True)
    g._CAPI_SetMetadata(None, None, 96, I["n"])
    g._CAPI_SetCOO(row, col, e, False, True)
    return [g, g._CAPI_GetCSC()]


def r_load_coo(G, I):
    s = sliced(G, I)
    row, col, _ = s._CAPI_GetCOO()
    g = G(False)
    g._CAPI_LoadCOO(row, col)
    return [int(g._CAPI_GetNumRows()), int(g._CAPI_GetNumEdges()), g._CAPI_GetCOORows(False), g._CAPI_GetCooCols(False)]


def r_decode(G, I):
    cp, _ = batch_ptrs(I)
    g, offs = base(G, I)._CAPI_BatchSlicing(I["seeds"], cp, 0, _CSC, _CSC + _COO, True, True)
    g._CAPI_Decode(I["n"])
    return [g, offs, g._CAPI_GetRows(), g._CAPI_GetCols()]


def r_load_with_col_ids(G, I):
    g = G(True)
    g._CAPI_LoadCSCWithColIds(I["seeds"][:8], torch.arange(9, device="cuda") * 3, I["rows"][:24])
    return [g, g._CAPI_GetCols(), int(g._CAPI_GetNumRows())]


RECIPES = {
    "_CAPI_LoadCSC": lambda G, I: base(G, I),
    "_CAPI_LoadCOO": r_load_coo,
    "_CAPI_LoadCSCWithColIds": lambda G, I: r_load_with_col_ids(G, I),
    "_CAPI_SetData": lambda G, I: base(G, I)._CAPI_GetData("default"),
    "_CAPI_GetData": lambda G, I: sliced(G, I)._CAPI_GetData("default"),
    "_CAPI_GetNumRows": lambda G, I: int(sliced(G, I)._CAPI_GetNumRows()),
    "_CAPI_GetNumCols": lambda G, I: int(sliced(G, I)._CAPI_GetNumCols()),
    "_CAPI_GetNumEdges": lambda G, I: int(sliced(G, I)._CAPI_GetNumEdges()),
    "_CAPI_Slicing": lambda G, I: [sliced(G, I), sliced(G, I)._CAPI_Slicing(I["rows"], 1, _CSC, _CSC + _COO, False),
                                   sliced(G, I)._CAPI_Slicing(I["rows"], 1, _CSR, _COO, False),
                                   base(G, I)._CAPI_Slicing(I["seeds"], 0, _CSC, _COO, True)],
    "_CAPI_BatchSlicing": lambda G, I: list(base(G, I)._CAPI_BatchSlicing(I["seeds"], batch_ptrs(I)[0], 0, _CSC,
                                                                         _CSC + _COO, False, True)),
    "_CAPI_FusionSlicing": lambda G, I: base(G, I)._CAPI_FusionSlicing(I["seeds"], I["rows"]),
    "_CAPI_BatchFusionSlicing": lambda G, I: base(G, I)._CAPI_BatchFusionSlicing(I["seeds"], batch_ptrs(I)[0], I["rows"],
                                                                                 batch_ptrs(I)[1]),
    "_CAPI_EDivUSum": lambda G, I: list(sliced(G, I, _COO)._CAPI_EDivUSum(torch.ones(I["n"], device="cuda") * 2)),
    "_CAPI_Split": lambda G, I: list(sliced(G, I)._CAPI_Split(40)),
    "_CAPI_Decode": r_decode,
    "_CAPI_Sampling": lambda G, I: [sliced(G, I)._CAPI_Sampling(0, 4, False, _CSC, _CSC + _COO),
                                    sliced(G, I)._CAPI_Sampling(0, 3, True, _CSC, _CSC)],
    "_CAPI_SamplingWithProbs": lambda G, I: (lambda s: s._CAPI_SamplingWithProbs(0, s._CAPI_GetData("default"), 5, False,
                                                                                 _CSC, _CSC + _COO))(sliced(G, I)),
    "_CAPI_FusedColumnwiseSlicingSampling": lambda G, I: [base(G, I)._CAPI_FusedColumnwiseSlicingSampling(I["seeds"], 6, False),
                                                          base(G, I)._CAPI_FusedColumnwiseSlicingSampling(I["seeds"], 1, True)],
    "_CAPI_AllValidNode": lambda G, I: sliced(G, I)._CAPI_AllValidNode(),
    "_CAPI_all_indices": lambda G, I: sliced(G, I)._CAPI_all_indices(),
    "_CAPI_GetRows": lambda G, I: sliced(G, I)._CAPI_Slicing(I["rows"], 1, _CSC, _CSC, False)._CAPI_GetRows(),
    "_CAPI_GetCols": lambda G, I: sliced(G, I)._CAPI_GetCols(),
    "_CAPI_GetValidRows": lambda G, I: sliced(G, I)._CAPI_GetValidRows(),
    "_CAPI_GetValidCols": lambda G, I: sliced(G, I)._CAPI_GetValidCols(),
    "_CAPI_GetCOORows": lambda G, I: [sliced(G, I)._CAPI_GetCOORows(True), sliced(G, I)._CAPI_GetCOORows(False)],
    "_CAPI_GetCooCols": lambda G, I: [sliced(G, I)._CAPI_GetCooCols(True), sliced(G, I)._CAPI_GetCooCols(False)],
    "_CAPI_Relabel": lambda G, I: [list(sliced(G, I)._CAPI_Relabel()), list(sliced(G, I, _COO)._CAPI_Relabel())],
    "_CAPI_Sum": lambda G, I: [sliced(G, I)._CAPI_Sum(0, 2, _CSC), sliced(G, I)._CAPI_Sum(1, 1, _COO),
                               sliced(G, I)._CAPI_Sum(1, 2, _CSR)],
    "_CAPI_Normalize": lambda G, I: [sliced(G, I)._CAPI_Normalize(0, _CSC), sliced(G, I)._CAPI_Normalize(1, _CSR)],
    "_CAPI_Divide": lambda G, I: [sliced(G, I)._CAPI_Divide(torch.ones(96, device="cuda") * 3, 0, _CSC),
                                  sliced(G, I)._CAPI_Divide(torch.ones(I["n"], device="cuda") * 3, 1, _COO)],
    "_CAPI_Metadata": lambda G, I: list(sliced(G, I)._CAPI_Metadata()),
    "_CAPI_COOMetadata": lambda G, I: list(sliced(G, I)._CAPI_COOMetadata()),
    "_CAPI_CSCMetadata": lambda G, I: list(sliced(G, I)._CAPI_CSCMetadata()),
    "_CAPI_RandomWalk": lambda G, I: base(G, I)._CAPI_RandomWalk(I["seeds"], 5),
    "_CAPI_SDDMM": r_sddmm,
    "_CAPI_GetCSC": lambda G, I: list(sliced(G, I, _COO)._CAPI_GetCSC()),
    "_CAPI_GetCOO": lambda G, I: list(sliced(G, I, _CSC)._CAPI_GetCOO()),
    "_CAPI_SetCOO": r_set_coo,
    "_CAPI_SetMetadata": r_set_coo,
}


def snake(name):
    """Registered snake_case spelling of a CamelCase name (src/pybind.cc registers one, python/gs calls the other)."""
    special = {"_CAPI_GetCooCols": "_CAPI_get_coo_cols", "_CAPI_GetCOORows": "_CAPI_get_coo_rows",
               "_CAPI_GetCSC": "_CAPI_get_csc", "_CAPI_GetCOO": "_CAPI_get_coo", "_CAPI_SetCOO": "_CAPI_set_coo",
               "_CAPI_LoadCSC": "_CAPI_load_csc", "_CAPI_LoadCOO": "_CAPI_load_coo", "_CAPI_SDDMM": "_CAPI_sddmm",
               "_CAPI_COOMetadata": "_CAPI_coo_metadata", "_CAPI_CSCMetadata": "_CAPI_csc_metadata",
               "_CAPI_LoadCSCWithColIds": "_CAPI_load_csc_with_col_ids", "_CAPI_EDivUSum": "_CAPI_e_div_u_sum",
               "_CAPI_SamplingWithProbs": "_CAPI_sampling_with_probs",
               "_CAPI_FusedColumnwiseSlicingSampling": "_CAPI_fused_columnwise_slicing_sampling"}
    if name in special:
        return special[name]
    body = name[len("_CAPI_"):]
    out = ""
    for i, ch in enumerate(body):
        out += ("_" if ch.isupper() and i else "") + ch.lower()
    return "_CAPI_" + out


def test_every_registered_method_exists_on_both_faces_and_has_a_recipe(faces):
    ts = faces["torchscript"][0](False)
    names = sorted(n for n in ts._method_names() if n.startswith("_CAPI_"))
    assert len(names) >= 2 * len(RECIPES) - 2
    py = faces["python"][0](False)
    missing = [n for n in names if not hasattr(py, n)]
    assert not missing, f"registered in lib/libgs.so but unknown to the Python face: {missing}"
    camel = [n for n in names if n in RECIPES]
    covered = set(camel) | {snake(n) for n in camel}
    uncovered = [n for n in names if n not in covered]
    assert not uncovered, f"registered names without a recipe in this test: {uncovered}"


@pytest.mark.parametrize("name", sorted(RECIPES))
def test_both_faces_return_the_same(faces, inputs, name):
    results = {}
    for face, (Graph, set_seed) in faces.items():
        set_seed(4321)
        results[face] = snapshot(RECIPES[name](Graph, inputs))
    same(results["python"], results["torchscript"], name)
    # the snake_case alias answers on both faces
    alias = snake(name)
    for face, (Graph, _) in faces.items():
        g = Graph(False)
        assert hasattr(g, alias) or alias in getattr(g, "_method_names", lambda: [])(), (face, alias)
