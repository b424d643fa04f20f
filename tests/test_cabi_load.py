"""CPU-side checks of the C-ABI library: it is built, loads, and exports every symbol the public
header declares (no kernel is launched here)."""
import ctypes
import os

import pytest

from graph_sampling_b200 import build as gsb_build
from graph_sampling_b200 import cabi


@pytest.fixture(scope="module")
def lib():
    gsb_build.build()
    return cabi.load()


def test_header_declares_entry_points():
    syms = cabi.declared_symbols()
    for must in ["gsb_ctx_create", "gsb_col_slice_count", "gsb_col_slice_fill", "gsb_sample_uniform",
                 "gsb_unique_relabel", "gsb_random_walk"]:
        assert must in syms


def test_library_exports_every_declared_symbol(lib):
    for s in cabi.declared_symbols():
        assert hasattr(lib, s), s


def test_every_entry_point_is_bound_with_its_declared_arity(lib):
    """The ctypes binding takes its argument lists from the header, so a caller with a stale argument list gets a
    TypeError instead of a corrupted stack (no kernel is launched: the calls below fail in ctypes)."""
    protos = cabi.declared_prototypes()
    assert set(protos) == set(cabi.declared_symbols())
    for name, (restype, argtypes) in protos.items():
        fn = getattr(lib, name)
        assert fn.argtypes is not None and len(fn.argtypes) == len(argtypes), name
    assert len(protos["gsb_sage_hop"][1]) == 24 and len(protos["gsb_col_slice_count"][1]) == 8
    assert len(protos["gsb_random_walk"][1]) == 12 and len(protos["gsb_ctx_set_option"][1]) == 3
    with pytest.raises((TypeError, ctypes.ArgumentError)):
        lib.gsb_col_slice_count(None, None)
    # options and the self-test are refused without a context (no device needed)
    assert lib.gsb_ctx_set_option(None, 0, 5) == -1
    assert lib.gsb_selftest_lookback(None, None, 4, -1, None) == -1


def test_status_strings_and_version(lib):
    assert cabi.status_string(0) == "ok"
    assert "capacity" in cabi.status_string(-4)
    assert "sm_100a" in cabi.version()


def test_no_torch_dependency_in_kernel_library():
    # the boundary is plain C: the kernel library must not link against torch / c10
    out = os.popen(f"ldd {cabi.LIB_PATH}").read()
    names = [line.split()[0] for line in out.splitlines() if line.strip()]   # library names only, not load addresses
    assert not [n for n in names if "torch" in n or "c10" in n], names


def test_ctx_create_fails_cleanly_without_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    h = ctypes.c_void_p()
    st = lib.gsb_ctx_create(0, ctypes.byref(h))
    assert st != 0 and not h.value


def test_package_has_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from graph_sampling_b200 import ops
    with pytest.raises(RuntimeError):
        ops.Context()


def test_torchscript_glue_registers_reference_names():
    """lib/libgs.so loads in torch and registers gs_classes.Graph / gs_ops with the reference's method names
    (src/pybind.cc) in both spellings; without a GPU a call fails with an exception, not an abort."""
    import torch
    torch.classes.load_library(gsb_build.build_glue())
    g = torch.classes.gs_classes.Graph(False)
    for name in ["_CAPI_LoadCSC", "_CAPI_load_csc", "_CAPI_Slicing", "_CAPI_slicing", "_CAPI_Sampling",
                 "_CAPI_SamplingWithProbs", "_CAPI_FusedColumnwiseSlicingSampling",
                 "_CAPI_fused_columnwise_slicing_sampling", "_CAPI_AllValidNode", "_CAPI_all_indices", "_CAPI_Relabel",
                 "_CAPI_relabel", "_CAPI_RandomWalk", "_CAPI_SDDMM", "_CAPI_Sum", "_CAPI_Normalize", "_CAPI_Divide",
                 "_CAPI_Metadata", "_CAPI_GetCooCols", "_CAPI_GetCSC", "_CAPI_GetCOO", "_CAPI_BatchSlicing",
                 "_CAPI_FusionSlicing", "_CAPI_BatchFusionSlicing", "_CAPI_EDivUSum", "_CAPI_Split", "_CAPI_Decode"]:
        assert hasattr(g, name), name
    for op in ["_CAPI_ListSampling", "_CAPI_ListSamplingWithProbs", "_CAPI_Unique", "list_sampling",
               "list_sampling_with_probs", "_CAPI_BatchCSRRelabel", "_CAPI_BatchListSamplingWithProbs", "_CAPI_IndexSearch",
               "_CAPI_SplitByOffset", "_CAPI_IndptrSplitBySize", "_CAPI_IndptrSplitByOffset", "_CAPI_BatchConcat",
               "_CAPI_BatchUnique", "_CAPI_BatchUniqueByKey", "_CAPI_BatchUnique2", "_CAPI_BatchUniqueByKey2",
               "_CAPI_BatchCSRRelabelByKey", "_CAPI_BatchCOORelabelByKey", "_CAPI_BatchCOORelabel", "_CAPI_BatchSplit",
               "_CAPI_BatchCOOSlicing", "_CAPI_BatchEncode", "_CAPI_BatchDecode", "_CAPI_GetBatchOffsets",
               "_CAPI_COORowSlicingGlobalId"]:   # every name of the reference's gs_ops registry (src/pybind.cc:62-85)
        assert hasattr(torch.ops.gs_ops, op), op
    hg = torch.classes.gs_classes.HeteroGraph()
    for name in ["_CAPI_LoadFromHomo", "_CAPI_GetHomoGraph", "_CAPI_MetapathRandomWalkFused"]:
        assert hasattr(hg, name), name
    if not torch.cuda.is_available():
        with pytest.raises(Exception):
            g._CAPI_LoadCSC(torch.arange(3), torch.arange(2))
