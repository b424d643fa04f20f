"""Error behaviour of the C ABI on the GPU: bad input is reported through status codes / exceptions, the
process survives (the reference LOG(FATAL)s), the context stays usable afterwards, and nothing here makes
a kernel fault — every case is caught by a bounds or capacity check that skips the access."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def ops():
    from graph_sampling_b200 import ops as _ops
    return _ops


def test_output_capacity_too_small_is_reported_not_overrun(ops):
    from graph_sampling_b200.cabi import GsbError
    ctx = ops.default_context()
    indptr = dev(np.arange(101, dtype=np.int64) * 8)
    indices = dev(np.arange(800, dtype=np.int64))
    S, k = 100, 4
    out_indptr = torch.empty(S + 1, dtype=torch.int64, device="cuda")
    guard = torch.full((64 + 16,), -5, dtype=torch.int64, device="cuda")  # only 64 of the 400 needed entries
    nnz = ctypes.c_int64(0)
    st = ctx.lib.gsb_sample_uniform(ctx.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                    ctypes.c_void_p(indptr.data_ptr()), ctypes.c_void_p(indices.data_ptr()),
                                    ctypes.c_void_p(0), ctypes.c_int64(S), ctypes.c_int64(k), ctypes.c_int(0),
                                    ctypes.c_uint64(1), ctypes.c_void_p(out_indptr.data_ptr()),
                                    ctypes.c_void_p(guard.data_ptr()), ctypes.c_void_p(guard.data_ptr()),
                                    ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
                                    ctypes.c_int64(64), ctypes.byref(nnz))
    assert st == -4  # GSB_ERR_CAPACITY
    assert nnz.value == 400            # the exact requirement is still reported
    assert torch.all(guard[64:] == -5)  # nothing was written past the stated capacity
    # the context is usable again and the error flag is cleared
    ctx.check_device()
    r = ops.csc_col_sampling(indptr, indices, k, False, with_coo=False, seed=1)
    assert r[2].numel() == 400
    with pytest.raises(GsbError):
        ctx.check(-4, "synthetic")


def test_negative_ids_in_unique_are_rejected(ops):
    from graph_sampling_b200.cabi import GsbError
    items = dev(np.array([3, 5, -2, 7], dtype=np.int64))
    with pytest.raises(GsbError) as e:
        ops.tensor_unique(items)
    assert e.value.status == -8  # GSB_ERR_INDEX_RANGE
    # next call works
    assert ops.tensor_unique(dev(np.array([3, 5, 3], dtype=np.int64))).cpu().tolist() == [3, 5]


def test_batched_relabel_rejects_ids_beyond_32_bits(ops):
    from graph_sampling_b200.cabi import GsbError
    seeds = dev(np.array([1, 2], dtype=np.int64))
    ptr = dev(np.array([0, 2], dtype=np.int64))
    indices = dev(np.array([1 << 40, 2], dtype=np.int64))
    iptr = dev(np.array([0, 2], dtype=np.int64))
    with pytest.raises(GsbError) as e:
        ops.batch_csr_relabel(seeds, ptr, indices, iptr)
    assert e.value.status == -8


def test_wrong_dtype_and_device_raise_type_errors(ops):
    indptr = dev(np.arange(5, dtype=np.int64))
    indices = dev(np.arange(4, dtype=np.int64))
    with pytest.raises(TypeError):
        ops.csc_col_slicing(indptr.int(), indices, dev(np.array([0])))
    with pytest.raises(TypeError):
        ops.csc_col_slicing(indptr.cpu(), indices, dev(np.array([0])))
    with pytest.raises(TypeError):
        ops.csc_col_sampling_probs(indptr, indices, indices, 2, False)  # probs must be float32


def test_invalid_arguments_return_status_not_abort(ops):
    ctx = ops.default_context()
    st = ctx.lib.gsb_col_slice_count(ctx.handle, ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
                                     ctypes.c_int64(-1), ctypes.c_void_p(0), ctypes.c_void_p(0))
    assert st == -1
    st = ctx.lib.gsb_random_walk(ctx.handle, ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
                                 ctypes.c_void_p(0), ctypes.c_int64(4), ctypes.c_int64(2), ctypes.c_uint64(0),
                                 ctypes.c_int(7), ctypes.c_int64(0), ctypes.c_void_p(0))
    assert st == -1


def test_graph_methods_raise_where_the_reference_aborts():
    import graph_sampling_b200.gs as gs
    g = gs.Graph(False)
    g._CAPI_load_csc(torch.arange(5).cuda(), torch.arange(4).cuda())
    with pytest.raises(RuntimeError):
        g._CAPI_slicing(torch.arange(2).cuda(), 0, gs._CSC, gs._CSR, False)  # CSC -> CSR output: not implemented
    with pytest.raises(RuntimeError):
        g._CAPI_all_valid_node()  # col_ids missing
    with pytest.raises(RuntimeError, match="Require DCSC, get CSC instead"):
        g._CAPI_slicing(torch.arange(2).cuda(), 0, gs._DCSC, gs._CSC, False)  # holds a plain CSC (src/graph.cc:609-613)
