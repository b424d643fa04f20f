"""Row gather (feature / edge-data load) from device memory and from pinned host memory read in place."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from graph_sampling_b200 import ops as m
    return m


@pytest.mark.parametrize("F", [1, 3, 4, 7, 8, 16, 20, 64, 100, 128, 256, 602])
@pytest.mark.parametrize("pinned", [False, True])
def test_gather_rows_matches_torch_index(ops, F, pinned):
    g = torch.Generator().manual_seed(F)
    src = torch.randn(5000, F, generator=g)
    idx = torch.randint(0, 5000, (12345,), generator=g)
    want = src[idx]
    s = src.pin_memory() if pinned else src.cuda()
    got = ops.gather_rows(s, idx.cuda())
    assert torch.equal(got.cpu(), want)          # a copy: bit-exact
    assert ops.gather_rows(s, idx[:0].cuda()).shape == (0, F)


def test_gather_vector_misaligned_and_errors(ops):
    from graph_sampling_b200.cabi import GsbError
    src = torch.arange(1000, dtype=torch.float32).cuda()
    idx = torch.tensor([5, 0, 999, 5], device="cuda")
    assert ops.gather_rows(src, idx).tolist() == [5.0, 0.0, 999.0, 5.0]
    base = torch.randn(4 * 64 + 1, device="cuda")
    mis = base[1:].view(4, 64)                     # 4-byte aligned rows of 256 bytes: takes the scalar path
    assert torch.equal(ops.gather_rows(mis, torch.tensor([3, 1], device="cuda")), mis[[3, 1]])
    with pytest.raises(TypeError):
        ops.gather_rows(torch.randn(4, 4), idx)    # pageable host memory is refused before any launch
    ctx = ops.default_context()
    pageable = torch.randn(16, 4)
    out = torch.empty(2, 4, device="cuda")
    st = ctx.lib.gsb_gather_rows(ctx.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                 ctypes.c_void_p(pageable.data_ptr()), ctypes.c_int64(16), ctypes.c_int64(4),
                                 ctypes.c_void_p(idx.data_ptr()), ctypes.c_int64(2), ctypes.c_void_p(out.data_ptr()))
    assert st == -1
    # an index out of range is skipped and reported, not dereferenced
    guard = torch.full((3, 8), -1.0, device="cuda")
    zeros = torch.zeros(10, 8, device="cuda")
    bad = torch.tensor([1, 77, -3], device="cuda")
    ctx.lib.gsb_gather_rows(ctx.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                            ctypes.c_void_p(zeros.data_ptr()), ctypes.c_int64(10), ctypes.c_int64(8),
                            ctypes.c_void_p(bad.data_ptr()), ctypes.c_int64(3), ctypes.c_void_p(guard.data_ptr()))
    with pytest.raises(GsbError) as e:
        ctx.check_device()
    assert e.value.status == -8
    assert torch.all(guard[0] == 0) and torch.all(guard[1:] == -1)
    ctx.check_device()
