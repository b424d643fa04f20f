"""Tensor-level operators: the Python mirror of the reference's `gs::impl::*CUDA` functions
(src/cuda/graph_ops.h:10-75, src/cuda/tensor_ops.h:11-105, src/cuda/fusion/*.h) over torch CUDA
tensors.  Each function allocates its outputs with torch, passes raw device pointers and torch's
current stream to the C ABI, and returns tensors in the reference's tuple order.

Arguments must be contiguous CUDA tensors, int64 for ids/offsets and float32 for data; anything
else raises (the reference instantiates only those types and aborts otherwise).
"""
import ctypes

import torch

from . import cabi
from .cabi import GsbError, c_i64, c_i64p, c_int, c_u64, c_vp

_contexts = {}
_seed_state = {"base": 7777, "counter": 0, "auto_advance": True}


def set_seed(seed, auto_advance=True):
    """Base seed of the stochastic operators.  With auto_advance (default) every call that does not
    pass its own seed consumes the next value of an internal counter, so repeated calls draw
    different samples (the reference uses the constant 7777 and repeats itself:
    src/cuda/sampling.cu:138)."""
    _seed_state["base"] = int(seed)
    _seed_state["counter"] = 0
    _seed_state["auto_advance"] = bool(auto_advance)


def next_seed(seed=None):
    if seed is not None:
        return int(seed) & 0xFFFFFFFFFFFFFFFF
    s = (_seed_state["base"] * 0x9E3779B97F4A7C15 + _seed_state["counter"]) & 0xFFFFFFFFFFFFFFFF
    if _seed_state["auto_advance"]:
        _seed_state["counter"] += 1
    return s


class Context:
    """Owns one gsb_ctx (scratch arena, counters).  Calls through one Context must be ordered on
    one stream; create one Context per stream for concurrent work."""

    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("graph_sampling_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.lib = cabi.load()
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else torch.device(device).index or 0)
        h = c_vp()
        with torch.cuda.device(self.device):
            st = self.lib.gsb_ctx_create(self.device.index, ctypes.byref(h))
        if st != 0:
            raise GsbError(st, "gsb_ctx_create")
        self.handle = h

    def close(self):
        if getattr(self, "handle", None):
            self.lib.gsb_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, st, where):
        if st != 0:
            raise GsbError(st, where, self.lib.gsb_last_error_message(self.handle).decode())

    def check_device(self, where="device status"):
        self.check(self.lib.gsb_check_device_status(self.handle, _stream()), where)

    def launch_count(self):
        return int(self.lib.gsb_launch_count(self.handle))

    def read_counts(self):
        a, b = c_i64(0), c_i64(0)
        self.check(self.lib.gsb_read_counts(self.handle, _stream(), ctypes.byref(a), ctypes.byref(b)), "gsb_read_counts")
        return a.value, b.value


def default_context(device=None):
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    ctx = _contexts.get(idx)
    if ctx is None:
        ctx = Context(torch.device("cuda", idx))
        _contexts[idx] = ctx
    return ctx


def _stream():
    return c_vp(torch.cuda.current_stream().cuda_stream)


def _i64(t, name, allow_none=False):
    if t is None:
        if allow_none:
            return None
        raise TypeError(f"{name} is required")
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.int64):
        raise TypeError(f"{name} must be an int64 CUDA tensor")
    return t if t.is_contiguous() else t.contiguous()


def _f32(t, name, allow_none=False):
    if t is None:
        if allow_none:
            return None
        raise TypeError(f"{name} is required")
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32):
        raise TypeError(f"{name} must be a float32 CUDA tensor")
    return t if t.is_contiguous() else t.contiguous()


def _p(t):
    return c_vp(0) if t is None else c_vp(t.data_ptr())


def _empty(n, like, dtype=torch.int64):
    return torch.empty(int(n), dtype=dtype, device=like.device)


# ---------------------------------------------------------------------------------------------
def csc_col_slicing(indptr, indices, column_ids, with_coo=True, data=None, e_ids=None, ctx=None):
    """CSCColSlicingCUDA (src/cuda/slicing.cu:170-182) → (sub_indptr, coo_col | None, sub_indices,
    select_index[, sliced_data]).  `column_ids=None` slices every column."""
    indptr, indices = _i64(indptr, "indptr"), _i64(indices, "indices")
    column_ids = _i64(column_ids, "column_ids", allow_none=True)
    data, e_ids = _f32(data, "data", True), _i64(e_ids, "e_ids", True)
    ctx = ctx or default_context(indptr.device)
    lib = ctx.lib
    S = column_ids.numel() if column_ids is not None else indptr.numel() - 1
    sub_indptr = _empty(S + 1, indptr)
    nnz = c_i64(0)
    ctx.check(lib.gsb_col_slice_count(ctx.handle, _stream(), _p(indptr), _p(column_ids), c_i64(S), _p(sub_indptr),
                                      ctypes.byref(nnz)), "gsb_col_slice_count")
    n = nnz.value
    sub_indices, select = _empty(n, indptr), _empty(n, indptr)
    coo_col = _empty(n, indptr) if with_coo else None
    out_data = _empty(n, indptr, torch.float32) if data is not None else None
    ctx.check(lib.gsb_col_slice_fill(ctx.handle, _stream(), _p(indptr), _p(indices), _p(column_ids), c_i64(S),
                                     _p(sub_indptr), _p(sub_indices), _p(select), _p(coo_col), _p(data), _p(e_ids),
                                     _p(out_data)), "gsb_col_slice_fill")
    if data is not None:
        return sub_indptr, coo_col, sub_indices, select, out_data
    return sub_indptr, coo_col, sub_indices, select


def _sample_uniform(indptr, indices, column_ids, fanout, replace, with_coo, seed, data, e_ids, ctx):
    indptr, indices = _i64(indptr, "indptr"), _i64(indices, "indices")
    column_ids = _i64(column_ids, "column_ids", allow_none=True)
    data, e_ids = _f32(data, "data", True), _i64(e_ids, "e_ids", True)
    ctx = ctx or default_context(indptr.device)
    S = column_ids.numel() if column_ids is not None else indptr.numel() - 1
    cap = S * int(fanout)
    sub_indptr = _empty(S + 1, indptr)
    sub_indices, select = _empty(cap, indptr), _empty(cap, indptr)
    coo_col = _empty(cap, indptr) if with_coo else None
    out_data = _empty(cap, indptr, torch.float32) if data is not None else None
    nnz = c_i64(0)
    ctx.check(ctx.lib.gsb_sample_uniform(ctx.handle, _stream(), _p(indptr), _p(indices), _p(column_ids), c_i64(S),
                                         c_i64(int(fanout)), c_int(int(bool(replace))), c_u64(next_seed(seed)),
                                         _p(sub_indptr), _p(sub_indices), _p(select), _p(coo_col), _p(data), _p(e_ids),
                                         _p(out_data), c_i64(cap), ctypes.byref(nnz)), "gsb_sample_uniform")
    n = nnz.value
    out = [sub_indptr, coo_col[:n] if with_coo else None, sub_indices[:n], select[:n]]
    if data is not None:
        out.append(out_data[:n])
    return tuple(out)


def csc_col_sampling(indptr, indices, fanout, replace, with_coo=True, seed=None, data=None, e_ids=None, ctx=None):
    """CSCColSamplingCUDA (src/cuda/sampling.cu:156-167): sample every column of the operand →
    (sub_indptr, coo_col | None, sub_indices, select_index[, data])."""
    return _sample_uniform(indptr, indices, None, fanout, replace, with_coo, seed, data, e_ids, ctx)


def fused_csc_col_slicing_sampling(indptr, indices, column_ids, fanout, replace, seed=None, data=None, e_ids=None,
                                   ctx=None):
    """FusedCSCColSlicingSamplingCUDA (src/cuda/fusion/slice_sampling.cu:145-151) →
    (sub_indptr, sub_indices, select_index[, data]); select_index points into the ORIGINAL indices."""
    r = _sample_uniform(indptr, indices, column_ids, fanout, replace, False, seed, data, e_ids, ctx)
    return (r[0],) + tuple(r[2:])


def fused_csc_col_slicing_sampling_one_keepdim(indptr, indices, column_ids, seed=None, ctx=None):
    """FusedCSCColSlicingSamplingOneKeepDimCUDA (src/cuda/fusion/slice_sampling.cu:156-200)."""
    indptr, indices, column_ids = _i64(indptr, "indptr"), _i64(indices, "indices"), _i64(column_ids, "column_ids")
    ctx = ctx or default_context(indptr.device)
    S = column_ids.numel()
    sub_indptr, sub_indices, select = _empty(S + 1, indptr), _empty(S, indptr), _empty(S, indptr)
    ctx.check(ctx.lib.gsb_sample_one_keepdim(ctx.handle, _stream(), _p(indptr), _p(indices), _p(column_ids), c_i64(S),
                                             c_u64(next_seed(seed)), _p(sub_indptr), _p(sub_indices), _p(select)),
              "gsb_sample_one_keepdim")
    return sub_indptr, sub_indices, select


def _ptr_array(tensors):
    arr = (c_vp * max(1, len(tensors)))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if t.numel() > 0 else 0
    return arr


def _len_array(tensors):
    arr = (c_i64 * max(1, len(tensors)))()
    for i, t in enumerate(tensors):
        arr[i] = t.numel()
    return arr


def relabel(mapping_tensors, data_requiring_relabel, ctx=None):
    """RelabelCUDA (src/cuda/unique_reindex.cu:179-199) → (unique_tensor, [relabeled tensors]).
    unique_tensor lists the distinct ids of cat(mapping_tensors) in order of first occurrence."""
    maps = [_i64(t, "mapping tensor") for t in mapping_tensors]
    rels = [_i64(t, "tensor to relabel") for t in data_requiring_relabel]
    if not maps:
        raise ValueError("at least one mapping tensor is required")
    if len(maps) > 4 or len(rels) > 4:
        raise ValueError("at most 4 mapping tensors and 4 tensors to relabel per call")
    ctx = ctx or default_context(maps[0].device)
    n = sum(t.numel() for t in maps)
    uniq = _empty(n, maps[0])
    outs = [torch.empty_like(t) for t in rels]
    nu = c_i64(0)
    ctx.check(ctx.lib.gsb_unique_relabel(ctx.handle, _stream(), _ptr_array(maps), _len_array(maps), c_int(len(maps)),
                                         _p(uniq), _ptr_array(rels), _len_array(rels), _ptr_array(outs),
                                         c_int(len(rels)), ctypes.byref(nu)), "gsb_unique_relabel")
    return uniq[:nu.value], outs


def tensor_unique(node_ids, ctx=None):
    """TensorUniqueCUDA (src/cuda/unique_reindex.cu:174-177): distinct ids in first-occurrence order."""
    return relabel([node_ids], [], ctx)[0]


def fused_random_walk(seeds, walk_length, indices, indptr, seed=None, layout=0, walker_offset=0, ctx=None):
    """FusedRandomWalkCUDA (src/cuda/fusion/random_walk.cu:52-68).  layout=0 returns the reference's
    result exactly as it does: step-major memory viewed as [num_seeds, walk_length + 1]; layout=1
    returns a true walker-major [num_seeds, walk_length + 1] trace."""
    seeds, indptr, indices = _i64(seeds, "seeds"), _i64(indptr, "indptr"), _i64(indices, "indices")
    ctx = ctx or default_context(indptr.device)
    W, L = seeds.numel(), int(walk_length)
    out = _empty(W * (L + 1), indptr)
    ctx.check(ctx.lib.gsb_random_walk(ctx.handle, _stream(), _p(indptr), _p(indices), _p(seeds), c_i64(W), c_i64(L),
                                      c_u64(next_seed(seed)), c_int(int(layout)), c_i64(int(walker_offset)), _p(out)),
              "gsb_random_walk")
    return out.reshape(W, L + 1)
