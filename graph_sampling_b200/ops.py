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

    OPTIONS = {"max_polls": 0, "table_slots": 1, "relabel_path": 2, "direct_table_budget": 3, "blocking_wait": 4}

    def set_option(self, name, value):
        """gsb_ctx_set_option by name: max_polls, table_slots, relabel_path (0 auto, 1 hash regions, 2 direct-address tables, 3 partitioned),
        direct_table_budget (bytes), blocking_wait (0 / 1)."""
        self.check(self.lib.gsb_ctx_set_option(self.handle, c_int(self.OPTIONS[name]), c_i64(int(value))),
                   "gsb_ctx_set_option")

    def get_option(self, name):
        v = c_i64(0)
        self.check(self.lib.gsb_ctx_get_option(self.handle, c_int(self.OPTIONS[name]), ctypes.byref(v)),
                   "gsb_ctx_get_option")
        return v.value

    def launch_count(self):
        return int(self.lib.gsb_launch_count(self.handle))

    # ---- per-kernel timing (gsb_profile_*) ----
    def profile_enable(self, on=True):
        self.check(self.lib.gsb_profile_enable(self.handle, c_int(int(bool(on)))), "gsb_profile_enable")

    def profile_reset(self):
        self.check(self.lib.gsb_profile_reset(self.handle), "gsb_profile_reset")

    def profile_read(self):
        """{kernel class name: (total device ms, launches)} for classes with at least one timed launch."""
        self.lib.gsb_profile_kernel_name.restype = ctypes.c_char_p
        out = {}
        for kid in range(int(self.lib.gsb_profile_num_kernels())):
            ms, n = ctypes.c_double(0), c_i64(0)
            self.check(self.lib.gsb_profile_read(self.handle, c_int(kid), ctypes.byref(ms), ctypes.byref(n)),
                       "gsb_profile_read")
            if n.value:
                out[self.lib.gsb_profile_kernel_name(kid).decode()] = (ms.value, n.value)
        return out

    def read_counts(self):
        a, b = c_i64(0), c_i64(0)
        self.check(self.lib.gsb_read_counts(self.handle, _stream(), ctypes.byref(a), ctypes.byref(b)), "gsb_read_counts")
        return a.value, b.value


def default_context(device=None):
    if device is not None and torch.device(device).type != "cuda":       # a pinned host tensor's device
        device = None
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    ctx = _contexts.get(idx)
    if ctx is None:
        ctx = Context(torch.device("cuda", idx))
        _contexts[idx] = ctx
    return ctx


def _stream():
    return c_vp(torch.cuda.current_stream().cuda_stream)


def _resident(t):
    """Memory a kernel can read in place: device memory, or pinned host memory through the unified address
    space (the reference accepts pinned graph arrays the same way: src/graph_ops.cc:144,226)."""
    return t.is_cuda or t.is_pinned()


def _contiguous(t, name):
    if not t.is_cuda:
        raise TypeError(f"{name}: a pinned host tensor must be contiguous")
    return t.contiguous()


def cuda_device_of(t):
    """Where results derived from `t` are allocated: its own device, or the current one for pinned host memory."""
    return t.device if t.is_cuda else torch.device("cuda", torch.cuda.current_device())


def _i64(t, name, allow_none=False):
    if t is None:
        if allow_none:
            return None
        raise TypeError(f"{name} is required")
    if not (isinstance(t, torch.Tensor) and _resident(t) and t.dtype == torch.int64):
        raise TypeError(f"{name} must be an int64 CUDA (or pinned host) tensor")
    return t if t.is_contiguous() else _contiguous(t, name)


def _f32(t, name, allow_none=False):
    if t is None:
        if allow_none:
            return None
        raise TypeError(f"{name} is required")
    if not (isinstance(t, torch.Tensor) and _resident(t) and t.dtype == torch.float32):
        raise TypeError(f"{name} must be a float32 CUDA (or pinned host) tensor")
    return t if t.is_contiguous() else _contiguous(t, name)


def _p(t):
    return c_vp(0) if t is None else c_vp(t.data_ptr())


def _empty(n, like, dtype=torch.int64):
    return torch.empty(int(n), dtype=dtype, device=cuda_device_of(like))


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
    num_cols = indptr.numel() - 1
    ctx.check(lib.gsb_col_slice_count(ctx.handle, _stream(), _p(indptr), c_i64(num_cols), _p(column_ids), c_i64(S),
                                      _p(sub_indptr), ctypes.byref(nnz)), "gsb_col_slice_count")
    n = nnz.value
    sub_indices, select = _empty(n, indptr), _empty(n, indptr)
    coo_col = _empty(n, indptr) if with_coo else None
    out_data = _empty(n, indptr, torch.float32) if data is not None else None
    ctx.check(lib.gsb_col_slice_fill(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(num_cols), _p(column_ids),
                                     c_i64(S), _p(sub_indptr), c_i64(n), _p(sub_indices), _p(select), _p(coo_col),
                                     _p(data), _p(e_ids), _p(out_data)), "gsb_col_slice_fill")
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
    ctx.check(ctx.lib.gsb_sample_uniform(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(indptr.numel() - 1),
                                         _p(column_ids), c_i64(S),
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
    ctx.check(ctx.lib.gsb_sample_one_keepdim(ctx.handle, _stream(), _p(indptr), _p(indices),
                                             c_i64(indptr.numel() - 1), _p(column_ids), c_i64(S),
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
    ctx.check(ctx.lib.gsb_random_walk(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(indptr.numel() - 1),
                                      _p(seeds), c_i64(W), c_i64(L),
                                      c_u64(next_seed(seed)), c_int(int(layout)), c_i64(int(walker_offset)), _p(out)),
              "gsb_random_walk")
    return out.reshape(W, L + 1)


def fused_metapath_random_walk(seeds, metapath, graphs, seed=None, layout=0, walker_offset=0, ctx=None):
    """FusedMetapathRandomWalkCUDA (src/cuda/fusion/metapath_random_walk.cu:52-67): `graphs` is a list of
    (indptr, indices) CSC pairs, `metapath` the relation index of every step.  Layouts as in fused_random_walk."""
    seeds = _i64(seeds, "seeds")
    pairs = [(_i64(a, "indptr"), _i64(b, "indices")) for a, b in graphs]
    path = [int(r) for r in metapath]
    ctx = ctx or default_context(seeds.device)
    W, L = seeds.numel(), len(path)
    out = _empty(W * (L + 1), seeds)
    ip = (c_vp * max(1, len(pairs)))(*[a.data_ptr() for a, _ in pairs])
    ix = (c_vp * max(1, len(pairs)))(*[b.data_ptr() for _, b in pairs])
    mp = (c_i64 * max(1, L))(*path)
    nn = (c_i64 * max(1, len(pairs)))(*[a.numel() - 1 for a, _ in pairs])
    ctx.check(ctx.lib.gsb_metapath_random_walk(ctx.handle, _stream(), ip, ix, nn, c_int(len(pairs)), mp, c_i64(L),
                                               _p(seeds), c_i64(W), c_u64(next_seed(seed)), c_int(int(layout)),
                                               c_i64(int(walker_offset)), _p(out)), "gsb_metapath_random_walk")
    return out.reshape(W, L + 1)


def csc_col_row_slicing(indptr, indices, column_ids, row_ids, col_ptr=None, row_ptr=None, encoding_size=0,
                        data=None, e_ids=None, ctx=None):
    """CSCColRowSlicingCUDA / BatchCSCColRowSlicingCUDA (src/cuda/fusion/column_row_slicing.cu:101-365) →
    (sub_indptr, sub_indices, select_index[, sliced_data]).  Without col_ptr / row_ptr the kept row ids are
    renumbered to their position in row_ids; with them (the super-batch form) a column of batch b is matched
    against batch b's rows and row ids stay as they are.  select_index points into `indices`."""
    indptr, indices = _i64(indptr, "indptr"), _i64(indices, "indices")
    column_ids, row_ids = _i64(column_ids, "column_ids"), _i64(row_ids, "row_ids")
    col_ptr, row_ptr = _i64(col_ptr, "col_ptr", True), _i64(row_ptr, "row_ptr", True)
    data, e_ids = _f32(data, "data", True), _i64(e_ids, "e_ids", True)
    if (col_ptr is None) != (row_ptr is None):
        raise ValueError("col_ptr and row_ptr go together")
    ctx = ctx or default_context(indptr.device)
    S, R = column_ids.numel(), row_ids.numel()
    G = 1 if col_ptr is None else col_ptr.numel() - 1
    slice_indptr = _empty(S + 1, indptr)
    d = c_i64(0)
    num_cols = indptr.numel() - 1
    ctx.check(ctx.lib.gsb_col_slice_count(ctx.handle, _stream(), _p(indptr), c_i64(num_cols), _p(column_ids), c_i64(S),
                                          _p(slice_indptr), ctypes.byref(d)), "gsb_col_slice_count")
    D = d.value
    sub_indptr = _empty(S + 1, indptr)
    sub_indices, select = _empty(D, indptr), _empty(D, indptr)
    out_data = _empty(D, indptr, torch.float32) if data is not None else None
    nnz = c_i64(0)
    ctx.check(ctx.lib.gsb_col_row_slice(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(num_cols),
                                        _p(column_ids), c_i64(S),
                                        _p(slice_indptr), c_i64(D), _p(row_ids), c_i64(R), _p(col_ptr), _p(row_ptr),
                                        c_i64(G), c_i64(int(encoding_size)), c_int(1 if col_ptr is None else 0),
                                        _p(sub_indptr), _p(sub_indices), _p(select), _p(data), _p(e_ids),
                                        _p(out_data), ctypes.byref(nnz)), "gsb_col_row_slice")
    n = nnz.value
    sub_indices, select = sub_indices[:n], select[:n]
    if out_data is not None:
        out_data = out_data[:n]
    if data is not None:
        return sub_indptr, sub_indices, select, out_data
    return sub_indptr, sub_indices, select


def gather_rows(src, index, ctx=None):
    """out[i] = src[index[i]] for a float32 matrix (or vector) `src` that lives on the GPU or in pinned host memory
    (read in place by the GPU, like IndexSelectCPUFromGPU, src/cuda/index_select_uvm.cu:8-45)."""
    index = _i64(index, "index")
    if not (isinstance(src, torch.Tensor) and src.dtype == torch.float32 and src.is_contiguous()):
        raise TypeError("src must be a contiguous float32 tensor")
    if not (src.is_cuda or src.is_pinned()):
        raise TypeError("src must live on the GPU or in pinned host memory")
    ctx = ctx or default_context(index.device)
    num_rows = src.shape[0] if src.dim() > 0 else 0
    row_len = 1
    for d in src.shape[1:]:
        row_len *= int(d)
    out = torch.empty((index.numel(),) + tuple(src.shape[1:]), dtype=torch.float32, device=index.device)
    if row_len == 0:
        return out
    ctx.check(ctx.lib.gsb_gather_rows(ctx.handle, _stream(), c_vp(src.data_ptr()), c_i64(num_rows), c_i64(row_len),
                                      _p(index), c_i64(index.numel()), _p(out)), "gsb_gather_rows")
    return out


index_select_cpu_from_gpu = gather_rows


def take(src, index):
    """src[index] for a per-edge array (float32 edge data, int64 edge ids) that lives on the GPU or in pinned host
    memory, where the GPU reads it in place (src/graph.cc:296-306 does the same through IndexSelectCPUFromGPU)."""
    if src.is_cuda:
        return src[index]
    if src.dtype == torch.int64:                         # copied as rows of two 32-bit words
        return gather_rows(src.view(torch.float32).view(-1, 2), index).view(torch.int64).view(-1)
    return gather_rows(src, index)


def index_search(origin_data, keys, ctx=None):
    """gs::IndexSearch (src/tensor_ops.cc:23-31): position of every key in origin_data, -1 if absent."""
    origin_data, keys = _i64(origin_data, "origin_data"), _i64(keys, "keys")
    ctx = ctx or default_context(keys.device)
    out = torch.empty_like(keys)
    ctx.check(ctx.lib.gsb_index_search(ctx.handle, _stream(), _p(origin_data), c_i64(origin_data.numel()), _p(keys),
                                       c_i64(keys.numel()), _p(out)), "gsb_index_search")
    return out


def coo_e_div_u_sum(coo_row, coo_col, data, divisor, num_cols, ctx=None):
    """COOEDivUSum (src/cuda/fusion/edge_map_reduce.cu:10-24) → (out_data, out_sum): edge data divided by the
    divisor of the edge's row node, and the per-column sums of the result."""
    coo_row, coo_col = _i64(coo_row, "coo_row"), _i64(coo_col, "coo_col")
    data, divisor = _f32(data, "data", True), _f32(divisor, "divisor")
    ctx = ctx or default_context(coo_row.device)
    E = coo_row.numel()
    out = _empty(E, coo_row, torch.float32)
    out_sum = torch.zeros(int(num_cols), dtype=torch.float32, device=coo_row.device)
    ctx.check(ctx.lib.gsb_edge_div_u_sum(ctx.handle, _stream(), _p(coo_row), _p(coo_col), c_i64(E), _p(data),
                                         _p(divisor), _p(out), _p(out_sum)), "gsb_edge_div_u_sum")
    return out, out_sum


# ---------------------------------------------------------------------------------------------
def csc_col_sampling_probs(indptr, indices, probs, fanout, replace, with_coo=True, seed=None, column_ids=None,
                           data=None, e_ids=None, ctx=None):
    """CSCColSamplingProbsCUDA (src/cuda/sampling_probs.cu:267-282) → (sub_indptr, coo_col | None,
    sub_indices, select_index[, data]).  `probs[j]` pairs with `indices[j]`.  `column_ids` (not in the
    reference) fuses a column slice in front."""
    indptr, indices, probs = _i64(indptr, "indptr"), _i64(indices, "indices"), _f32(probs, "probs")
    column_ids = _i64(column_ids, "column_ids", allow_none=True)
    data, e_ids = _f32(data, "data", True), _i64(e_ids, "e_ids", True)
    if probs.numel() != indices.numel():
        raise ValueError("probs must have one entry per edge of the operand")
    ctx = ctx or default_context(indptr.device)
    S = column_ids.numel() if column_ids is not None else indptr.numel() - 1
    cap = S * int(fanout)
    sub_indptr = _empty(S + 1, indptr)
    sub_indices, select = _empty(cap, indptr), _empty(cap, indptr)
    coo_col = _empty(cap, indptr) if with_coo else None
    out_data = _empty(cap, indptr, torch.float32) if data is not None else None
    nnz = c_i64(0)
    ctx.check(ctx.lib.gsb_sample_weighted(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(indptr.numel() - 1),
                                          _p(probs), _p(column_ids),
                                          c_i64(S), c_i64(int(fanout)), c_int(int(bool(replace))),
                                          c_u64(next_seed(seed)), _p(sub_indptr), _p(sub_indices), _p(select),
                                          _p(coo_col), _p(data), _p(e_ids), _p(out_data), c_i64(cap),
                                          ctypes.byref(nnz)), "gsb_sample_weighted")
    n = nnz.value
    out = [sub_indptr, coo_col[:n] if with_coo else None, sub_indices[:n], select[:n]]
    if data is not None:
        out.append(out_data[:n])
    return tuple(out)


def list_sampling(data, num_picks, replace, probs=None, seed=None, ctx=None):
    """ListSamplingCUDA (src/cuda/list_sampling.cu:76-83) / ListSamplingProbsCUDA
    (src/cuda/list_sampling_probs.cu:185-191) → (selected_data, selected_index)."""
    data = _i64(data, "data")
    probs = _f32(probs, "probs", allow_none=True)
    if probs is not None and probs.numel() != data.numel():
        raise ValueError("probs must have one entry per item")
    ctx = ctx or default_context(data.device)
    N, k = data.numel(), int(num_picks)
    cap = max(N if (not replace and N <= k) else k, 1)
    out_d, out_i = _empty(cap, data), _empty(cap, data)
    n_out = c_i64(0)
    ctx.check(ctx.lib.gsb_list_sample(ctx.handle, _stream(), _p(data), _p(probs), c_i64(N), c_i64(k),
                                      c_int(int(bool(replace))), c_u64(next_seed(seed)), _p(out_d), _p(out_i),
                                      ctypes.byref(n_out)), "gsb_list_sample")
    return out_d[:n_out.value], out_i[:n_out.value]


SDDMM_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "copy_lhs": 4, "copy_rhs": 5, "dot": 6}


def calc_bcast_off(op, lhs, rhs):
    """CalcBcastOff (src/bcast.cc:24-76) on tensor shapes → dict(lhs_len, rhs_len, out_len, reduce_size,
    lhs_off, rhs_off); the offset lists are None when no broadcasting is needed."""
    ls, rs = list(lhs.shape), list(rhs.shape)
    lhs_len = 1
    for d in ls[1:]:
        lhs_len *= d
    rhs_len = 1
    for d in rs[1:]:
        rhs_len *= d
    use_bcast = False
    if op not in ("copy_lhs", "copy_rhs"):
        use_bcast = len(ls) != len(rs) or any(ls[i] != rs[i] for i in range(1, len(ls)))
    reduce_size, lhs_off, rhs_off = 1, None, None
    if use_bcast:
        max_ndim = max(len(ls), len(rs)) - 1
        out_len, j = 1, 0
        if op == "dot":
            reduce_size = ls[-1]
            j = 1
        stride_l = stride_r = 1
        lhs_off, rhs_off = [0], [0]
        while j < max_ndim:
            dl = 1 if len(ls) - 1 - j < 1 else ls[len(ls) - 1 - j]
            dr = 1 if len(rs) - 1 - j < 1 else rs[len(rs) - 1 - j]
            for i in range(1, max(dl, dr)):
                for q in range(out_len):
                    lhs_off.append(lhs_off[q] + i * (1 if i < dl else 0) * stride_l)
                    rhs_off.append(rhs_off[q] + i * (1 if i < dr else 0) * stride_r)
            out_len *= max(dl, dr)
            stride_l *= dl
            stride_r *= dr
            j += 1
    else:
        out_len = rhs_len if op == "copy_rhs" else lhs_len
        if op == "dot":
            reduce_size = ls[-1]
            out_len //= reduce_size
    return dict(lhs_len=lhs_len, rhs_len=rhs_len, out_len=out_len, reduce_size=reduce_size, lhs_off=lhs_off,
                rhs_off=rhs_off)


def sddmm(op, lhs, rhs, out, lhs_target, rhs_target, row, col=None, indptr=None, e_ids=None, ctx=None):
    """SDDMMCOO (col given) / SDDMMCSC (col=None, indptr given) (src/cuda/sddmm.cu:255-291): writes
    op(lhs[target], rhs[target]) per edge into the caller's `out` ([E, out_len], fp32)."""
    if op not in SDDMM_OPS:
        raise ValueError(f"unknown SDDMM op {op!r}")
    row = _i64(row, "row")
    col, indptr, e_ids = _i64(col, "col", True), _i64(indptr, "indptr", True), _i64(e_ids, "e_ids", True)
    lhs, rhs = _f32(lhs, "lhs", op == "copy_rhs"), _f32(rhs, "rhs", op == "copy_lhs")
    if not (isinstance(out, torch.Tensor) and out.is_cuda and out.dtype == torch.float32 and out.is_contiguous()):
        raise TypeError("out must be a contiguous float32 CUDA tensor")
    ctx = ctx or default_context(row.device)
    bc = calc_bcast_off(op, lhs if lhs is not None else rhs, rhs if rhs is not None else lhs)
    E = row.numel()
    if out.numel() != E * bc["out_len"]:
        raise ValueError(f"out has {out.numel()} elements, expected {E} x {bc['out_len']}")
    lo = torch.tensor(bc["lhs_off"], dtype=torch.int64, device=row.device) if bc["lhs_off"] is not None else None
    ro = torch.tensor(bc["rhs_off"], dtype=torch.int64, device=row.device) if bc["rhs_off"] is not None else None
    num_cols = indptr.numel() - 1 if indptr is not None else 0
    ctx.check(ctx.lib.gsb_sddmm(ctx.handle, _stream(), c_int(SDDMM_OPS[op]), _p(row), _p(col), _p(indptr),
                                c_i64(num_cols), _p(e_ids), c_i64(E), _p(lhs), _p(rhs), _p(out), c_int(int(lhs_target)),
                                c_int(int(rhs_target)), c_i64(bc["lhs_len"]), c_i64(bc["rhs_len"]), c_i64(bc["out_len"]),
                                c_i64(bc["reduce_size"]), _p(lo), _p(ro)), "gsb_sddmm")
    return out


def csc_sum(indptr, e_ids, data, out, powk, ctx=None):
    """CSCSumCUDA (src/cuda/graph_ops.cu:66-96): out[s] = sum over segment s of data^powk (data=None → ones)."""
    indptr, e_ids, data = _i64(indptr, "indptr"), _i64(e_ids, "e_ids", True), _f32(data, "data", True)
    ctx = ctx or default_context(indptr.device)
    ctx.check(ctx.lib.gsb_segment_sum_csc(ctx.handle, _stream(), _p(indptr), c_i64(indptr.numel() - 1), _p(e_ids),
                                          _p(data), c_i64(int(powk)), _p(out)), "gsb_segment_sum_csc")
    return out


def coo_sum(target, e_ids, data, out, powk, ctx=None, targets_in_runs=False):
    """COOSumCUDA (src/cuda/graph_ops.cu:98-125): out[target[e]] += data[e]^powk; `out` must be zeroed.
    targets_in_runs: equal targets are adjacent (the sorted coordinate of a COO) — a hint, not a requirement."""
    target, e_ids, data = _i64(target, "target"), _i64(e_ids, "e_ids", True), _f32(data, "data", True)
    ctx = ctx or default_context(target.device)
    ctx.check(ctx.lib.gsb_segment_sum_coo(ctx.handle, _stream(), _p(target), c_i64(target.numel()), _p(e_ids),
                                          _p(data), c_i64(int(powk)), c_int(int(bool(targets_in_runs))), _p(out)),
              "gsb_segment_sum_coo")
    return out


def csc_normalize(indptr, e_ids, data, out, ctx=None):
    """CSCNormalizeCUDA (src/cuda/graph_ops.cu:160-188): out[e] = data[e] / (sum of its segment)."""
    indptr, e_ids, data = _i64(indptr, "indptr"), _i64(e_ids, "e_ids", True), _f32(data, "data")
    ctx = ctx or default_context(indptr.device)
    ctx.check(ctx.lib.gsb_segment_normalize_csc(ctx.handle, _stream(), _p(indptr), c_i64(indptr.numel() - 1),
                                                _p(e_ids), _p(data), _p(out)), "gsb_segment_normalize_csc")
    return out


def csc_row_slicing(indptr, indices, row_ids, with_coo=True, ctx=None):
    """CSCRowSlicingCUDA (src/cuda/slicing.cu:528-539) → (out_indptr, coo_col | None, out_indices,
    select_index); kept row ids are renumbered to their position in row_ids."""
    indptr, indices, row_ids = _i64(indptr, "indptr"), _i64(indices, "indices"), _i64(row_ids, "row_ids")
    ctx = ctx or default_context(indptr.device)
    nc, E = indptr.numel() - 1, indices.numel()
    out_indptr = _empty(nc + 1, indptr)
    oi, osel = _empty(E, indptr), _empty(E, indptr)
    oc = _empty(E, indptr) if with_coo else None
    nnz = c_i64(0)
    ctx.check(ctx.lib.gsb_row_slice_csc(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(nc), c_i64(E),
                                        _p(row_ids), c_i64(row_ids.numel()), _p(out_indptr), _p(oi), _p(osel), _p(oc),
                                        ctypes.byref(nnz)), "gsb_row_slice_csc")
    n = nnz.value
    return out_indptr, (oc[:n] if with_coo else None), oi[:n], osel[:n]


def coo_row_slicing(coo_row, coo_col, row_ids, ctx=None):
    """COORowSlicingCUDA (src/cuda/slicing.cu:768-771) → (renumbered_row, col, select_index)."""
    coo_row, coo_col, row_ids = _i64(coo_row, "coo_row"), _i64(coo_col, "coo_col"), _i64(row_ids, "row_ids")
    ctx = ctx or default_context(coo_row.device)
    E = coo_row.numel()
    o_r, o_c, o_s = _empty(E, coo_row), _empty(E, coo_row), _empty(E, coo_row)
    nnz = c_i64(0)
    ctx.check(ctx.lib.gsb_row_slice_coo(ctx.handle, _stream(), _p(coo_row), _p(coo_col), c_i64(E), _p(row_ids),
                                        c_i64(row_ids.numel()), _p(o_r), _p(o_c), _p(o_s), ctypes.byref(nnz)),
              "gsb_row_slice_coo")
    n = nnz.value
    return o_r[:n], o_c[:n], o_s[:n]


def csc2coo(indptr, indices, ctx=None):
    """CSC2COOCUDA (src/cuda/format_transform.cu:35-46) → (row = indices, col)."""
    indptr, indices = _i64(indptr, "indptr"), _i64(indices, "indices")
    ctx = ctx or default_context(indptr.device)
    col = _empty(indices.numel(), indptr)
    ctx.check(ctx.lib.gsb_csc2coo(ctx.handle, _stream(), _p(indptr), c_i64(indptr.numel() - 1), _p(col)),
              "gsb_csc2coo")
    return indices, col


def coo2csc(row, col, num_cols, col_sorted, ctx=None):
    """COO2CSCCUDA (src/cuda/format_transform.cu:135-156) → (indptr, sorted_row, sort_index | None).
    For CSR pass (col, row, num_rows, row_sorted)."""
    row, col = _i64(row, "row"), _i64(col, "col")
    ctx = ctx or default_context(row.device)
    E = row.numel()
    indptr = _empty(int(num_cols) + 1, row)
    out_row = _empty(E, row)
    perm = None if col_sorted else _empty(E, row)
    ctx.check(ctx.lib.gsb_coo2csc(ctx.handle, _stream(), _p(col), _p(row), c_i64(E), c_i64(int(num_cols)),
                                  c_int(int(bool(col_sorted))), _p(indptr), _p(out_row), _p(perm)), "gsb_coo2csc")
    return indptr, out_row, perm


# ---- batched ("super-batch") operators --------------------------------------------------------------
def batch_csr_relabel(seeds, seeds_ptr, indices, indices_ptr, indices_count=None, ctx=None, sync=True, num_nodes=0,
                      seeds_distinct=False):
    """BatchCSRRelabelCUDA (src/cuda/batch_relabel.cu, gs_ops._CAPI_BatchCSRRelabel) →
    (unique_tensor, unique_tensor_ptr, relabeled_indices, indices_ptr): per batch b, the distinct ids of
    cat(seeds[seeds_ptr[b]:seeds_ptr[b+1]], indices[indices_ptr[b]:indices_ptr[b+1]]) in first-occurrence
    order and the batch-local positions of its indices.  `indices` may be longer than the valid edge
    count (indices_ptr[-1]); with sync=False the outputs keep their upper-bound length and the exact
    sizes stay on the device.  num_nodes > 0 (every id is below it) allows the direct-address tables;
    seeds_distinct promises that no id repeats among the seeds of a batch."""
    seeds, seeds_ptr = _i64(seeds, "seeds"), _i64(seeds_ptr, "seeds_ptr")
    indices, indices_ptr = _i64(indices, "indices"), _i64(indices_ptr, "indices_ptr")
    ctx = ctx or default_context(seeds.device)
    G = seeds_ptr.numel() - 1
    cap = indices.numel() if indices_count is None else int(indices_count)
    uniq = _empty(seeds.numel() + cap, seeds)
    uniq_ptr = _empty(G + 1, seeds)
    rel = _empty(cap, seeds)
    nu, ne = c_i64(0), c_i64(0)
    ctx.check(ctx.lib.gsb_batch_unique_relabel(ctx.handle, _stream(), _p(seeds), _p(seeds_ptr), c_i64(seeds.numel()),
                                               _p(indices), _p(indices_ptr), c_i64(cap), c_i64(G),
                                               c_i64(int(num_nodes)), c_int(1 if seeds_distinct else 0), _p(uniq),
                                               _p(uniq_ptr), _p(rel), ctypes.byref(nu) if sync else None,
                                               ctypes.byref(ne) if sync else None), "gsb_batch_unique_relabel")
    if sync:
        return uniq[:nu.value], uniq_ptr, rel[:ne.value], indices_ptr
    return uniq, uniq_ptr, rel, indices_ptr


def batch_edge_offsets(sub_indptr, seeds_ptr, ctx=None):
    """indices_ptr[b] = sub_indptr[seeds_ptr[b]] (what GetBatchCSC derives, examples/graphsage/batching.py:66)."""
    sub_indptr, seeds_ptr = _i64(sub_indptr, "sub_indptr"), _i64(seeds_ptr, "seeds_ptr")
    ctx = ctx or default_context(sub_indptr.device)
    out = _empty(seeds_ptr.numel(), seeds_ptr)
    ctx.check(ctx.lib.gsb_batch_edge_offsets(ctx.handle, _stream(), _p(sub_indptr), _p(seeds_ptr),
                                             c_i64(seeds_ptr.numel() - 1), _p(out)), "gsb_batch_edge_offsets")
    return out


# ---- the rest of the super-batch family (gs_ops registry, src/pybind.cc:65-84) ------------------
def batch_encode(data, data_ptr, encoding_size, ctx=None):
    """BatchEncodeCUDA (src/cuda/batch_coding.cu:64-85): data[i] + batch(i) * encoding_size."""
    data, data_ptr = _i64(data, "data"), _i64(data_ptr, "data_ptr")
    ctx = ctx or default_context(data.device)
    out = torch.empty_like(data)
    ctx.check(ctx.lib.gsb_batch_encode(ctx.handle, _stream(), _p(data), _p(data_ptr), c_i64(data_ptr.numel() - 1),
                                       c_i64(data.numel()), c_i64(int(encoding_size)), _p(out)), "gsb_batch_encode")
    return out


def batch_decode(data, encoding_size, ctx=None):
    """BatchDecodeCUDA (src/cuda/batch_coding.cu:87-98): data[i] mod encoding_size."""
    data = _i64(data, "data")
    ctx = ctx or default_context(data.device)
    out = torch.empty_like(data)
    ctx.check(ctx.lib.gsb_batch_decode(ctx.handle, _stream(), _p(data), c_i64(data.numel()),
                                       c_i64(int(encoding_size)), _p(out)), "gsb_batch_decode")
    return out


def get_batch_offsets(data, num_batches, encoding_size, ctx=None):
    """GetBatchOffsets (src/cuda/batch_coding.cu:100-121) → (data_ptr[num_batches + 1], decoded ids)."""
    data = _i64(data, "data")
    ctx = ctx or default_context(data.device)
    ptr = _empty(int(num_batches) + 1, data)
    dec = torch.empty_like(data)
    ctx.check(ctx.lib.gsb_get_batch_offsets(ctx.handle, _stream(), _p(data), c_i64(data.numel()),
                                            c_i64(int(num_batches)), c_i64(int(encoding_size)), _p(ptr), _p(dec)),
              "gsb_get_batch_offsets")
    return ptr, dec


def batch_csc_col_slicing(indptr, indices, column_ids, nid_ptr, encoding_size, with_coo=True, encoding=False,
                          data=None, e_ids=None, ctx=None):
    """BatchCSCColSlicingCUDA (src/cuda/slicing.cu:275-295) → (sub_indptr, coo_col | None, sub_indices,
    select_index, coo_offsets[, sliced_data]).  With `encoding` the row ids of batch b carry b * encoding_size."""
    indptr, indices = _i64(indptr, "indptr"), _i64(indices, "indices")
    column_ids, nid_ptr = _i64(column_ids, "column_ids"), _i64(nid_ptr, "nid_ptr")
    data, e_ids = _f32(data, "data", True), _i64(e_ids, "e_ids", True)
    ctx = ctx or default_context(indptr.device)
    S, G = column_ids.numel(), nid_ptr.numel() - 1
    sub_indptr = _empty(S + 1, indptr)
    nnz = c_i64(0)
    num_cols = indptr.numel() - 1
    ctx.check(ctx.lib.gsb_col_slice_count(ctx.handle, _stream(), _p(indptr), c_i64(num_cols), _p(column_ids), c_i64(S),
                                          _p(sub_indptr), ctypes.byref(nnz)), "gsb_col_slice_count")
    n = nnz.value
    sub_indices, select = _empty(n, indptr), _empty(n, indptr)
    coo_col = _empty(n, indptr) if with_coo else None
    offsets = _empty(G + 1, indptr)
    out_data = _empty(n, indptr, torch.float32) if data is not None else None
    ctx.check(ctx.lib.gsb_batch_col_slice_fill(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(num_cols),
                                               _p(column_ids), c_i64(S),
                                               _p(nid_ptr), c_i64(G), c_i64(int(encoding_size) if encoding else 0),
                                               _p(sub_indptr), _p(sub_indices), _p(select), _p(coo_col), _p(offsets),
                                               _p(data), _p(e_ids), _p(out_data)), "gsb_batch_col_slice_fill")
    if data is not None:
        return sub_indptr, coo_col, sub_indices, select, offsets, out_data
    return sub_indptr, coo_col, sub_indices, select, offsets


def batch_unique(data, data_ptr, sort=False, ctx=None):
    """BatchUniqueCUDA (first-occurrence order) / BatchUnique2CUDA (sort=True: ascending per batch)
    (src/cuda/batch_unique.cu:131-278) → (unique, unique_ptr, unique_key)."""
    data, data_ptr = _i64(data, "data"), _i64(data_ptr, "data_ptr")
    ctx = ctx or default_context(data.device)
    n, G = data.numel(), data_ptr.numel() - 1
    uniq, key, ptr = _empty(n, data), _empty(n, data), _empty(G + 1, data)
    nu = c_i64(0)
    ctx.check(ctx.lib.gsb_batch_unique(ctx.handle, _stream(), _p(data), _p(data_ptr), c_i64(n), c_i64(G),
                                       c_int(1 if sort else 0), _p(uniq), _p(ptr), _p(key), ctypes.byref(nu)),
              "gsb_batch_unique")
    return uniq[:nu.value], ptr, key[:nu.value]


def batch_coo_relabel(seeds, seeds_ptr, coo_col, coo_row, coo_ptr, ctx=None):
    """BatchCOORelabelCUDA (src/cuda/batch_relabel.cu:349-497) →
    (unique_tensor, unique_tensor_ptr, relabeled_row, relabeled_col, coo_ptr)."""
    seeds, seeds_ptr = _i64(seeds, "seeds"), _i64(seeds_ptr, "seeds_ptr")
    coo_col, coo_row, coo_ptr = _i64(coo_col, "coo_col"), _i64(coo_row, "coo_row"), _i64(coo_ptr, "coo_ptr")
    if coo_col.numel() != coo_row.numel():
        raise ValueError("coo_col and coo_row must have the same length")
    ctx = ctx or default_context(seeds.device)
    G, E = seeds_ptr.numel() - 1, coo_row.numel()
    uniq, ptr = _empty(seeds.numel() + E, seeds), _empty(G + 1, seeds)
    out_row, out_col = _empty(E, seeds), _empty(E, seeds)
    nu = c_i64(0)
    ctx.check(ctx.lib.gsb_batch_coo_relabel(ctx.handle, _stream(), _p(seeds), _p(seeds_ptr), c_i64(seeds.numel()),
                                            _p(coo_col), _p(coo_row), _p(coo_ptr), c_i64(E), c_i64(G), _p(uniq),
                                            _p(ptr), _p(out_row), _p(out_col), ctypes.byref(nu)),
              "gsb_batch_coo_relabel")
    return uniq[:nu.value], ptr, out_row, out_col, coo_ptr


def batch_coo_slicing(axis, coo_row, coo_col, batch_ptr, neighbors, neighbors_ptr, ctx=None):
    """BatchCOOSlicingCUDA (src/cuda/batch_slicing.cu:166-263) → (sub_coo_row, sub_coo_col, sub_ptr): per batch
    the edges whose column (axis 0) / row (axis 1) id is among the batch's neighbours; ids unchanged."""
    coo_row, coo_col = _i64(coo_row, "coo_row"), _i64(coo_col, "coo_col")
    batch_ptr = _i64(batch_ptr, "batch_ptr", True)
    neighbors, neighbors_ptr = _i64(neighbors, "neighbors"), _i64(neighbors_ptr, "neighbors_ptr", True)
    ctx = ctx or default_context(coo_row.device)
    G = 1 if batch_ptr is None else batch_ptr.numel() - 1
    E = coo_row.numel()
    out_row, out_col, out_ptr = _empty(E, coo_row), _empty(E, coo_row), _empty(G + 1, coo_row)
    n = c_i64(0)
    ctx.check(ctx.lib.gsb_batch_coo_slice(ctx.handle, _stream(), c_int(int(axis)), _p(coo_row), _p(coo_col),
                                          _p(batch_ptr), c_i64(E), _p(neighbors), _p(neighbors_ptr),
                                          c_i64(neighbors.numel()), c_i64(G), _p(out_row), _p(out_col), _p(out_ptr),
                                          ctypes.byref(n)), "gsb_batch_coo_slice")
    return out_row[:n.value], out_col[:n.value], out_ptr


def coo_row_slicing_global_id(coo_row, coo_col, row_ids, ctx=None):
    """COORowSlicingGlobalIdCUDA (src/cuda/batch_slicing.cu:265-317) → (coo_row, coo_col) of the edges whose
    row id is in row_ids; ids unchanged."""
    r, c, _ = batch_coo_slicing(1, coo_row, coo_col, None, row_ids, None, ctx=ctx)
    return r, c


def batch_concat(data_tensors, offset_tensors, ctx=None):
    """BatchConcatCUDA (src/cuda/batch_concat.cu:50-121) → (data, key, data_ptr): batch b of the result is
    batch b of every input in turn."""
    datas = [_i64(t, "data tensor") for t in data_tensors]
    offs = [_i64(t, "offset tensor") for t in offset_tensors]
    if not datas or len(datas) != len(offs) or len(datas) > 8:
        raise ValueError("between 1 and 8 (data, offsets) pairs are required")
    ctx = ctx or default_context(datas[0].device)
    G = offs[0].numel() - 1
    total = sum(t.numel() for t in datas)
    out, key, ptr = _empty(total, datas[0]), _empty(total, datas[0]), _empty(G + 1, datas[0])
    ctx.check(ctx.lib.gsb_batch_concat(ctx.handle, _stream(), _ptr_array(datas), _ptr_array(offs), _len_array(datas),
                                       c_int(len(datas)), c_i64(G), _p(out), _p(key), _p(ptr)), "gsb_batch_concat")
    return out, key, ptr


def batch_split(data, data_ptr, data_key, out_tensors, out_ptr_tensors, ctx=None):
    """BatchSplit2CUDA (src/cuda/batch_split2.cu:40-106): the inverse of batch_concat; fills the caller's
    out_tensors (partitioned by out_ptr_tensors) and returns (out_tensors, out_ptr_tensors).  data_key is
    accepted for signature compatibility; the batch of an item is derived from data_ptr."""
    data, data_ptr = _i64(data, "data"), _i64(data_ptr, "data_ptr")
    outs = [_i64(t, "output tensor") for t in out_tensors]
    optrs = [_i64(t, "output offsets") for t in out_ptr_tensors]
    if not outs or len(outs) != len(optrs) or len(outs) > 8:
        raise ValueError("between 1 and 8 (output, offsets) pairs are required")
    ctx = ctx or default_context(data.device)
    ctx.check(ctx.lib.gsb_batch_split(ctx.handle, _stream(), _p(data), _p(data_ptr), c_i64(data.numel()),
                                      c_i64(data_ptr.numel() - 1), _ptr_array(outs), _ptr_array(optrs),
                                      c_int(len(outs))), "gsb_batch_split")
    return outs, optrs


def batch_list_sampling_probs(probs, num_picks, replace, range_ptr, seed=None, ctx=None):
    """BatchListSamplingProbsCUDA (src/cuda/list_sampling_probs.cu:110-183) → (out_idx, out_range): weighted
    sampling without replacement of min(num_picks, size) positions from every segment of `probs`."""
    if replace:
        raise NotImplementedError("segmented list sampling with replacement (the reference aborts as well)")
    probs, range_ptr = _f32(probs, "probs"), _i64(range_ptr, "range")
    ctx = ctx or default_context(probs.device)
    N, G = probs.numel(), range_ptr.numel() - 1
    out = _empty(min(N, G * int(num_picks)), range_ptr)
    out_range = _empty(G + 1, range_ptr)
    n = c_i64(0)
    ctx.check(ctx.lib.gsb_batch_list_sample(ctx.handle, _stream(), _p(probs), c_i64(N), _p(range_ptr), c_i64(G),
                                            c_i64(int(num_picks)), c_u64(next_seed(seed)), _p(out), _p(out_range),
                                            ctypes.byref(n)), "gsb_batch_list_sample")
    return out[:n.value], out_range


def split_by_offset(data, offsets):
    """gs::SplitByOffset (src/tensor_ops.cc:33-45): views of `data` cut at `offsets` (one host read of the sizes)."""
    sizes = (offsets[1:] - offsets[:-1]).tolist()
    return list(torch.split(data, sizes))


def indptr_split_by_offset(indptr, offsets, ctx=None):
    """SplitIndptrByOffsetCUDA (src/cuda/batch_split.cu:66-97): per-batch offset arrays, each rebased to 0."""
    indptr, offsets = _i64(indptr, "indptr"), _i64(offsets, "offsets")
    ctx = ctx or default_context(indptr.device)
    G = offsets.numel() - 1
    host = offsets.tolist()
    out = _empty(host[-1] - host[0] + G, indptr)
    if host[0] != 0:
        raise ValueError("offsets must start at 0")
    ctx.check(ctx.lib.gsb_split_indptr(ctx.handle, _stream(), _p(indptr), _p(offsets), c_i64(G), c_i64(0), _p(out)),
              "gsb_split_indptr")
    return list(torch.split(out, [host[b + 1] - host[b] + 1 for b in range(G)]))


def indptr_split_by_size(indptr, size, ctx=None):
    """SplitIndptrBySizeCUDA (src/cuda/batch_split.cu:11-48): batches of `size` columns each."""
    indptr = _i64(indptr, "indptr")
    ctx = ctx or default_context(indptr.device)
    G = (indptr.numel() - 1) // int(size)
    out = _empty(G * (int(size) + 1), indptr)
    ctx.check(ctx.lib.gsb_split_indptr(ctx.handle, _stream(), _p(indptr), _p(None), c_i64(G), c_i64(int(size)),
                                       _p(out)), "gsb_split_indptr")
    return list(torch.split(out, int(size) + 1))


class OutputArena:
    """Reusable output buffers for a loop that calls the same operator again and again (a sampler feeding a
    trainer): the first calls allocate, with 25 % headroom, and later calls of similar size allocate nothing, so
    the loop never waits for cudaMalloc — which serialises across the processes of a multi-GPU job.
    Results handed out from an arena are overwritten by the next call that uses it."""

    def __init__(self):
        self._buffers = {}

    def get(self, key, n, like, dtype=torch.int64):
        n = int(n)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n or buf.device != cuda_device_of(like) or buf.dtype != dtype:
            buf = torch.empty(max(16, n + n // 4), dtype=dtype, device=cuda_device_of(like))
            self._buffers[key] = buf
        return buf[:n]

    def bytes(self):
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


def sage_sample_batches(indptr, indices, seeds, seeds_ptr, fanouts, replace=False, seed=None, ctx=None, sync=True,
                        arena=None, batch_ids=None, seeds_distinct=False, size_hints=None):
    """Multi-hop GraphSAGE sampling of G minibatches at once (the loop of
    examples/graphsage/batching.py:56-90): per hop one fused slice+sample over the seeds of all batches,
    then one batched unique + relabel; each batch's frontier becomes its seeds for the next hop.

    Returns a list (one entry per hop) of dicts with: seeds, seeds_ptr (columns of the hop and their
    per-batch offsets), sub_indptr (offsets over all columns), indices (global ids), relabeled
    (batch-local ids), select_index, indices_ptr, frontier, frontier_ptr.

    sync=True waits once per hop and trims every array to its exact length.  sync=False queues all hops
    without waiting for the GPU: arrays keep their upper-bound length (S·k edges, S·(1+k) frontier entries
    per hop, so capacities grow by (1+k) per hop), the valid prefixes are given by the offset arrays, and
    every dict carries `counts`, a 3-element device tensor (seeds, edges, frontier) to read when convenient.

    arena: an OutputArena to take the output arrays from (they are then valid until the next call with it).

    batch_ids: int64 device tensor with one caller-chosen number (< 2^32) per minibatch, e.g. its index in the
    epoch.  With it the draws of a minibatch are keyed by (seed, its number, column index inside the minibatch),
    so the minibatch receives the same sample whichever call, group size or GPU processes it; without it the key
    is the column's position in the call.
    seeds_distinct: promise that no id repeats among the seeds of one minibatch (the frontiers that feed hops
    2, 3, ... are distinct by construction and are always treated so).

    size_hints (with sync=False): one (seed_bound, edge_bound) pair per hop — sizes the caller knows from earlier
    calls of the same shape, e.g. the sizes of the previous epoch plus a margin — used instead of the worst-case
    bounds S·(1+k), which overshoot the real sizes several times over and cost grid, clear and scratch work in
    proportion.  The first hop's seed bound is ignored (its seed count is exact).  If a hop meets more seeds or edges
    than hinted, the device records GSB_ERR_CAPACITY (ctx.check_device() raises it) and the caller repeats the call
    without hints; nothing is written out of bounds."""
    ctx = ctx or default_context(indptr.device)
    out = []
    base_seed = next_seed(seed)
    batch_ids = _i64(batch_ids, "batch_ids", allow_none=True)
    if batch_ids is not None and batch_ids.numel() != seeds_ptr.numel() - 1:
        raise ValueError("batch_ids needs one entry per minibatch")
    num_nodes = indptr.numel() - 1

    def alloc(name, hop, n):
        return _empty(n, indptr) if arena is None else arena.get((name, hop), n, indptr)

    if size_hints is not None and (sync or len(size_hints) != len(fanouts)):
        raise ValueError("size_hints needs sync=False and one (seed_bound, edge_bound) pair per hop")
    for hop, k in enumerate(fanouts):
        S = seeds.numel()
        G = seeds_ptr.numel() - 1
        cap = S * int(k)
        if size_hints is not None:
            if hop > 0:
                S = min(S, int(size_hints[hop][0]))
                seeds = seeds[:S]
            cap = min(S * int(k), int(size_hints[hop][1]))
        sub_indptr = alloc("sub_indptr", hop, S + 1)
        sub_indices, select, rel = alloc("indices", hop, cap), alloc("select", hop, cap), alloc("relabeled", hop, cap)
        indices_ptr, uniq_ptr = alloc("indices_ptr", hop, G + 1), alloc("frontier_ptr", hop, G + 1)
        uniq = alloc("frontier", hop, S + cap)
        nu, ne = c_i64(0), c_i64(0)
        flags = 1 if (hop > 0 or seeds_distinct) else 0
        ctx.check(ctx.lib.gsb_sage_hop(ctx.handle, _stream(), _p(indptr), _p(indices), c_i64(num_nodes), _p(seeds),
                                       _p(seeds_ptr), _p(batch_ids), c_i64(G), c_i64(S), c_i64(int(k)), c_i64(cap),
                                       c_int(int(bool(replace))), c_u64((base_seed + hop) & (2**64 - 1)),
                                       c_int(flags), _p(sub_indptr), _p(sub_indices),
                                       _p(select), _p(indices_ptr), _p(uniq), _p(uniq_ptr), _p(rel),
                                       ctypes.byref(nu) if sync else None, ctypes.byref(ne) if sync else None),
                  "gsb_sage_hop")
        if sync:
            E, U = ne.value, nu.value
            out.append(dict(seeds=seeds, seeds_ptr=seeds_ptr, sub_indptr=sub_indptr, indices=sub_indices[:E],
                            relabeled=rel[:E], select_index=select[:E], indices_ptr=indices_ptr, frontier=uniq[:U],
                            frontier_ptr=uniq_ptr))
            seeds, seeds_ptr = uniq[:U], uniq_ptr
        else:
            counts = torch.cat([seeds_ptr[G:], indices_ptr[G:], uniq_ptr[G:]])
            out.append(dict(seeds=seeds, seeds_ptr=seeds_ptr, sub_indptr=sub_indptr, indices=sub_indices,
                            relabeled=rel, select_index=select, indices_ptr=indices_ptr, frontier=uniq,
                            frontier_ptr=uniq_ptr, counts=counts))
            seeds, seeds_ptr = uniq, uniq_ptr
    return out
