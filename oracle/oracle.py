"""numpy front-end of the CPU oracle (TEST INFRASTRUCTURE — only tests/, the smoke check and the
CPU-baseline leg of bench.py may import this module; the shipped package never does).

Every function mirrors one reference operator and returns numpy arrays in the reference's tuple
order: slicing / sampling → (sub_indptr, coo_col | None, sub_indices, select_index)
(src/cuda/slicing.cu:167, src/cuda/sampling.cu:153); fused slice+sample → (sub_indptr,
sub_indices, select_index) (src/cuda/fusion/slice_sampling.cu:142).
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

I64 = np.int64
F32 = np.float32

OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "copy_lhs": 4, "copy_rhs": 5, "dot": 6}


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libgs_oracle.so")
        if not os.path.exists(path):
            from . import build as _b  # type: ignore
            _b.build()
        _LIB = ctypes.CDLL(path)
        _LIB.gso_col_slice_count.restype = ctypes.c_int64
        _LIB.gso_sample_uniform_count.restype = ctypes.c_int64
        _LIB.gso_list_sample.restype = ctypes.c_int64
        _LIB.gso_unique_relabel.restype = ctypes.c_int64
        _LIB.gso_row_slice_csc.restype = ctypes.c_int64
        _LIB.gso_row_slice_coo.restype = ctypes.c_int64
        _LIB.gso_sage_batch.restype = ctypes.c_int64
        _LIB.gso_rand_word.restype = ctypes.c_uint32
        _LIB.gso_ares_key_of.restype = ctypes.c_float
        _LIB.gso_num_threads.restype = ctypes.c_int
    return _LIB


def _p(a):
    if a is None:
        return ctypes.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def _i64(a):
    return None if a is None else np.ascontiguousarray(a, dtype=I64)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=F32)


def _c(v):
    return ctypes.c_int64(int(v))


def _u(v):
    return ctypes.c_uint64(int(v) & 0xFFFFFFFFFFFFFFFF)


def num_threads():
    return int(lib().gso_num_threads())


def set_num_threads(n):
    lib().gso_set_num_threads(ctypes.c_int(int(n)))


def philox_block(ctr, key):
    c = np.asarray(ctr, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    out = np.zeros(4, dtype=np.uint32)
    lib().gso_philox_block(_p(c), _p(k), _p(out))
    return out


def rand_word(seed, item, slot, stream):
    return int(lib().gso_rand_word(_u(seed), _u(item), _u(slot), ctypes.c_uint32(stream)))


def ares_key(r, w):
    return float(lib().gso_ares_key_of(ctypes.c_uint32(r), ctypes.c_float(w)))


def col_slice(indptr, indices, seeds, with_coo=True):
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    S = len(seeds) if seeds is not None else len(indptr) - 1
    sub_indptr = np.empty(S + 1, dtype=I64)
    nnz = lib().gso_col_slice_count(_p(indptr), _p(seeds), _c(S), _p(sub_indptr))
    out_i = np.empty(nnz, dtype=I64)
    out_s = np.empty(nnz, dtype=I64)
    out_c = np.empty(nnz, dtype=I64) if with_coo else None
    lib().gso_col_slice_fill(_p(indptr), _p(indices), _p(seeds), _c(S), _p(sub_indptr), _p(out_i), _p(out_s),
                             _p(out_c))
    return sub_indptr, out_c, out_i, out_s


def sample_uniform(indptr, indices, seeds, k, replace, seed=0, algo=0, with_coo=False, item_base=0):
    """seeds=None → plain Sampling over every column; else fused slice+sample.  item_base: see
    gso_sample_uniform_fill (minibatch number << 32 for the minibatch-keyed stream)."""
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    S = len(seeds) if seeds is not None else len(indptr) - 1
    sub_indptr = np.empty(S + 1, dtype=I64)
    nnz = lib().gso_sample_uniform_count(_p(indptr), _p(seeds), _c(S), _c(k), ctypes.c_int(int(replace)),
                                         _p(sub_indptr))
    out_i = np.empty(nnz, dtype=I64)
    out_s = np.empty(nnz, dtype=I64)
    out_c = np.empty(nnz, dtype=I64) if with_coo else None
    lib().gso_sample_uniform_fill(_p(indptr), _p(indices), _p(seeds), _c(S), _c(k), ctypes.c_int(int(replace)),
                                  _u(seed), ctypes.c_int(algo), _p(sub_indptr), _p(out_i), _p(out_s), _p(out_c),
                                  _u(item_base))
    return sub_indptr, out_c, out_i, out_s


def sample_one_keepdim(indptr, indices, seeds, seed=0):
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    S = len(seeds)
    sub_indptr = np.empty(S + 1, dtype=I64)
    out_i = np.empty(S, dtype=I64)
    out_s = np.empty(S, dtype=I64)
    lib().gso_sample_one_keepdim(_p(indptr), _p(indices), _p(seeds), _c(S), _u(seed), _p(sub_indptr), _p(out_i),
                                 _p(out_s))
    return sub_indptr, out_i, out_s


def sample_weighted(indptr, indices, probs, seeds, k, replace, seed=0, with_coo=False):
    indptr, indices, seeds, probs = _i64(indptr), _i64(indices), _i64(seeds), _f32(probs)
    S = len(seeds) if seeds is not None else len(indptr) - 1
    sub_indptr = np.empty(S + 1, dtype=I64)
    nnz = lib().gso_sample_uniform_count(_p(indptr), _p(seeds), _c(S), _c(k), ctypes.c_int(int(replace)),
                                         _p(sub_indptr))
    out_i = np.empty(nnz, dtype=I64)
    out_s = np.empty(nnz, dtype=I64)
    out_c = np.empty(nnz, dtype=I64) if with_coo else None
    lib().gso_sample_weighted_fill(_p(indptr), _p(indices), _p(probs), _p(seeds), _c(S), _c(k),
                                   ctypes.c_int(int(replace)), _u(seed), _p(sub_indptr), _p(out_i), _p(out_s),
                                   _p(out_c))
    return sub_indptr, out_c, out_i, out_s


def list_sample(data, probs, k, replace, seed=0):
    data, probs = _i64(data), _f32(probs)
    N = len(data)
    cap = max(N, k)
    out_d = np.empty(cap, dtype=I64)
    out_x = np.empty(cap, dtype=I64)
    n = lib().gso_list_sample(_p(data), _p(probs), _c(N), _c(k), ctypes.c_int(int(replace)), _u(seed), _p(out_d),
                              _p(out_x))
    return out_d[:n].copy(), out_x[:n].copy()


def unique_relabel(mapping, to_relabel=None):
    """mapping: list of arrays (concatenated in order) → (frontier, [relabeled arrays])."""
    items = _i64(np.concatenate([np.asarray(m, dtype=I64) for m in mapping])) if len(mapping) else np.empty(0, I64)
    N = len(items)
    uniq = np.empty(N, dtype=I64)
    if to_relabel is None:
        U = lib().gso_unique_relabel(_p(items), _c(N), _p(uniq), _p(None), _c(0), _p(None))
        return uniq[:U].copy(), []
    sizes = [len(t) for t in to_relabel]
    rel_in = _i64(np.concatenate([np.asarray(t, dtype=I64) for t in to_relabel])) if sizes else np.empty(0, I64)
    rel_out = np.empty(len(rel_in), dtype=I64)
    U = lib().gso_unique_relabel(_p(items), _c(N), _p(uniq), _p(rel_in), _c(len(rel_in)), _p(rel_out))
    outs, o = [], 0
    for s in sizes:
        outs.append(rel_out[o:o + s].copy())
        o += s
    return uniq[:U].copy(), outs


def random_walk(indptr, indices, seeds, length, seed=0, layout=0, walker_offset=0):
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    W = len(seeds)
    out = np.empty(W * (length + 1), dtype=I64)
    lib().gso_random_walk(_p(indptr), _p(indices), _p(seeds), _c(W), _c(length), _u(seed), ctypes.c_int(layout),
                          _c(walker_offset), _p(out))
    # the reference returns the step-major memory reshaped to [W, L+1] without a transpose
    return out.reshape(W, length + 1)


def calc_bcast(op, lhs_shape, rhs_shape):
    """Restates CalcBcastOff (src/bcast.cc:24-76) on shapes. Returns dict with lhs_len, rhs_len,
    out_len, reduce_size, lhs_off, rhs_off (None when no broadcasting)."""
    lhs_len = int(np.prod(lhs_shape[1:])) if len(lhs_shape) > 1 else 1
    rhs_len = int(np.prod(rhs_shape[1:])) if len(rhs_shape) > 1 else 1
    use_bcast = False
    if op not in ("copy_lhs", "copy_rhs"):
        if len(lhs_shape) != len(rhs_shape):
            use_bcast = True
        else:
            use_bcast = any(lhs_shape[i] != rhs_shape[i] for i in range(1, len(lhs_shape)))
    reduce_size = 1
    lhs_off = rhs_off = None
    if use_bcast:
        max_ndim = max(len(lhs_shape), len(rhs_shape)) - 1
        out_len, j = 1, 0
        if op == "dot":
            reduce_size = lhs_shape[-1]
            j = 1
        stride_l = stride_r = 1
        lhs_off, rhs_off = [0], [0]
        while j < max_ndim:
            dl = 1 if len(lhs_shape) - 1 - j < 1 else lhs_shape[len(lhs_shape) - 1 - j]
            dr = 1 if len(rhs_shape) - 1 - j < 1 else rhs_shape[len(rhs_shape) - 1 - j]
            for i in range(1, max(dl, dr)):
                for k in range(out_len):
                    lhs_off.append(lhs_off[k] + i * (1 if i < dl else 0) * stride_l)
                    rhs_off.append(rhs_off[k] + i * (1 if i < dr else 0) * stride_r)
            out_len *= max(dl, dr)
            stride_l *= dl
            stride_r *= dr
            j += 1
    else:
        out_len = rhs_len if op == "copy_rhs" else lhs_len
        if op == "dot":
            reduce_size = lhs_shape[-1]
            out_len //= reduce_size
    return dict(lhs_len=lhs_len, rhs_len=rhs_len, out_len=out_len, reduce_size=reduce_size, lhs_off=lhs_off,
                rhs_off=rhs_off)


def sddmm_coo(op, row, col, lhs, rhs, lhs_target=0, rhs_target=2, e_ids=None):
    row, col, e_ids = _i64(row), _i64(col), _i64(e_ids)
    lhs, rhs = _f32(lhs), _f32(rhs)
    E = len(row)
    bc = calc_bcast(op, lhs.shape if lhs is not None else rhs.shape, rhs.shape if rhs is not None else lhs.shape)
    out = np.zeros((E, bc["out_len"]), dtype=F32)
    lo = _i64(np.asarray(bc["lhs_off"])) if bc["lhs_off"] is not None else None
    ro = _i64(np.asarray(bc["rhs_off"])) if bc["rhs_off"] is not None else None
    lib().gso_sddmm_coo(ctypes.c_int(OPS[op]), _p(row), _p(col), _p(e_ids), _c(E), _p(lhs), _p(rhs), _p(out),
                        ctypes.c_int(lhs_target), ctypes.c_int(rhs_target), _c(bc["lhs_len"]), _c(bc["rhs_len"]),
                        _c(bc["out_len"]), _c(bc["reduce_size"]), _p(lo), _p(ro))
    return out


def segment_sum_csc(indptr, data, powk=1, e_ids=None):
    indptr, data, e_ids = _i64(indptr), _f32(data), _i64(e_ids)
    n = len(indptr) - 1
    out = np.zeros(n, dtype=F32)
    lib().gso_segment_sum_csc(_p(indptr), _c(n), _p(e_ids), _p(data), _c(powk), _p(out))
    return out


def segment_sum_coo(target, num_out, data, powk=1, e_ids=None):
    target, data, e_ids = _i64(target), _f32(data), _i64(e_ids)
    out = np.zeros(num_out, dtype=F32)
    lib().gso_segment_sum_coo(_p(target), _c(len(target)), _p(e_ids), _p(data), _c(powk), _p(out))
    return out


def segment_normalize_csc(indptr, data, e_ids=None):
    indptr, data, e_ids = _i64(indptr), _f32(data), _i64(e_ids)
    out = np.empty_like(data)
    lib().gso_segment_normalize_csc(_p(indptr), _c(len(indptr) - 1), _p(e_ids), _p(data), _p(out))
    return out


def row_slice_csc(indptr, indices, row_ids, with_coo=False):
    indptr, indices, row_ids = _i64(indptr), _i64(indices), _i64(row_ids)
    nc = len(indptr) - 1
    out_indptr = np.empty(nc + 1, dtype=I64)
    oi = np.empty(len(indices), dtype=I64)
    os_ = np.empty(len(indices), dtype=I64)
    oc = np.empty(len(indices), dtype=I64) if with_coo else None
    n = lib().gso_row_slice_csc(_p(indptr), _p(indices), _c(nc), _p(row_ids), _c(len(row_ids)), _p(out_indptr),
                                _p(oi), _p(os_), _p(oc))
    return out_indptr, (oc[:n].copy() if with_coo else None), oi[:n].copy(), os_[:n].copy()


def row_slice_coo(coo_row, coo_col, row_ids):
    coo_row, coo_col, row_ids = _i64(coo_row), _i64(coo_col), _i64(row_ids)
    E = len(coo_row)
    o_r, o_c, o_s = (np.empty(E, dtype=I64) for _ in range(3))
    n = lib().gso_row_slice_coo(_p(coo_row), _p(coo_col), _c(E), _p(row_ids), _c(len(row_ids)), _p(o_r), _p(o_c),
                                _p(o_s))
    return o_r[:n].copy(), o_c[:n].copy(), o_s[:n].copy()


def csc2coo(indptr, indices):
    indptr = _i64(indptr)
    col = np.empty(len(indices), dtype=I64)
    lib().gso_csc2coo(_p(indptr), _c(len(indptr) - 1), _p(col))
    return _i64(indices), col


def coo2csc(row, col, num_cols, col_sorted=False):
    """→ (indptr, sorted_row, perm | None); pass (col, row) swapped for CSR."""
    row, col = _i64(row), _i64(col)
    E = len(row)
    indptr = np.empty(num_cols + 1, dtype=I64)
    out_row = np.empty(E, dtype=I64)
    perm = None if col_sorted else np.empty(E, dtype=I64)
    lib().gso_coo2csc(_p(col), _p(row), _c(E), _c(num_cols), ctypes.c_int(int(col_sorted)), _p(indptr),
                      _p(out_row), _p(perm))
    return indptr, out_row, perm


def sage_batch(indptr, indices, seeds, fanouts, seed=0, want_frontier=False, batch_id=None):
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    f = _i64(np.asarray(fanouts))
    flen = ctypes.c_int64(0)
    cap = 0
    fr = None
    if want_frontier:
        cap = len(seeds)
        for k in fanouts:
            cap = cap * (1 + int(k))
        fr = np.empty(cap, dtype=I64)
    e = lib().gso_sage_batch(_p(indptr), _p(indices), _p(seeds), _c(len(seeds)), _p(f), ctypes.c_int(len(fanouts)),
                             _u(seed), _p(fr), _c(cap), ctypes.byref(flen),
                             _u(0 if batch_id is None else int(batch_id) << 32))
    if want_frontier:
        return int(e), fr[:flen.value].copy()
    return int(e)


# ---- super-batch family (src/pybind.cc:65-84): ids of G batches in one array + an offset array ----------
def _batch_ids(ptr, n):
    """Batch number of each of n items partitioned by ptr (src/cuda/batch_unique.cu:184-194 _RepeatKernel)."""
    ptr = np.asarray(ptr, dtype=I64)
    return (np.searchsorted(ptr, np.arange(n, dtype=I64), side="right") - 1).astype(I64)


def batch_encode(data, data_ptr, encoding_size):
    """src/cuda/batch_coding.cu:10-28."""
    data = np.asarray(data, dtype=I64)
    return data + _batch_ids(data_ptr, len(data)) * encoding_size


def batch_decode(data, encoding_size):
    """src/cuda/batch_coding.cu:87-98."""
    data = np.asarray(data, dtype=I64)
    return data - (data // encoding_size) * encoding_size


def get_batch_offsets(data, num_batches, encoding_size):
    """src/cuda/batch_coding.cu:100-121 → (ptr, decoded): ptr[b+1] = upper bound of b among the batch numbers."""
    data = np.asarray(data, dtype=I64)
    mask = data // encoding_size
    ptr = np.zeros(num_batches + 1, dtype=I64)
    ptr[1:] = np.searchsorted(mask, np.arange(num_batches, dtype=I64), side="right")
    return ptr, data - mask * encoding_size


def batch_col_slice(indptr, indices, seeds, nid_ptr, encoding_size, with_coo=True, encoding=False):
    """src/cuda/slicing.cu:184-270 → (sub_indptr, coo_col | None, sub_indices, select_index, coo_offsets)."""
    sub_indptr, coo_col, sub_indices, select = col_slice(indptr, indices, seeds, with_coo=True)
    nid_ptr = np.asarray(nid_ptr, dtype=I64)
    if encoding:
        sub_indices = sub_indices + _batch_ids(nid_ptr, len(seeds))[coo_col] * encoding_size
    return sub_indptr, (coo_col if with_coo else None), sub_indices, select, sub_indptr[nid_ptr]


def batch_unique(data, data_ptr, sort=False):
    """src/cuda/batch_unique.cu:131-278 → (unique, unique_ptr, unique_key); first-occurrence order per batch,
    or ascending when sort (the cub segment-sort flavour, :215-260)."""
    data, data_ptr = np.asarray(data, dtype=I64), np.asarray(data_ptr, dtype=I64)
    G = len(data_ptr) - 1
    parts, ptr = [], np.zeros(G + 1, dtype=I64)
    for b in range(G):
        u = unique_relabel([data[data_ptr[b]:data_ptr[b + 1]]])[0]
        if sort:
            u = np.sort(u)
        parts.append(u)
        ptr[b + 1] = ptr[b] + len(u)
    uniq = np.concatenate(parts) if parts else np.empty(0, I64)
    return uniq.astype(I64), ptr, _batch_ids(ptr, len(uniq))


def batch_csr_relabel(seeds, seeds_ptr, indices, indices_ptr):
    """src/cuda/batch_relabel.cu:214-320 → (unique, unique_ptr, relabeled_indices)."""
    seeds, seeds_ptr = np.asarray(seeds, dtype=I64), np.asarray(seeds_ptr, dtype=I64)
    indices, indices_ptr = np.asarray(indices, dtype=I64), np.asarray(indices_ptr, dtype=I64)
    G = len(seeds_ptr) - 1
    us, rels, ptr = [], [], np.zeros(G + 1, dtype=I64)
    for b in range(G):
        ind = indices[indices_ptr[b]:indices_ptr[b + 1]]
        u, (r,) = unique_relabel([seeds[seeds_ptr[b]:seeds_ptr[b + 1]], ind], [ind])
        us.append(u)
        rels.append(r)
        ptr[b + 1] = ptr[b] + len(u)
    cat = lambda xs: np.concatenate(xs).astype(I64) if xs else np.empty(0, I64)
    return cat(us), ptr, cat(rels)


def batch_coo_relabel(seeds, seeds_ptr, coo_col, coo_row, coo_ptr):
    """src/cuda/batch_relabel.cu:349-497 → (unique, unique_ptr, relabeled_row, relabeled_col): the frontier of a
    batch is unique(cat(seeds_b, coo_row_b)); a column id that is not in it maps to -1."""
    seeds, seeds_ptr = np.asarray(seeds, dtype=I64), np.asarray(seeds_ptr, dtype=I64)
    coo_col, coo_row, coo_ptr = (np.asarray(a, dtype=I64) for a in (coo_col, coo_row, coo_ptr))
    G = len(seeds_ptr) - 1
    us, rows, cols, ptr = [], [], [], np.zeros(G + 1, dtype=I64)
    for b in range(G):
        r = coo_row[coo_ptr[b]:coo_ptr[b + 1]]
        c = coo_col[coo_ptr[b]:coo_ptr[b + 1]]
        u, (rr, cc) = unique_relabel([seeds[seeds_ptr[b]:seeds_ptr[b + 1]], r], [r, c])
        us.append(u)
        rows.append(rr)
        cols.append(cc)
        ptr[b + 1] = ptr[b] + len(u)
    cat = lambda xs: np.concatenate(xs).astype(I64) if xs else np.empty(0, I64)
    return cat(us), ptr, cat(rows), cat(cols)


def batch_coo_slice(axis, coo_row, coo_col, batch_ptr, neighbors, neighbors_ptr):
    """src/cuda/batch_slicing.cu:166-263 → (sub_row, sub_col, sub_ptr); ids unchanged, order kept."""
    coo_row, coo_col = np.asarray(coo_row, dtype=I64), np.asarray(coo_col, dtype=I64)
    batch_ptr, neighbors_ptr = np.asarray(batch_ptr, dtype=I64), np.asarray(neighbors_ptr, dtype=I64)
    neighbors = np.asarray(neighbors, dtype=I64)
    target = coo_col if axis == 0 else coo_row
    G = len(batch_ptr) - 1
    keep = np.zeros(len(target), dtype=bool)
    ptr = np.zeros(G + 1, dtype=I64)
    for b in range(G):
        sl = slice(batch_ptr[b], batch_ptr[b + 1])
        keep[sl] = np.isin(target[sl], neighbors[neighbors_ptr[b]:neighbors_ptr[b + 1]])
        ptr[b + 1] = ptr[b] + keep[sl].sum()
    return coo_row[keep], coo_col[keep], ptr


def batch_concat(datas, ptrs):
    """src/cuda/batch_concat.cu:11-121 → (data, key, ptr)."""
    datas = [np.asarray(d, dtype=I64) for d in datas]
    ptrs = [np.asarray(p, dtype=I64) for p in ptrs]
    G = len(ptrs[0]) - 1
    parts, keys = [], []
    for b in range(G):
        for d, p in zip(datas, ptrs):
            parts.append(d[p[b]:p[b + 1]])
            keys.append(np.full(p[b + 1] - p[b], b, dtype=I64))
    out_ptr = np.sum(np.stack(ptrs), axis=0).astype(I64)
    cat = lambda xs: np.concatenate(xs).astype(I64) if xs else np.empty(0, I64)
    return cat(parts), cat(keys), out_ptr


def batch_split(data, data_ptr, out_ptrs):
    """src/cuda/batch_split2.cu:11-106 → list of arrays: the inverse of batch_concat."""
    data, data_ptr = np.asarray(data, dtype=I64), np.asarray(data_ptr, dtype=I64)
    out_ptrs = [np.asarray(p, dtype=I64) for p in out_ptrs]
    G = len(data_ptr) - 1
    outs = [np.empty(p[-1], dtype=I64) for p in out_ptrs]
    for b in range(G):
        o = data_ptr[b]
        for out, p in zip(outs, out_ptrs):
            n = p[b + 1] - p[b]
            out[p[b]:p[b + 1]] = data[o:o + n]
            o += n
    return outs


def list_keys(probs, seed=0):
    probs = _f32(probs)
    keys = np.empty(len(probs), dtype=np.float32)
    lib().gso_list_keys(_p(probs), _c(len(probs)), _u(seed), _p(keys))
    return keys


def batch_list_sample(probs, range_ptr, k, seed=0):
    """src/cuda/list_sampling_probs.cu:110-183 → (out_idx, out_range): per segment the min(k, size) positions
    with the largest A-Res keys, in descending key order (ties: smaller position first)."""
    keys = list_keys(probs, seed)
    range_ptr = np.asarray(range_ptr, dtype=I64)
    G = len(range_ptr) - 1
    outs, out_range = [], np.zeros(G + 1, dtype=I64)
    for b in range(G):
        lo, hi = range_ptr[b], range_ptr[b + 1]
        seg = keys[lo:hi]
        order = np.lexsort((np.arange(hi - lo), -seg.astype(np.float64)))
        take = order[:min(k, hi - lo)] + lo
        outs.append(take.astype(I64))
        out_range[b + 1] = out_range[b] + len(take)
    return (np.concatenate(outs).astype(I64) if outs else np.empty(0, I64)), out_range


# ---- induced-subgraph slicing, metapath walk, index search, fused divide + sum ----------------------------
def metapath_random_walk(graphs, path, seeds, seed=0, layout=0, walker_offset=0):
    """src/cuda/fusion/metapath_random_walk.cu:9-67.  graphs: list of (indptr, indices); path: relation per step."""
    gs_ = [(_i64(a), _i64(b)) for a, b in graphs]
    ip = (ctypes.c_void_p * len(gs_))(*[a.ctypes.data for a, _ in gs_])
    ix = (ctypes.c_void_p * len(gs_))(*[b.ctypes.data for _, b in gs_])
    path, seeds = _i64(np.asarray(path)), _i64(seeds)
    W, L = len(seeds), len(path)
    out = np.empty(W * (L + 1), dtype=I64)
    lib().gso_metapath_random_walk(ip, ix, _p(path), _p(seeds), _c(W), _c(L), _u(seed), ctypes.c_int(layout),
                                   _c(walker_offset), _p(out))
    return out.reshape(W, L + 1)


def col_row_slice(indptr, indices, column_ids, row_ids, col_ptr=None, row_ptr=None, renumber=True):
    """src/cuda/fusion/column_row_slicing.cu:101-365 → (out_indptr, out_indices, select_index into `indices`).
    Single list: rows renumbered to their position in row_ids (largest position for a repeated id).  Batched
    (col_ptr / row_ptr): a column of batch b keeps the rows listed for batch b; row ids stay global."""
    indptr, indices = np.asarray(indptr, dtype=I64), np.asarray(indices, dtype=I64)
    column_ids, row_ids = np.asarray(column_ids, dtype=I64), np.asarray(row_ids, dtype=I64)
    S = len(column_ids)
    if col_ptr is None:
        col_batch, tables = np.zeros(S, dtype=I64), [{int(r): i for i, r in enumerate(row_ids)}]
    else:
        col_batch = _batch_ids(col_ptr, S)
        tables = [{int(r): int(row_ptr[b]) + i for i, r in enumerate(row_ids[row_ptr[b]:row_ptr[b + 1]])}
                  for b in range(len(row_ptr) - 1)]
    out_indptr = np.zeros(S + 1, dtype=I64)
    out_i, out_s = [], []
    for c in range(S):
        t = tables[col_batch[c]]
        for e in range(indptr[column_ids[c]], indptr[column_ids[c] + 1]):
            r = int(indices[e])
            if r in t:
                out_i.append(t[r] if renumber else r)
                out_s.append(e)
        out_indptr[c + 1] = len(out_i)
    return out_indptr, np.asarray(out_i, dtype=I64), np.asarray(out_s, dtype=I64)


def index_search(origin, keys):
    """src/tensor_ops.cc:23-31: position of each key in origin (largest for a repeated id), -1 if absent."""
    t = {int(v): i for i, v in enumerate(np.asarray(origin, dtype=I64))}
    return np.asarray([t.get(int(k), -1) for k in np.asarray(keys, dtype=I64)], dtype=I64)


def edge_div_u_sum(coo_row, coo_col, data, divisor, num_cols):
    """src/cuda/fusion/edge_map_reduce.cu:10-24 → (out_data, out_sum)."""
    data = np.ones(len(coo_row), dtype=np.float32) if data is None else np.asarray(data, dtype=np.float32)
    out = (data / np.asarray(divisor, dtype=np.float32)[np.asarray(coo_row, dtype=I64)]).astype(np.float32)
    s = np.zeros(num_cols, dtype=np.float64)
    np.add.at(s, np.asarray(coo_col, dtype=I64), out.astype(np.float64))
    return out, s.astype(np.float32)


def csc_split(indptr, indices, split_size):
    """src/cuda/graph_ops.cu:190-248: consecutive chunks of split_size columns, each with its own offsets."""
    indptr, indices = np.asarray(indptr, dtype=I64), np.asarray(indices, dtype=I64)
    n = len(indptr) - 1
    parts = []
    for c0 in range(0, n, split_size):
        c1 = min(n, c0 + split_size)
        parts.append((indptr[c0:c1 + 1] - indptr[c0], indices[indptr[c0]:indptr[c1]]))
    return parts
