"""`Graph`: the host-side mirror of the reference's `gs::Graph` (src/graph.h:13-126, src/graph.cc) for
the sampling hot path.  It keeps the same state (CSC / CSR / COO views created lazily, optional
edge data, row / column id maps), the same method names, argument meaning and result layout, and
forwards every piece of arithmetic to the sm_100a kernels through the C ABI (graph_sampling_b200.ops).

Differences kept on purpose:
  * errors raise Python exceptions where the reference LOG(FATAL)s and aborts the process;
  * the edge-data gather that follows slicing / sampling is fused into the kernel;
  * stochastic methods take their seed from `ops.set_seed` / an optional `seed=` argument (the
    reference hard-codes 7777 and returns the same sample on every call);
  * DCSC / DCSR (compact id) layouts, batched ("super-batch") methods and pinned-host graphs are
    not part of this path and raise NotImplementedError.
Every method is registered under the CamelCase name of src/pybind.cc and under the snake_case name
the reference's Python layer calls (python/gs/matrix_api/matrix.py).
"""
import torch

from . import ops

_COO, _CSC, _CSR, _DCSC, _DCSR = 1, 2, 4, 8, 16


class CSC:
    """struct CSC / CSR (src/graph_storage.h:9-15)."""
    __slots__ = ("indptr", "indices", "e_ids")

    def __init__(self, indptr, indices, e_ids=None):
        self.indptr, self.indices, self.e_ids = indptr, indices, e_ids


class COO:
    """struct COO (src/graph_storage.h:17-23)."""
    __slots__ = ("row", "col", "e_ids", "row_sorted", "col_sorted")

    def __init__(self, row, col, e_ids=None, row_sorted=False, col_sorted=False):
        self.row, self.col, self.e_ids = row, col, e_ids
        self.row_sorted, self.col_sorted = row_sorted, col_sorted


def _fatal(msg):
    raise RuntimeError(msg)


class Graph:
    def __init__(self, is_subgraph=False, col_ids=None, row_ids=None, num_cols=0, num_rows=0):
        self.is_subgraph_ = bool(is_subgraph)
        self.num_cols_, self.num_rows_, self.num_edges_ = int(num_cols), int(num_rows), 0
        self.csc_ = self.csr_ = self.coo_ = None
        self.data_ = None
        self.col_ids_, self.row_ids_ = col_ids, row_ids
        self.val_col_ids_ = self.val_row_ids_ = None

    # ---- loading (src/graph.cc:14-60) -------------------------------------------------------------
    def LoadCSC(self, indptr, indices):
        self.csc_ = CSC(indptr, indices)
        self.num_cols_ = self.num_rows_ = indptr.numel() - 1
        self.num_edges_ = indices.numel()

    def LoadCSR(self, indptr, indices):
        self.csr_ = CSC(indptr, indices)
        self.num_cols_ = self.num_rows_ = indptr.numel() - 1
        self.num_edges_ = indices.numel()

    def LoadCOO(self, row, col):
        self.coo_ = COO(row, col)
        n = max(torch.unique(row).numel(), torch.unique(col).numel())
        self.num_cols_ = self.num_rows_ = n
        self.num_edges_ = row.numel()

    def LoadCSCWithColIds(self, column_ids, indptr, indices):
        if column_ids.numel() != indptr.numel() - 1:
            _fatal("length of column_ids is not aligned with indptr")
        self.csc_ = CSC(indptr, indices)
        self.col_ids_ = column_ids
        self.num_cols_ = column_ids.numel()
        self.num_rows_ = int(indices.max().item()) + 1 if indices.numel() else 0
        self.num_edges_ = indices.numel()

    def SetMetaData(self, col_ids, row_ids, num_cols, num_rows):
        self.col_ids_, self.row_ids_ = col_ids, row_ids
        self.num_cols_, self.num_rows_ = int(num_cols), int(num_rows)

    def SetCOOByTensor(self, row, col, e_ids, row_sorted, col_sorted):
        self.coo_ = COO(row, col, e_ids, bool(row_sorted), bool(col_sorted))
        self._known_csc = self._known_csr = None

    def SetData(self, data):
        self.data_ = data

    def SetNumEdges(self, n):
        self.num_edges_ = int(n)

    def GetNumRows(self):
        return self.num_rows_

    def GetNumCols(self):
        return self.num_cols_

    def GetNumEdges(self):
        return self.num_edges_

    def _device(self):
        for f in (self.csc_, self.csr_):
            if f is not None:
                return ops.cuda_device_of(f.indptr)
        return ops.cuda_device_of(self.coo_.row)

    def _data_or_ones(self):
        if self.data_ is not None:
            return self.data_
        return torch.ones(self.num_edges_, dtype=torch.float32, device=self._device())

    def GetData(self, order="default"):
        """src/graph.cc:68-90."""
        data = self._data_or_ones()
        idx = None
        if order == "col":
            self.CreateSparseFormat(_CSC)
            idx = self.csc_.e_ids
        elif order == "row":
            self.CreateSparseFormat(_CSR)
            idx = self.csr_.e_ids
        return data[idx] if idx is not None else data

    # ---- lazy format creation (src/graph.cc:585-644, src/graph_ops.cc:13-60) ---------------------------
    def _csc2coo(self, csc, is_csc):
        expanded = ops.csc2coo(csc.indptr, csc.indices)[1]
        if is_csc:
            return COO(csc.indices, expanded, csc.e_ids, False, True)
        return COO(expanded, csc.indices, csc.e_ids, True, False)

    def _coo2csc(self, coo, num_items, to_csc):
        if to_csc:
            indptr, indices, sort_index = ops.coo2csc(coo.row, coo.col, num_items, coo.col_sorted)
        else:
            indptr, indices, sort_index = ops.coo2csc(coo.col, coo.row, num_items, coo.row_sorted)
        if coo.e_ids is not None:
            e_ids = coo.e_ids[sort_index] if sort_index is not None else coo.e_ids
        else:
            e_ids = sort_index
        return CSC(indptr, indices, e_ids)

    # Doubly compressed forms (DCSC / DCSR): offsets only over the columns (rows) that have edges, plus the list of
    # those ids (val_col_ids_ / val_row_ids_) — src/cuda/format_transform.cu:172-203, src/graph_ops.cc:62-110.
    def _coo2dcsc(self, coo, num_items, to_csc):
        dense = self._coo2csc(coo, num_items, to_csc)
        degree = dense.indptr[1:] - dense.indptr[:-1]
        val_ids = torch.nonzero(degree > 0).reshape(-1)
        return CSC(torch.cat([dense.indptr[val_ids], dense.indptr[-1:]]), dense.indices, dense.e_ids), val_ids

    def _dcsc2coo(self, csc, val_ids, is_csc):
        expanded = val_ids[ops.csc2coo(csc.indptr, csc.indices)[1]]
        if is_csc:
            return COO(csc.indices, expanded, csc.e_ids, False, True)
        return COO(expanded, csc.indices, csc.e_ids, True, False)

    def _any2coo(self):
        if self.csc_ is not None:
            if self.val_col_ids_ is not None:
                return self._dcsc2coo(self.csc_, self.val_col_ids_, True)
            return self._csc2coo(self.csc_, True)
        if self.val_row_ids_ is not None:
            return self._dcsc2coo(self.csr_, self.val_row_ids_, False)
        return self._csc2coo(self.csr_, False)

    def CSC2CSR(self):
        self.coo_ = self._csc2coo(self.csc_, True)
        self.csr_ = self._coo2csc(self.coo_, self.num_rows_, False)

    def CSC2DCSR(self):
        self.coo_ = self._csc2coo(self.csc_, True)
        self.csr_, self.val_row_ids_ = self._coo2dcsc(self.coo_, self.num_rows_, False)

    def CSR2CSC(self):
        self.coo_ = self._csc2coo(self.csr_, False)
        self.csc_ = self._coo2csc(self.coo_, self.num_cols_, True)

    def CSR2DCSC(self):
        self.coo_ = self._csc2coo(self.csr_, False)
        self.csc_, self.val_col_ids_ = self._coo2dcsc(self.coo_, self.num_cols_, True)

    def CreateSparseFormat(self, fmt):
        """src/graph.cc:585-644."""
        if fmt == _COO:
            if self.coo_ is None:
                self.coo_ = self._any2coo()
        elif fmt == _CSC:
            if self.csc_ is not None:
                if self.val_col_ids_ is not None:
                    _fatal("Require CSC, get DCSC instead")
                return
            if getattr(self, "_known_csc", None) is not None:
                self.csc_ = self._known_csc
            elif self.coo_ is not None:
                self.csc_ = self._coo2csc(self.coo_, self.num_cols_, True)
            else:
                self.CSR2CSC()
        elif fmt == _DCSC:
            if self.csc_ is not None:
                if self.val_col_ids_ is None:
                    _fatal("Require DCSC, get CSC instead")
                return
            if self.coo_ is not None:
                self.csc_, self.val_col_ids_ = self._coo2dcsc(self.coo_, self.num_cols_, True)
            else:
                self.CSR2DCSC()
        elif fmt == _CSR:
            if self.csr_ is not None:
                if self.val_row_ids_ is not None:
                    _fatal("Require CSR, get DCSR instead")
                return
            if getattr(self, "_known_csr", None) is not None:
                self.csr_ = self._known_csr
            elif self.coo_ is not None:
                self.csr_ = self._coo2csc(self.coo_, self.num_rows_, False)
            else:
                self.CSC2CSR()
        elif fmt == _DCSR:
            if self.csr_ is not None:
                if self.val_row_ids_ is None:
                    _fatal("Require DCSR, get CSR instead")
                return
            if self.coo_ is not None:
                self.csr_, self.val_row_ids_ = self._coo2dcsc(self.coo_, self.num_rows_, False)
            else:
                self.CSC2DCSR()
        else:
            _fatal("unknown sparse format")

    def _compact_col_slicing(self, fmt, val_ids, n_ids, with_coo, data, e_ids):
        """DCSCColSlicingCUDA (src/cuda/slicing.cu:298-413): column slice of a doubly compressed form.  A requested
        id that has no edges is absent from val_ids and yields an empty segment."""
        pos = ops.index_search(val_ids, n_ids)
        present = torch.nonzero(pos >= 0).reshape(-1)
        r = ops.csc_col_slicing(fmt.indptr, fmt.indices, pos[present].contiguous(), with_coo, data=data, e_ids=e_ids)
        counts = torch.zeros(n_ids.numel() + 1, dtype=torch.int64, device=n_ids.device)
        counts[present + 1] = r[0][1:] - r[0][:-1]
        out = [torch.cumsum(counts, 0), present[r[1]] if with_coo else None, r[2], r[3]]
        if data is not None:
            out.append(r[4])
        return out

    # ---- helpers -----------------------------------------------------------------------------------------
    def _child(self, col_ids, row_ids, num_cols, num_rows):
        return Graph(True, col_ids, row_ids, num_cols, num_rows)

    def _gather_args(self, fmt_struct):
        """(data, e_ids) handed to a kernel so that it emits data_[e_ids?[select_index]] itself."""
        if self.data_ is None:
            return None, None
        return self.data_, fmt_struct.e_ids

    # ---- Slicing (src/graph.cc:173-310) ----------------------------------------------------------------------
    def Slicing(self, n_ids, axis, on_format, output_format, relabel=False):
        self.CreateSparseFormat(on_format)
        with_coo = bool(output_format & _COO)
        if axis == 0:
            new_col_ids = self.col_ids_[n_ids] if self.col_ids_ is not None else n_ids
            new_row_ids, new_num_cols, new_num_rows = self.row_ids_, n_ids.numel(), self.num_rows_
        else:
            new_col_ids = self.col_ids_
            new_row_ids = self.row_ids_[n_ids] if self.row_ids_ is not None else n_ids
            new_num_cols, new_num_rows = self.num_cols_, n_ids.numel()
        csc_ptr = csr_ptr = coo_ptr = None
        known_csc = known_csr = None
        out_data = None
        new_val_cols = new_val_rows = None

        if on_format == _COO:
            coo = self.coo_
            if axis == 0:   # keep edges whose column is in n_ids (COOColSlicing, src/graph_ops.cc:173-190)
                new_col, new_row, select = ops.coo_row_slicing(coo.col, coo.row, n_ids)
            else:
                new_row, new_col, select = ops.coo_row_slicing(coo.row, coo.col, n_ids)
            coo_ptr = COO(new_row, new_col, None, coo.row_sorted, coo.col_sorted)
            new_num_edges = new_row.numel()
            e_ids = coo.e_ids
            if self.data_ is not None:
                out_data = self.data_[e_ids[select] if e_ids is not None else select]
        elif on_format in (_CSC, _DCSC):
            if output_format == _CSR:
                _fatal("Error in Slicing, Not implementation [on_format = CSC, output_forat = CSR]")
            data, e_ids = self._gather_args(self.csc_)
            if axis == 0:
                if self.val_col_ids_ is not None:
                    r = self._compact_col_slicing(self.csc_, self.val_col_ids_, n_ids, with_coo, data, e_ids)
                else:
                    r = ops.csc_col_slicing(self.csc_.indptr, self.csc_.indices, n_ids, with_coo, data=data,
                                            e_ids=e_ids)
                indptr, coo_col, indices = r[0], r[1], r[2]
                out_data = r[4] if data is not None else None
                if relabel:
                    frontier, (indices,) = ops.relabel([indices], [indices])
                    new_row_ids, new_num_rows = frontier, frontier.numel()
            else:
                if relabel:
                    _fatal("Not implemented warning")
                indptr, coo_col, indices, select = ops.csc_row_slicing(self.csc_.indptr, self.csc_.indices, n_ids,
                                                                       with_coo)
                new_val_cols = self.val_col_ids_
                if data is not None:
                    out_data = ops.take(data, ops.take(e_ids, select) if e_ids is not None else select)
            if output_format & _CSC:
                csc_ptr = CSC(indptr, indices)
            elif new_val_cols is None:
                known_csc = CSC(indptr, indices)
            if output_format & _COO:
                coo_ptr = COO(indices, coo_col, None, False, True)
            new_num_edges = indices.numel()
        elif on_format in (_CSR, _DCSR):
            if output_format == _CSC:
                _fatal("Error in Slicing, Not implementation [on_format = CSR, output_forat = CSC]")
            data, e_ids = self._gather_args(self.csr_)
            if axis == 0:
                if relabel:
                    _fatal("Not implemented warning")
                indptr, coo_row, indices, select = ops.csc_row_slicing(self.csr_.indptr, self.csr_.indices, n_ids,
                                                                       with_coo)
                new_val_rows = self.val_row_ids_
                if data is not None:
                    out_data = ops.take(data, ops.take(e_ids, select) if e_ids is not None else select)
            else:
                if self.val_row_ids_ is not None:
                    r = self._compact_col_slicing(self.csr_, self.val_row_ids_, n_ids, with_coo, data, e_ids)
                else:
                    r = ops.csc_col_slicing(self.csr_.indptr, self.csr_.indices, n_ids, with_coo, data=data,
                                            e_ids=e_ids)
                indptr, coo_row, indices = r[0], r[1], r[2]
                out_data = r[4] if data is not None else None
                if relabel:
                    frontier, (indices,) = ops.relabel([indices], [indices])
                    new_col_ids, new_num_cols = frontier, frontier.numel()
            if output_format & _CSR:
                csr_ptr = CSC(indptr, indices)
            elif new_val_rows is None:
                known_csr = CSC(indptr, indices)
            if output_format & _COO:
                coo_ptr = COO(coo_row, indices, None, True, False)
            new_num_edges = indices.numel()
        else:
            _fatal("Not implemented warning")

        ret = self._child(new_col_ids, new_row_ids, new_num_cols, new_num_rows)
        ret.num_edges_ = new_num_edges
        ret.coo_, ret.csc_, ret.csr_ = coo_ptr, csc_ptr, csr_ptr
        # The slice computed these offsets anyway.  The child does not HOLD the format (which formats a graph holds
        # decides, e.g., what Relabel returns), but a later CreateSparseFormat adopts it instead of converting the COO:
        # the arrays are exactly what that conversion would produce from a COO sorted along this axis.
        ret._known_csc, ret._known_csr = known_csc, known_csr
        ret.val_col_ids_, ret.val_row_ids_ = new_val_cols, new_val_rows
        if out_data is not None:
            ret.data_ = out_data
        return ret

    # ---- BatchSlicing (src/graph.cc:312-391) --------------------------------------------------------------
    def BatchSlicing(self, n_ids, nid_ptr, axis, on_format, output_format, relabel=False, encoding=False):
        """Column slice for the seeds of many batches at once → (Graph, coo_offsets).  The child's column ids are
        the seeds encoded with their batch number (id + batch * num_rows) and it spans num_rows * batches rows;
        with `encoding` the row ids of its edges are encoded the same way."""
        if axis != 0:
            _fatal("batch slicing only suppurt column slicing now")
        if on_format != _CSC:
            _fatal("Not Implementatin Error")
        self.CreateSparseFormat(on_format)
        with_coo = bool(output_format & _COO)
        batch_num = nid_ptr.numel() - 1
        new_col_ids = self.col_ids_[n_ids] if self.col_ids_ is not None else ops.batch_encode(n_ids, nid_ptr,
                                                                                               self.num_rows_)
        new_row_ids, new_num_rows = self.row_ids_, self.num_rows_ * batch_num
        data, e_ids = self._gather_args(self.csc_)
        r = ops.batch_csc_col_slicing(self.csc_.indptr, self.csc_.indices, n_ids, nid_ptr, self.num_rows_, with_coo,
                                      encoding, data=data, e_ids=e_ids)
        indptr, coo_col, indices, coo_offsets = r[0], r[1], r[2], r[4]
        if relabel:
            frontier, (indices,) = ops.relabel([indices], [indices])
            new_row_ids, new_num_rows = frontier, frontier.numel()
        ret = self._child(new_col_ids, new_row_ids, n_ids.numel(), new_num_rows)
        ret.num_edges_ = indices.numel()
        if output_format & _CSC:
            ret.csc_ = CSC(indptr, indices)
        if with_coo:
            ret.coo_ = COO(indices, coo_col, None, False, True)
        if data is not None:
            ret.data_ = r[5]
        return ret, coo_offsets

    # ---- induced subgraph (src/graph.cc:116-170) ----------------------------------------------------------
    def FusedBidirSlicing(self, column_seeds, row_seeds):
        """Columns `column_seeds` x rows `row_seeds` of the CSC in one pass; rows are renumbered to their position in
        row_seeds.  Edge data follows the kept edges (the reference gathers it with positions inside the column
        slice, src/graph.cc:131-137, which only works when every column is a seed)."""
        self.CreateSparseFormat(_CSC)
        col_ids = self.col_ids_[column_seeds] if self.col_ids_ is not None else column_seeds
        row_ids = self.row_ids_[row_seeds] if self.row_ids_ is not None else row_seeds
        data, e_ids = self._gather_args(self.csc_)
        r = ops.csc_col_row_slicing(self.csc_.indptr, self.csc_.indices, col_ids, row_ids, data=data, e_ids=e_ids)
        ret = self._child(col_ids, row_ids, column_seeds.numel(), row_seeds.numel())
        ret.csc_ = CSC(r[0], r[1])
        ret.num_edges_ = r[1].numel()
        if data is not None:
            ret.data_ = r[3]
        return ret

    def BatchFusedBidirSlicing(self, column_seeds, col_ptr, row_seeds, row_ptr):
        """Super-batch form: a column of batch b keeps the rows listed for batch b; row ids stay global."""
        self.CreateSparseFormat(_CSC)
        col_ids = self.col_ids_[column_seeds] if self.col_ids_ is not None else column_seeds
        data, e_ids = self._gather_args(self.csc_)
        r = ops.csc_col_row_slicing(self.csc_.indptr, self.csc_.indices, col_ids, row_seeds, col_ptr, row_ptr,
                                    self.num_rows_, data=data, e_ids=e_ids)
        ret = self._child(col_ids, self.row_ids_, column_seeds.numel(), self.num_rows_)
        ret.csc_ = CSC(r[0], r[1])
        ret.num_edges_ = r[1].numel()
        if data is not None:
            ret.data_ = r[3]
        return ret

    def EDivUSum(self, divisor):
        """(Graph with data / divisor[row], per-column sums of that) — src/graph.cc:732-755.  Edge data keeps its
        order; the reference pairs data_[i] with COO edge i and is only right when the COO carries no edge ids."""
        self.CreateSparseFormat(_COO)
        e_ids = self.coo_.e_ids
        data = self.data_ if (self.data_ is None or e_ids is None) else self.data_[e_ids]
        out, out_sum = ops.coo_e_div_u_sum(self.coo_.row, self.coo_.col, data, divisor, self.num_cols_)
        if e_ids is not None:
            full = torch.empty_like(out)
            full[e_ids] = out
            out = full
        return self._same_structure_child(out), out_sum

    def Split(self, split_size):
        """Consecutive chunks of split_size columns as separate graphs (src/graph.cc:987-1017)."""
        self.CreateSparseFormat(_CSC)
        n = self.csc_.indptr.numel() - 1
        split_size = int(split_size)
        bounds = list(range(0, n, split_size)) + [n]
        offsets = torch.tensor(bounds, dtype=torch.int64, device=ops.cuda_device_of(self.csc_.indptr))
        indptrs = ops.indptr_split_by_offset(self.csc_.indptr, offsets)
        edge_bounds = self.csc_.indptr[offsets]
        indices = ops.split_by_offset(self.csc_.indices, edge_bounds)
        eids = ops.split_by_offset(self.csc_.e_ids, edge_bounds) if self.csc_.e_ids is not None else None
        nids = torch.split(self.col_ids_, split_size) if self.col_ids_ is not None else None
        out = []
        for i in range(len(bounds) - 1):
            g = self._child(nids[i] if nids is not None else None, self.row_ids_, bounds[i + 1] - bounds[i],
                            self.num_rows_)
            g.csc_ = CSC(indptrs[i], indices[i], eids[i] if eids is not None else None)
            g.num_edges_ = indices[i].numel()
            out.append(g)
        return out

    # ---- Sampling / SamplingProbs (src/graph.cc:393-529) ---------------------------------------------------
    def _sampling_impl(self, axis, fanout, replace, on_format, output_format, probs, seed):
        self.CreateSparseFormat(on_format)
        with_coo = bool(output_format & _COO)
        ret = self._child(self.col_ids_, self.row_ids_, self.num_cols_, self.num_rows_)
        if axis == 0 and on_format == _CSC:
            if output_format == _CSR:
                _fatal("Error in Sampling, Not implementation [on_format = CSC, output_forat = CSR]")
            fmt = self.csc_
        elif axis == 1 and on_format == _CSR:
            if output_format == _CSC:
                _fatal("Error in Sampling, Not implementation [on_format = CSR, output_forat = CSC]")
            fmt = self.csr_
        else:
            _fatal("No implementation!")
        data, e_ids = self._gather_args(fmt)
        if probs is None:
            r = ops.csc_col_sampling(fmt.indptr, fmt.indices, fanout, replace, with_coo, seed=seed, data=data,
                                     e_ids=e_ids)
        else:
            r = ops.csc_col_sampling_probs(fmt.indptr, fmt.indices, probs, fanout, replace, with_coo, seed=seed,
                                           data=data, e_ids=e_ids)
        indptr, coo_other, indices = r[0], r[1], r[2]
        if axis == 0:
            if output_format & _CSC:
                ret.csc_ = CSC(indptr, indices)
            if output_format & _COO:
                ret.coo_ = COO(indices, coo_other, None, False, True)
        else:
            if output_format & _CSR:
                ret.csr_ = CSC(indptr, indices)
            if output_format & _COO:
                ret.coo_ = COO(coo_other, indices, None, True, False)
        ret.num_edges_ = indices.numel()
        if data is not None:
            ret.data_ = r[4]
        return ret

    def Sampling(self, axis, fanout, replace, on_format, output_format, seed=None):
        return self._sampling_impl(axis, fanout, replace, on_format, output_format, None, seed)

    def SamplingProbs(self, axis, edge_probs, fanout, replace, on_format, output_format, seed=None):
        return self._sampling_impl(axis, fanout, replace, on_format, output_format, edge_probs, seed)

    def ColumnwiseFusedSlicingAndSampling(self, column_index, fanout, replace, seed=None):
        """src/graph.cc:531-559 (+ keep-dim variant chosen like src/graph_ops.cc:223-247)."""
        col_ids = self.col_ids_[column_index] if self.col_ids_ is not None else column_index
        ret = self._child(col_ids, self.row_ids_, col_ids.numel(), self.num_rows_)
        csc = self.csc_
        if csc is None:
            _fatal("ColumnwiseFusedSlicingAndSampling needs a CSC graph")
        data, e_ids = self._gather_args(csc)
        if fanout == 1 and replace:
            indptr, indices, select = ops.fused_csc_col_slicing_sampling_one_keepdim(csc.indptr, csc.indices,
                                                                                     column_index, seed=seed)
            out_data = None
            if data is not None:
                safe = select.clamp(min=0)
                out_data = ops.take(data, ops.take(e_ids, safe) if e_ids is not None else safe)
        else:
            r = ops.fused_csc_col_slicing_sampling(csc.indptr, csc.indices, column_index, fanout, replace, seed=seed,
                                                   data=data, e_ids=e_ids)
            indptr, indices = r[0], r[1]
            out_data = r[3] if data is not None else None
        ret.csc_ = CSC(indptr, indices)
        ret.num_edges_ = indices.numel()
        if out_data is not None:
            ret.data_ = out_data
        return ret

    # ---- AllValidNode / Relabel (src/graph.cc:757-839) ----------------------------------------------------------
    def _require_col_ids(self):
        if self.col_ids_ is None:
            raise RuntimeError("For sampling, col_ids_ is necessary!")
        return self.col_ids_

    def AllValidNode(self):
        col_ids = self._require_col_ids()
        if self.csc_ is not None:
            rows = self.row_ids_ if self.row_ids_ is not None else self.csc_.indices
        elif self.coo_ is not None:
            rows = self.row_ids_ if self.row_ids_ is not None else self.coo_.row
        elif self.csr_ is not None:
            self.coo_ = self._csc2coo(self.csr_, False)
            rows = self.row_ids_ if self.row_ids_ is not None else self.coo_.row
        else:
            _fatal("Error in AllValidNode!")
        return ops.relabel([col_ids, rows], [])[0]

    def Relabel(self):
        col_ids = self._require_col_ids()
        if self.csc_ is not None:
            if self.val_col_ids_ is not None:
                col_ids = col_ids[self.val_col_ids_]
            row_indices = self.row_ids_[self.csc_.indices] if self.row_ids_ is not None else self.csc_.indices
            frontier, (relabeled,) = ops.relabel([col_ids, row_indices], [row_indices])
            return (frontier, frontier.numel(), col_ids.numel(), self.csc_.indptr.clone(), relabeled, self.csc_.e_ids,
                    "csc")
        if self.csr_ is not None or self.coo_ is not None:
            if self.coo_ is None:
                self.coo_ = self._csc2coo(self.csr_, False)
            coo_col = col_ids[self.coo_.col]
            coo_row = self.row_ids_[self.coo_.row] if self.row_ids_ is not None else self.coo_.row
            frontier, (rel_col, rel_row) = ops.relabel([col_ids, coo_row], [coo_col, coo_row])
            return (frontier, frontier.numel(), col_ids.numel(), rel_row, rel_col, self.coo_.e_ids, "coo")
        _fatal("Error in Relabel!")

    # ---- RandomWalk (src/graph.cc:646-648) -------------------------------------------------------------------------
    def RandomWalk(self, seeds, walk_length, seed=None, layout=0):
        """layout=0 reproduces the reference: step-major memory viewed as [len(seeds), walk_length+1]
        (undo with `.reshape(-1, len(seeds))`, as the reference's own tests do); layout=1 returns the
        walker-major trace."""
        if self.csc_ is None:
            _fatal("RandomWalk needs a CSC graph")
        return ops.fused_random_walk(seeds, walk_length, self.csc_.indices, self.csc_.indptr, seed=seed, layout=layout)

    # ---- SDDMM (src/graph.cc:967-985) ------------------------------------------------------------------------------------
    def SDDMM(self, op, lhs, rhs, out, lhs_target, rhs_target, on_format):
        self.CreateSparseFormat(on_format)
        if on_format in (_DCSC, _DCSR):
            # a compact form numbers its segments by position in val_*_ids_; the COO view has the node ids again and
            # carries the same edge ids, so the result lands in the same order
            self.CreateSparseFormat(_COO)
            on_format = _COO
        if on_format == _COO:
            ops.sddmm(op, lhs, rhs, out, lhs_target, rhs_target, self.coo_.row, self.coo_.col, e_ids=self.coo_.e_ids)
        elif on_format == _CSR:
            lt = lhs_target if lhs_target == 1 else 2 - lhs_target
            rt = rhs_target if rhs_target == 1 else 2 - rhs_target
            ops.sddmm(op, lhs, rhs, out, lt, rt, self.csr_.indices, None, indptr=self.csr_.indptr,
                      e_ids=self.csr_.e_ids)
        elif on_format == _CSC:
            ops.sddmm(op, lhs, rhs, out, lhs_target, rhs_target, self.csc_.indices, None, indptr=self.csc_.indptr,
                      e_ids=self.csc_.e_ids)
        else:
            _fatal("SDDMM only supports CSR and COO formats")

    # ---- Sum / Normalize / Divide (src/graph.cc:650-730) --------------------------------------------------------------------
    def Sum(self, axis, powk, on_format):
        self.CreateSparseFormat(on_format)
        data = self.data_
        out_size = self.num_cols_ if axis == 0 else self.num_rows_
        out = torch.zeros(out_size, dtype=torch.float32, device=self._device())
        if on_format == _COO:
            by_row = (1 - axis) == 0
            target = self.coo_.row if by_row else self.coo_.col
            ops.coo_sum(target, self.coo_.e_ids, data, out, powk,
                        targets_in_runs=self.coo_.row_sorted if by_row else self.coo_.col_sorted)
        elif (axis == 0 and on_format in (_CSC, _DCSC)) or (axis == 1 and on_format in (_CSR, _DCSR)):
            fmt, val_ids = (self.csc_, self.val_col_ids_) if axis == 0 else (self.csr_, self.val_row_ids_)
            if val_ids is None:
                ops.csc_sum(fmt.indptr, fmt.e_ids, data, out, powk)
            else:  # segment c of a compact form belongs to node val_ids[c] (src/cuda/graph_ops.cu:15-39)
                compact = torch.zeros(val_ids.numel(), dtype=torch.float32, device=out.device)
                ops.csc_sum(fmt.indptr, fmt.e_ids, data, compact, powk)
                out[val_ids] = compact
        else:
            _fatal("axis should be 0 or 1? on_format and axis do not match?")
        return out

    def _same_structure_child(self, data):
        ret = Graph(self.is_subgraph_, self.col_ids_, self.row_ids_, self.num_cols_, self.num_rows_)
        ret.csc_, ret.csr_, ret.coo_ = self.csc_, self.csr_, self.coo_
        ret.num_edges_ = self.num_edges_
        ret.data_ = data
        ret.val_col_ids_, ret.val_row_ids_ = self.val_col_ids_, self.val_row_ids_
        return ret

    def Normalize(self, axis, on_format):
        self.CreateSparseFormat(on_format)
        in_data = self._data_or_ones()
        out = torch.empty_like(in_data)
        if axis == 0 and on_format in (_CSC, _DCSC):
            ops.csc_normalize(self.csc_.indptr, self.csc_.e_ids, in_data, out)
        elif axis == 1 and on_format in (_CSR, _DCSR):
            ops.csc_normalize(self.csr_.indptr, self.csr_.e_ids, in_data, out)
        else:
            _fatal("Not Implementation Error")
        return self._same_structure_child(out)

    def Divide(self, divisor, axis, on_format):
        self.CreateSparseFormat(on_format)
        in_data = self._data_or_ones()
        out = torch.zeros(self.num_edges_, dtype=torch.float32, device=in_data.device)
        if on_format == _COO:
            rhs_target = 0 if (1 - axis) == 0 else 2
            ops.sddmm("div", in_data, divisor, out, 1, rhs_target, self.coo_.row, self.coo_.col,
                      e_ids=self.coo_.e_ids)
        elif (axis == 0 and on_format in (_CSC, _DCSC)) or (axis == 1 and on_format in (_CSR, _DCSR)):
            fmt, val_ids = (self.csc_, self.val_col_ids_) if axis == 0 else (self.csr_, self.val_row_ids_)
            per_segment = divisor if val_ids is None else divisor[val_ids].contiguous()
            ops.sddmm("div", in_data, per_segment, out, 1, 2, fmt.indices, None, indptr=fmt.indptr, e_ids=fmt.e_ids)
        return self._same_structure_child(out)

    # ---- getters (src/graph.cc:841-965) ------------------------------------------------------------------------------------
    def GetRows(self):
        if self.row_ids_ is not None:
            return self.row_ids_
        return torch.arange(self.num_rows_, dtype=torch.int64, device=self._device())

    def GetCols(self):
        if self.col_ids_ is not None:
            return self.col_ids_
        return torch.arange(self.num_cols_, dtype=torch.int64, device=self._device())

    def GetCOORows(self, is_original):
        if self.coo_ is not None:
            rows = self.coo_.row
        elif self.csc_ is not None and self.csc_.e_ids is None:
            rows = self.csc_.indices
        elif self.csr_ is not None and self.csr_.e_ids is None:
            self.coo_ = self._csc2coo(self.csr_, False)
            rows = self.coo_.row
        else:
            _fatal("Error in GetCOORows!")
        return self.row_ids_[rows] if (is_original and self.row_ids_ is not None) else rows

    def GetCOOCols(self, is_original):
        if self.coo_ is not None:
            cols = self.coo_.col
        elif self.csc_ is not None and self.csc_.e_ids is None:
            self.coo_ = self._csc2coo(self.csc_, True)
            cols = self.coo_.col
        elif self.csr_ is not None and self.csr_.e_ids is None:
            cols = self.csr_.indices
        else:
            _fatal("Error in GetCOOCols!")
        return self.col_ids_[cols] if (is_original and self.col_ids_ is not None) else cols

    def GetValidRows(self):
        local = self.val_row_ids_ if self.val_row_ids_ is not None else torch.unique(self.GetCOORows(False))
        return self.row_ids_[local] if self.row_ids_ is not None else local

    def GetValidCols(self):
        local = self.val_col_ids_ if self.val_col_ids_ is not None else torch.unique(self.GetCOOCols(False))
        return self.col_ids_[local] if self.col_ids_ is not None else local

    def MetaData(self):
        if self.csc_ is not None:
            return [self.col_ids_, self.row_ids_, self._data_or_ones(), self.csc_.indptr, self.csc_.indices]
        if self.csr_ is not None:
            return [self.col_ids_, self.row_ids_, self._data_or_ones(), self.csr_.indptr, self.csr_.indices]
        return [self.coo_.row, self.coo_.col]

    def COOMetaData(self):
        if self.coo_ is None:
            return []
        return [self.col_ids_, self.row_ids_, self.data_, self.coo_.row, self.coo_.col]

    def CSCMetaData(self):
        if self.csc_ is None:
            return []
        return [self.col_ids_, self.row_ids_, self.data_, self.csc_.indptr, self.csc_.indices]

    def GetCSCTensor(self):
        self.CreateSparseFormat(_CSC)
        return [self.csc_.indptr, self.csc_.indices, self.csc_.e_ids]

    def GetCOOTensor(self):
        self.CreateSparseFormat(_COO)
        if not self.coo_.col_sorted:
            _fatal("Check failed: coo_->col_sorted == true")
        return [self.coo_.row, self.coo_.col, self.coo_.e_ids]

    def Decode(self, encoding_size):
        """Strips the batch encoding from both id maps.  (The reference's version aborts whenever an id map is
        present and dereferences it when it is absent, src/graph.cc:1035-1040; this one does what its name says.)"""
        if self.col_ids_ is None or self.row_ids_ is None:
            _fatal("Error: Decoding should have both row and column id")
        self.col_ids_ = ops.batch_decode(self.col_ids_, encoding_size)
        self.row_ids_ = ops.batch_decode(self.row_ids_, encoding_size)


# Registered names: src/pybind.cc:14-52 (CamelCase) and the spelling used by python/gs + examples.
_NAME_MAP = {
    "SetData": ("_CAPI_SetData", "_CAPI_set_data"),
    "GetData": ("_CAPI_GetData", "_CAPI_get_data"),
    "GetNumRows": ("_CAPI_GetNumRows", "_CAPI_get_num_rows"),
    "GetNumCols": ("_CAPI_GetNumCols", "_CAPI_get_num_cols"),
    "GetNumEdges": ("_CAPI_GetNumEdges", "_CAPI_get_num_edges"),
    "Slicing": ("_CAPI_Slicing", "_CAPI_slicing"),
    "Sampling": ("_CAPI_Sampling", "_CAPI_sampling"),
    "SamplingProbs": ("_CAPI_SamplingWithProbs", "_CAPI_sampling_with_probs"),
    "ColumnwiseFusedSlicingAndSampling": ("_CAPI_FusedColumnwiseSlicingSampling",
                                          "_CAPI_fused_columnwise_slicing_sampling"),
    "LoadCSC": ("_CAPI_LoadCSC", "_CAPI_load_csc", "load_csc"),
    "LoadCOO": ("_CAPI_LoadCOO", "_CAPI_load_coo"),
    "LoadCSCWithColIds": ("_CAPI_LoadCSCWithColIds", "_CAPI_load_csc_with_col_ids"),
    "AllValidNode": ("_CAPI_AllValidNode", "_CAPI_all_valid_node", "_CAPI_all_indices"),
    "GetRows": ("_CAPI_GetRows", "_CAPI_get_rows"),
    "GetCols": ("_CAPI_GetCols", "_CAPI_get_cols"),
    "GetValidRows": ("_CAPI_GetValidRows", "_CAPI_get_valid_rows"),
    "GetValidCols": ("_CAPI_GetValidCols", "_CAPI_get_valid_cols"),
    "GetCOORows": ("_CAPI_GetCOORows", "_CAPI_get_coo_rows"),
    "GetCOOCols": ("_CAPI_GetCooCols", "_CAPI_get_coo_cols"),
    "Relabel": ("_CAPI_Relabel", "_CAPI_relabel"),
    "Sum": ("_CAPI_Sum", "_CAPI_sum"),
    "Normalize": ("_CAPI_Normalize", "_CAPI_normalize"),
    "Divide": ("_CAPI_Divide", "_CAPI_divide"),
    "MetaData": ("_CAPI_Metadata", "_CAPI_metadata"),
    "COOMetaData": ("_CAPI_COOMetadata", "_CAPI_coo_metadata"),
    "CSCMetaData": ("_CAPI_CSCMetadata", "_CAPI_csc_metadata"),
    "RandomWalk": ("_CAPI_RandomWalk", "_CAPI_random_walk"),
    "SDDMM": ("_CAPI_SDDMM", "_CAPI_sddmm"),
    "GetCSCTensor": ("_CAPI_GetCSC", "_CAPI_get_csc"),
    "GetCOOTensor": ("_CAPI_GetCOO", "_CAPI_get_coo"),
    "SetCOOByTensor": ("_CAPI_SetCOO", "_CAPI_set_coo"),
    "SetMetaData": ("_CAPI_SetMetadata", "_CAPI_set_metadata"),
    "FusedBidirSlicing": ("_CAPI_FusionSlicing", "_CAPI_fusion_slicing"),
    "CSC2DCSR": ("_CAPI_CSC2DCSR",),
    "CSR2DCSC": ("_CAPI_CSR2DCSC",),
    "BatchSlicing": ("_CAPI_BatchSlicing", "_CAPI_batch_slicing"),
    "BatchFusedBidirSlicing": ("_CAPI_BatchFusionSlicing", "_CAPI_batch_fusion_slicing"),
    "Split": ("_CAPI_Split", "_CAPI_split"),
    "Decode": ("_CAPI_Decode", "_CAPI_decode"),
    "EDivUSum": ("_CAPI_EDivUSum", "_CAPI_e_div_u_sum"),
}
for _method, _aliases in _NAME_MAP.items():
    for _alias in _aliases:
        setattr(Graph, _alias, getattr(Graph, _method))


def ListSampling(data, num_picks, replace, seed=None):
    """gs::ListSampling (src/tensor_ops.cc:5-9); registered as gs_ops._CAPI_ListSampling / list_sampling."""
    return ops.list_sampling(data, num_picks, replace, seed=seed)


def ListSamplingProbs(data, probs, num_picks, replace, seed=None):
    """gs::ListSamplingProbs (src/tensor_ops.cc:11-16); gs_ops._CAPI_ListSamplingWithProbs / list_sampling_with_probs."""
    return ops.list_sampling(data, num_picks, replace, probs=probs, seed=seed)


class HeteroGraph:
    """gs::HeteroGraph (src/hetero_graph.h:38-70, src/hetero_graph.cc:20-75): named relations, each a homogeneous
    Graph, and the fused metapath random walk over them."""

    def __init__(self):
        self.node_type_mapping_, self.edge_type_mapping_ = {}, {}
        self.hetero_edges_ = {}

    def LoadFromHomo(self, node_types, edge_types, edge_relations):
        if len(edge_types) != len(edge_relations):
            _fatal("edge_types and edge_relations differ in length")
        self.node_type_mapping_ = {name: i for i, name in enumerate(node_types)}
        self.edge_type_mapping_, self.hetero_edges_ = {}, {}
        for i, ((src, etype, dst), graph) in enumerate(zip(edge_types, edge_relations)):
            self.edge_type_mapping_[etype] = i
            graph.CreateSparseFormat(_CSC)
            self.hetero_edges_[i] = (self.node_type_mapping_[src], self.node_type_mapping_[dst], graph)

    def GetHomoGraph(self, edge_type):
        return self.hetero_edges_[self.edge_type_mapping_[edge_type]][2]

    def MetapathRandomWalkFused(self, seeds, metapath, seed=None, layout=0):
        """Trace of shape [num_seeds, len(metapath) + 1]; layout 0 is the reference's step-major memory viewed
        with that shape (as Graph.RandomWalk), layout 1 a true walker-major trace."""
        path = [self.edge_type_mapping_[name] for name in metapath]
        graphs = [(self.hetero_edges_[i][2].csc_.indptr, self.hetero_edges_[i][2].csc_.indices)
                  for i in range(len(self.hetero_edges_))]
        return ops.fused_metapath_random_walk(seeds, path, graphs, seed=seed, layout=layout)

    _CAPI_LoadFromHomo = _CAPI_load_from_homo = LoadFromHomo
    _CAPI_GetHomoGraph = _CAPI_get_homo_graph = GetHomoGraph
    _CAPI_MetapathRandomWalkFused = _CAPI_metapath_random_walk_fused = MetapathRandomWalkFused


# Free operators of the super-batch family under their registered names (src/pybind.cc:65-84).
def _batch_ops():
    o = ops
    return {
        "_CAPI_BatchListSamplingWithProbs": o.batch_list_sampling_probs,
        "_CAPI_SplitByOffset": o.split_by_offset,
        "_CAPI_IndptrSplitBySize": o.indptr_split_by_size,
        "_CAPI_IndptrSplitByOffset": o.indptr_split_by_offset,
        "_CAPI_BatchConcat": o.batch_concat,
        "_CAPI_BatchUnique": lambda d, p: o.batch_unique(d, p, sort=False),
        "_CAPI_BatchUniqueByKey": lambda d, p, k: o.batch_unique(d, p, sort=False),
        "_CAPI_BatchUnique2": lambda d, p: o.batch_unique(d, p, sort=True),
        "_CAPI_BatchUniqueByKey2": lambda d, p, k: o.batch_unique(d, p, sort=True),
        "_CAPI_BatchCSRRelabel": o.batch_csr_relabel,
        "_CAPI_BatchCSRRelabelByKey": lambda s, sp, sk, i, ip, ik: o.batch_csr_relabel(s, sp, i, ip),
        "_CAPI_BatchCOORelabel": o.batch_coo_relabel,
        "_CAPI_BatchCOORelabelByKey": lambda s, sp, sk, c, r, p, k: o.batch_coo_relabel(s, sp, c, r, p),
        "_CAPI_BatchSplit": o.batch_split,
        "_CAPI_BatchCOOSlicing": o.batch_coo_slicing,
        "_CAPI_BatchEncode": o.batch_encode,
        "_CAPI_BatchDecode": o.batch_decode,
        "_CAPI_GetBatchOffsets": o.get_batch_offsets,
        "_CAPI_COORowSlicingGlobalId": o.coo_row_slicing_global_id,
        "_CAPI_IndexSearch": o.index_search,
    }


class _GsOps:
    """Stand-in for `torch.ops.gs_ops` in the Python face: gs_ops._CAPI_BatchUnique(...) and so on."""

    def __getattr__(self, name):
        table = _batch_ops()
        table.update({"_CAPI_ListSampling": ListSampling, "_CAPI_ListSamplingWithProbs": ListSamplingProbs,
                      "_CAPI_Unique": Unique, "_CAPI_SetSeed": ops.set_seed, "list_sampling": ListSampling,
                      "list_sampling_with_probs": ListSamplingProbs})
        for key in (name, "_CAPI_" + name):
            if key in table:
                return table[key]
        raise AttributeError(f"gs_ops has no operator {name}")


gs_ops = _GsOps()


def Unique(node_ids):
    """gs_ops._CAPI_Unique = gs::impl::TensorUniqueCUDA (src/pybind.cc:85)."""
    return ops.tensor_unique(node_ids)
