"""`Matrix`: thin object wrapper over `Graph`, method for method the reference's gs.Matrix
(python/gs/matrix_api/matrix.py:13-119), plus `normalize`, which the reference's examples call but its
Matrix lacks."""
from dataclasses import dataclass
from typing import Optional

import torch
import torch.fx

from ..graph import Graph, _COO, _CSC, _CSR


@dataclass
class Block:
    """DGL-free description of one message-flow block: what `to_dgl_block` hands to DGL in the
    reference (python/gs/matrix_api/matrix.py:40-64).  `format` is "csc" (indptr, indices) or "coo"
    (row, col); ids are local: rows index `src_ids`, columns index the first `num_dst` entries."""
    format: str
    tensor1: torch.Tensor
    tensor2: torch.Tensor
    num_src: int
    num_dst: int
    src_ids: Optional[torch.Tensor]
    edge_ids: Optional[torch.Tensor]
    edge_weight: Optional[torch.Tensor]


class Matrix:
    def __init__(self, graph: Optional[Graph] = None):
        self._graph = graph if graph is not None else Graph(False)

    def load_csc(self, indptr, indices, weight=None):
        self._graph._CAPI_load_csc(indptr, indices)
        if weight is not None:
            self._graph._CAPI_set_data(weight)
        return self

    def set_data(self, data):
        self._graph._CAPI_set_data(data)

    def get_data(self, order: str = "default"):
        return self._graph._CAPI_get_data(order)

    def get_num_rows(self):
        return self._graph._CAPI_get_num_rows()

    def get_num_cols(self):
        return self._graph._CAPI_get_num_cols()

    def to_block(self) -> Block:
        frontier, num_row, num_col, t1, t2, e_ids, fmt = self._graph._CAPI_relabel()
        data = self._graph._CAPI_get_data("default")
        if data is not None and e_ids is not None:
            data = data[e_ids]
        return Block(fmt, t1, t2, num_row, num_col, frontier, e_ids, data)

    to_dgl_block = to_block

    def columnwise_slicing(self, t):
        return Matrix(self._graph._CAPI_slicing(t, 0, _CSC, _COO, False))

    def columnwise_sampling(self, fanout, replace=True, bias=None):
        if bias is None:
            return Matrix(self._graph._CAPI_sampling(0, fanout, replace, _CSC, _COO))
        return Matrix(self._graph._CAPI_sampling_with_probs(0, bias, fanout, replace, _CSC, _COO))

    def sum(self, axis, powk=1) -> torch.Tensor:
        return self._graph._CAPI_sum(axis, powk, _CSC if axis == 0 else _CSR)

    def divide(self, divisor, axis):
        return Matrix(self._graph._CAPI_divide(divisor, axis, _COO))

    def normalize(self, axis):
        return Matrix(self._graph._CAPI_normalize(axis, _CSC if axis == 0 else _CSR))

    def row_ids(self, remove_isolated=True, unique=None) -> torch.Tensor:
        if unique is not None:  # spelling used by the reference's examples
            remove_isolated = unique
        return self._graph._CAPI_get_valid_rows() if remove_isolated else self._graph._CAPI_get_rows()

    def all_indices(self) -> torch.Tensor:
        return self._graph._CAPI_all_valid_node()

    def row_indices(self) -> torch.Tensor:
        return self._graph._CAPI_get_coo_rows(True)

    def __getitem__(self, data):
        ret = self._graph
        r_slice, c_slice = data[0], data[1]
        if isinstance(c_slice, (torch.Tensor, torch.fx.Proxy)):
            ret = ret._CAPI_slicing(c_slice, 0, _CSC, _COO, False)
        if isinstance(r_slice, (torch.Tensor, torch.fx.Proxy)):
            ret = ret._CAPI_slicing(r_slice, 1, _CSR, _COO, False)
        return Matrix(ret)

    def fused_columnwise_slicing_sampling(self, seeds, fanouts, replace):
        return Matrix(self._graph._CAPI_fused_columnwise_slicing_sampling(seeds, fanouts, replace))

    def random_walk(self, seeds, walk_length):
        return self._graph._CAPI_random_walk(seeds, walk_length)

    def relabel(self):
        self._graph._CAPI_relabel()
        return self


class HeteroMatrix:
    """Named relations over `HeteroGraph`, method for method the reference's gs.HeteroMatrix
    (python/gs/matrix_api/hetero_matrix.py:5-30), bound to the registered
    `_CAPI_*` method names (src/pybind.cc:54-59)."""

    def __init__(self, hetero_graph=None):
        from ..graph import HeteroGraph
        self._hetero_graph = hetero_graph if hetero_graph is not None else HeteroGraph()

    def load_from_homo(self, node_types, edge_types, homo_matrices):
        self._hetero_graph._CAPI_LoadFromHomo(node_types, edge_types, [m._graph for m in homo_matrices])

    def get_homo_matrix(self, etype: str) -> Matrix:
        return Matrix(self._hetero_graph._CAPI_GetHomoGraph(etype))

    def metapath_random_walk(self, seeds, metapath):
        """One fused slice + 1-neighbour sample per relation, trace stacked step-major [len(metapath) + 1,
        num_seeds].  Every walker needs a neighbour at every step: an empty column yields no row, so
        the steps would differ in length (the fused walk carries -1 instead)."""
        ret = [seeds]
        for etype in metapath:
            sub = self.get_homo_matrix(etype).fused_columnwise_slicing_sampling(seeds, 1, True)
            seeds = sub.row_indices()
            ret.append(seeds)
        return torch.stack(ret)

    def metapath_random_walk_fused(self, seeds, metapath):
        return self._hetero_graph._CAPI_MetapathRandomWalkFused(seeds, metapath)
