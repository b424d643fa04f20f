"""`gs`: the Python face of the sampler, shaped like the reference's `python/gs` package
(python/gs/__init__.py): `gs.Graph`, `gs.Matrix`, `gs.ops` (g-SDDMM front end), the format flags and
`gs.utils.SeedGenerator`; `gs.gs_ops` stands in for `torch.ops.gs_ops` (list sampling and the super-batch operators).  Import as `import graph_sampling_b200.gs as gs`.

`gs.jit.compile` traces a function written against `Matrix` and rewrites it onto the fused operators.
`gs.HeteroMatrix` wraps `HeteroGraph` as the reference's does.  `Matrix.to_block` and
`gs.utils.create_block_from_{csc,coo}` return a plain DGL-free `Block`; with DGL importable the two
builders hand the same fields to DGL as the reference does.
"""
from ..graph import Graph, HeteroGraph, ListSampling, ListSamplingProbs, Unique, gs_ops, _COO, _CSC, _CSR, _DCSC, _DCSR
from ..ops import set_seed
from . import ops, utils
from .matrix import Block, HeteroMatrix, Matrix
from . import jit

list_sampling = ListSampling
list_sampling_with_probs = ListSamplingProbs

__all__ = ["Graph", "HeteroGraph", "Matrix", "HeteroMatrix", "Block", "ops", "utils", "jit", "gs_ops", "set_seed", "list_sampling", "list_sampling_with_probs",
           "ListSampling", "ListSamplingProbs", "Unique", "_COO", "_CSC", "_CSR", "_DCSC", "_DCSR"]
