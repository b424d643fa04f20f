"""`gs`: the Python face of the sampler, shaped like the reference's `python/gs` package
(python/gs/__init__.py): `gs.Graph`, `gs.Matrix`, `gs.ops` (g-SDDMM front end), the format flags and
`gs.utils.SeedGenerator`; `gs.gs_ops` stands in for `torch.ops.gs_ops` (list sampling and the super-batch operators).  Import as `import graph_sampling_b200.gs as gs`.

`gs.jit.compile` traces a function written against `Matrix` and rewrites it onto the fused operators.
`HeteroMatrix` and the DGL block builders of the reference are framework glue and are not provided;
`Matrix.to_block` returns a plain DGL-free block description instead of a DGL object.
"""
from ..graph import Graph, HeteroGraph, ListSampling, ListSamplingProbs, Unique, gs_ops, _COO, _CSC, _CSR, _DCSC, _DCSR
from ..ops import set_seed
from . import ops, utils
from .matrix import Block, Matrix
from . import jit

list_sampling = ListSampling
list_sampling_with_probs = ListSamplingProbs

__all__ = ["Graph", "HeteroGraph", "Matrix", "Block", "ops", "utils", "jit", "gs_ops", "set_seed", "list_sampling", "list_sampling_with_probs",
           "ListSampling", "ListSamplingProbs", "Unique", "_COO", "_CSC", "_CSR", "_DCSC", "_DCSR"]
