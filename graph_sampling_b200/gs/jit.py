"""`gs.jit.compile`: trace a sampling function written against `gs.Matrix` into a torch.fx graph of `_CAPI_*`
method calls and rewrite it so that it runs on the fused operators.  Same call convention as the reference's
`gs.jit.compile(func, args)` (python/gs/jit/module.py:84-137): `Matrix` arguments are traced through their graph
handle, list / tuple arguments (fanouts, metapaths) are frozen as constants, everything else stays an input.

Rewrites (python/gs/jit/optimize.py:7-82, python/gs/jit/passes.py:15-58 are the reference's versions):

* slicing + sampling fusion: `g._CAPI_slicing(seeds, 0, CSC, *, False)._CAPI_sampling(0, k, replace, CSC, *)`
  becomes `g._CAPI_fused_columnwise_slicing_sampling(seeds, k, replace)` when the slice has no other user and the
  sample is only used by format-agnostic methods (the fused operator yields a CSC-only graph, so `_CAPI_relabel`
  then reports "csc" instead of "coo"; `Matrix.to_block` handles both).  The reference's pass matches method
  names its tracer never produces (`_CAPI_columnwise_*`) and therefore never fires.
* `_CAPI_all_valid_node` / `_CAPI_all_indices` next to `_CAPI_relabel` on the same graph: the frontier is taken
  from the relabel result (both are unique(cat(col_ids, rows)) in first-occurrence order).
* common-subexpression elimination for deterministic methods only (two sampling calls with equal arguments are two
  samples and stay two calls), and dead-code elimination that keeps methods with side effects.

Tracing runs no kernel and needs no GPU.
"""
import operator

import torch
import torch.fx as fx

from ..graph import _COO, _CSC
from .matrix import Matrix

_FRONTIER = ("_CAPI_all_valid_node", "_CAPI_all_indices", "_CAPI_AllValidNode")
_RELABEL = ("_CAPI_relabel", "_CAPI_Relabel")
_SLICING = ("_CAPI_slicing", "_CAPI_Slicing")
_SAMPLING = ("_CAPI_sampling", "_CAPI_Sampling")
# methods whose result does not depend on which sparse formats the graph object currently holds
_FORMAT_AGNOSTIC = set(_FRONTIER + _RELABEL) | {
    "_CAPI_get_coo_rows", "_CAPI_get_coo_cols", "_CAPI_GetCOORows", "_CAPI_GetCooCols", "_CAPI_get_rows",
    "_CAPI_get_cols", "_CAPI_GetRows", "_CAPI_GetCols", "_CAPI_get_valid_rows", "_CAPI_get_valid_cols",
    "_CAPI_GetValidRows", "_CAPI_GetValidCols", "_CAPI_get_num_rows", "_CAPI_get_num_cols", "_CAPI_get_num_edges",
    "_CAPI_GetNumRows", "_CAPI_GetNumCols", "_CAPI_GetNumEdges", "_CAPI_get_data", "_CAPI_GetData"}
# methods that draw random numbers (never merged) or change their receiver / an argument (never removed)
_STOCHASTIC = {"_CAPI_sampling", "_CAPI_Sampling", "_CAPI_sampling_with_probs", "_CAPI_SamplingWithProbs",
               "_CAPI_fused_columnwise_slicing_sampling", "_CAPI_FusedColumnwiseSlicingSampling", "_CAPI_random_walk",
               "_CAPI_RandomWalk", "_CAPI_metapath_random_walk_fused", "_CAPI_MetapathRandomWalkFused",
               "list_sampling", "list_sampling_with_probs", "ListSampling", "ListSamplingProbs"}
_SIDE_EFFECTS = {"_CAPI_set_data", "_CAPI_SetData", "_CAPI_sddmm", "_CAPI_SDDMM", "_CAPI_load_csc", "_CAPI_LoadCSC",
                 "_CAPI_load_coo", "_CAPI_LoadCOO", "_CAPI_set_coo", "_CAPI_SetCOO", "_CAPI_set_metadata",
                 "_CAPI_SetMetadata", "_CAPI_decode", "_CAPI_Decode"}


class _Tracer(fx.Tracer):
    """Matrix values that reach an operator argument or the output are carried as `Matrix(graph handle)` nodes."""

    def create_arg(self, a):
        if isinstance(a, Matrix):
            return self.create_proxy("call_function", Matrix, (a._graph,), {}).node
        return super().create_arg(a)


def _flat_nodes(x):
    if isinstance(x, fx.Node):
        yield x
    elif isinstance(x, (list, tuple)):
        for y in x:
            yield from _flat_nodes(y)
    elif isinstance(x, dict):
        for y in x.values():
            yield from _flat_nodes(y)


def _name(node):
    """Method / function name a node calls, or None."""
    if node.op == "call_method":
        return node.target
    if node.op == "call_function":
        return getattr(node.target, "__name__", None)
    return None


def dce(gm: fx.GraphModule) -> fx.GraphModule:
    """Removes nodes nothing depends on; inputs, the output and methods with side effects are roots."""
    live = set()
    for node in reversed(list(gm.graph.nodes)):
        if node.op in ("output", "placeholder") or _name(node) in _SIDE_EFFECTS:
            live.add(node)
        if node in live:
            live.update(_flat_nodes(node.args))
            live.update(_flat_nodes(node.kwargs))
    for node in reversed(list(gm.graph.nodes)):
        if node not in live:
            gm.graph.erase_node(node)
    gm.graph.lint()
    gm.recompile()
    return gm


def cse(gm: fx.GraphModule) -> fx.GraphModule:
    """Merges repeated deterministic calls with identical arguments."""
    seen = {}
    dirty = set()   # graph handles that a side-effecting method has touched: later calls on them are not merged
    for node in list(gm.graph.nodes):
        name = _name(node)
        if name in _SIDE_EFFECTS:
            dirty.update(_flat_nodes(node.args))
            continue
        if node.op not in ("call_method", "call_function") or name in _STOCHASTIC:
            continue
        if any(a in dirty for a in _flat_nodes(node.args)):
            continue
        key = (node.op, str(node.target), str(node.args), str(node.kwargs))
        if key in seen:
            node.replace_all_uses_with(seen[key])
            gm.graph.erase_node(node)
        else:
            seen[key] = node
    gm.graph.lint()
    gm.recompile()
    return gm


def merge_relabel_and_all_indices(gm: fx.GraphModule) -> fx.GraphModule:
    """`g.all_valid_node()` next to `g.relabel()`: one relabel call serves both."""
    by_graph = {}
    for node in gm.graph.nodes:
        if node.op == "call_method" and (node.target in _FRONTIER or node.target in _RELABEL):
            by_graph.setdefault(node.args[0], []).append(node)
    for users in by_graph.values():
        relabels = [u for u in users if u.target in _RELABEL]
        frontiers = [u for u in users if u.target in _FRONTIER]
        if not relabels or not frontiers:
            continue
        first = min(users, key=lambda u: list(gm.graph.nodes).index(u))
        with gm.graph.inserting_before(first):
            merged = gm.graph.node_copy(relabels[0])
            frontier = gm.graph.call_function(operator.getitem, args=(merged, 0))
        for u in frontiers:
            u.replace_all_uses_with(frontier)
        for u in relabels:
            u.replace_all_uses_with(merged)
    return dce(gm)


def fuse_slicing_and_sampling(gm: fx.GraphModule) -> fx.GraphModule:
    """Column slice followed by column-wise uniform sampling → the fused operator."""
    for node in list(gm.graph.nodes):
        if not (node.op == "call_method" and node.target in _SAMPLING and len(node.args) == 6):
            continue
        src = node.args[0]
        if not (isinstance(src, fx.Node) and src.op == "call_method" and src.target in _SLICING and len(src.args) == 6):
            continue
        _, seeds, s_axis, s_on, _, s_relabel = src.args
        _, axis, fanout, replace, on_format, _ = node.args
        if (s_axis, s_on, s_relabel) != (0, _CSC, False) or (axis, on_format) != (0, _CSC):
            continue
        if len(src.users) != 1:
            continue
        users_ok = all((u.op == "call_method" and u.target in _FORMAT_AGNOSTIC) or
                       (u.op == "call_function" and u.target is Matrix) or u.op == "output" for u in node.users)
        if not users_ok:
            continue
        # Matrix(...) wrappers only forward the handle; look one level further
        if any(u.op == "call_function" and u.target is Matrix and
               any(not (w.op == "output" or (w.op == "call_method" and w.target in _FORMAT_AGNOSTIC)) for w in u.users)
               for u in node.users):
            continue
        with gm.graph.inserting_after(node):
            fused = gm.graph.call_method("_CAPI_fused_columnwise_slicing_sampling",
                                         args=(src.args[0], seeds, fanout, replace))
        node.replace_all_uses_with(fused)
    return dce(gm)


class compile:  # noqa: N801  (the reference's name)
    """compiled = gs.jit.compile(func, args); compiled(*args) runs the rewritten graph."""

    def __init__(self, func, args, fuse_slicing_sampling=True):
        self._kinds = []
        statics = {}
        for i, a in enumerate(args):
            if isinstance(a, Matrix):
                self._kinds.append("graph")
            elif isinstance(a, (list, tuple)) and not any(isinstance(x, torch.Tensor) for x in a):
                self._kinds.append("static")
                statics[i] = a
            else:
                self._kinds.append("dynamic")
        kinds = self._kinds

        def traced(dynamic_args, graph_args):
            rebuilt, d, g = [], 0, 0
            for i, kind in enumerate(kinds):
                if kind == "graph":
                    rebuilt.append(Matrix(graph_args[g]))
                    g += 1
                elif kind == "static":
                    rebuilt.append(statics[i])
                else:
                    rebuilt.append(dynamic_args[d])
                    d += 1
            return func(*rebuilt)

        traced.__name__ = getattr(func, "__name__", "sampler")
        tracer = _Tracer()
        graph = tracer.trace(traced)
        gm = fx.GraphModule(tracer.root, graph, traced.__name__)
        gm = merge_relabel_and_all_indices(gm)
        if fuse_slicing_sampling:
            gm = fuse_slicing_and_sampling(gm)
        gm = cse(gm)
        self.gm = dce(gm)

    def __call__(self, *args):
        if len(args) != len(self._kinds):
            raise TypeError(f"expected {len(self._kinds)} arguments, got {len(args)}")
        dynamic = tuple(a for a, k in zip(args, self._kinds) if k == "dynamic")
        graphs = tuple(a._graph for a, k in zip(args, self._kinds) if k == "graph")
        return self.gm(dynamic, graphs)

    def targets(self):
        """Names of the operators the compiled graph calls, in order (for inspection and tests)."""
        return [n.target if n.op == "call_method" else getattr(n.target, "__name__", str(n.target))
                for n in self.gm.graph.nodes if n.op in ("call_method", "call_function")]
