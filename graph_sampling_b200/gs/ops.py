"""g-SDDMM front end: shape inference, scalar-feature handling and the sub -> add(-rhs),
div -> mul(1/rhs) rewrites of the reference (python/gs/ops/sparse.py:56-129,
python/gs/ops/sddmm.py:35-131), plus the generated u_add_v ... e_dot_v helpers."""
import sys
from itertools import product

import torch

from ..graph import _COO

target_mapping = {"u": 0, "e": 1, "v": 2, "src": 0, "edge": 1, "dst": 2}


def infer_broadcast_shape(op, shp1, shp2):
    pad1, pad2 = tuple(shp1), tuple(shp2)
    if op == "dot" and shp1[-1] != shp2[-1]:
        raise ValueError(f"dot needs the same size on the last dimension, got {shp1} and {shp2}")
    if len(pad1) > len(pad2):
        pad2 = (1,) * (len(pad1) - len(pad2)) + pad2
    elif len(pad1) < len(pad2):
        pad1 = (1,) * (len(pad2) - len(pad1)) + pad1
    for d1, d2 in zip(pad1, pad2):
        if d1 != d2 and d1 != 1 and d2 != 1:
            raise ValueError(f"feature shapes {shp1} and {shp2} are not valid for broadcasting")
    rst = tuple(max(d1, d2) for d1, d2 in zip(pad1, pad2))
    return rst[:-1] + (1,) if op == "dot" else rst


def _gsddmm(gidx, op, lhs, rhs, lhs_target="u", rhs_target="v", on_format=_COO):
    if lhs.device != rhs.device:
        raise ValueError(f"operand devices differ: {lhs.device} and {rhs.device}")
    if lhs.dtype != rhs.dtype:
        raise ValueError(f"operand dtypes differ: {lhs.dtype} and {rhs.dtype}")
    expand_lhs = expand_rhs = False
    if lhs.dim() == 1:
        lhs, expand_lhs = lhs.unsqueeze(-1), True
    if rhs.dim() == 1:
        rhs, expand_rhs = rhs.unsqueeze(-1), True
    lt, rt = target_mapping[lhs_target], target_mapping[rhs_target]
    n_edges = gidx._CAPI_get_num_edges()
    out = torch.zeros((n_edges,) + infer_broadcast_shape(op, lhs.shape[1:], rhs.shape[1:]), dtype=lhs.dtype,
                      device=lhs.device)
    if n_edges > 0:
        gidx._CAPI_sddmm(op, lhs.contiguous(), rhs.contiguous(), out, lt, rt, on_format)
    if expand_lhs and expand_rhs:
        out = out.squeeze(-1)
    return out


def gsddmm_internal(gidx, op, lhs_data, rhs_data, lhs_target="u", rhs_target="v", on_format=_COO):
    if op == "sub":
        op, rhs_data = "add", -rhs_data
    if op == "div":
        op, rhs_data = "mul", 1.0 / rhs_data
    return _gsddmm(gidx, op, lhs_data, rhs_data, lhs_target, rhs_target, on_format)


def reshape_lhs_rhs(lhs_data, rhs_data):
    ls, rs = lhs_data.shape, rhs_data.shape
    if len(ls) != len(rs):
        nd = max(len(ls), len(rs))
        lhs_data = lhs_data.view((ls[0],) + (1,) * (nd - len(ls)) + tuple(ls[1:]))
        rhs_data = rhs_data.view((rs[0],) + (1,) * (nd - len(rs)) + tuple(rs[1:]))
    return lhs_data, rhs_data


def gsddmm(g, op, lhs_data, rhs_data, lhs_target="u", rhs_target="v", on_format=_COO):
    """x_e = op(x_lhs, x_rhs) for every edge of the gs.Matrix `g`."""
    lhs_data, rhs_data = reshape_lhs_rhs(lhs_data, rhs_data)
    return gsddmm_internal(g._graph, op, lhs_data, rhs_data, lhs_target, rhs_target, on_format)


__all__ = ["gsddmm", "gsddmm_internal", "infer_broadcast_shape"]


def _register():
    for lhs, rhs in product("uve", "uve"):
        if lhs == rhs:
            continue
        for binary_op in ("add", "sub", "mul", "div", "dot"):
            def func(g, x, y, on_format=_COO, _l=lhs, _r=rhs, _o=binary_op):
                return gsddmm(g, _o, x, y, lhs_target=_l, rhs_target=_r, on_format=on_format)
            func.__name__ = f"{lhs}_{binary_op}_{rhs}"
            func.__doc__ = f"Edge feature = {binary_op}({lhs} feature, {rhs} feature) with NumPy broadcasting."
            setattr(sys.modules[__name__], func.__name__, func)
            __all__.append(func.__name__)


_register()
