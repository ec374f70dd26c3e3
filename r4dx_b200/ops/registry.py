"""The kernel registry of the native library as Python data: which entry point implements which operation, on which
engine, under which geometry constraints (reference: third_party/libr4d/r4d.h:523-560 exposes the same kind of table).

    from r4dx_b200.ops import registry
    registry.kernels()                                  # list of dicts
    registry.covering("trellis_linear_rows_ge_16", N=5120, K=17408, kb=4)   # names of the kernels whose constraints hold
"""
from __future__ import annotations

import ctypes
from typing import Dict, List

from .. import native

_OPS = {0: "==", 1: "<=", 2: ">=", 3: "% == 0", 4: "in"}


class _Constraint(ctypes.Structure):
    _fields_ = [("key", ctypes.c_char_p), ("op", ctypes.c_int), ("ival", ctypes.c_longlong), ("sval", ctypes.c_char_p)]


class _Info(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("family", ctypes.c_char_p), ("op", ctypes.c_char_p), ("computes", ctypes.c_char_p),
                ("shape", ctypes.c_char_p), ("dtypes", ctypes.c_char_p), ("engine", ctypes.c_char_p),
                ("constraints", ctypes.POINTER(_Constraint)), ("n_constraints", ctypes.c_int)]


def _lib():
    L = native.host()
    L.r4dxb_kernel_count.restype = ctypes.c_int
    L.r4dxb_kernel_at.restype = ctypes.POINTER(_Info)
    L.r4dxb_kernel_at.argtypes = [ctypes.c_int]
    L.r4dxb_kernel_covers.restype = ctypes.c_int
    L.r4dxb_kernel_covers.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_longlong), ctypes.c_int]
    return L


def kernels() -> List[Dict[str, object]]:
    L = _lib()
    out = []
    for i in range(L.r4dxb_kernel_count()):
        k = L.r4dxb_kernel_at(i).contents
        cons = []
        for c in range(k.n_constraints):
            cc = k.constraints[c]
            cons.append({"key": cc.key.decode(), "op": _OPS[cc.op], "value": ([int(w) for w in cc.sval.decode().split()] if cc.op == 4 else int(cc.ival))})
        out.append({"name": k.name.decode(), "family": k.family.decode(), "op": k.op.decode(), "computes": k.computes.decode(),
                    "shape": k.shape.decode(), "dtypes": k.dtypes.decode(), "engine": k.engine.decode(), "constraints": cons})
    return out


def covers(name: str, **geometry: int) -> bool:
    """True when no constraint of kernel ``name`` on the given parameters fails (necessary, not sufficient)."""
    L = _lib()
    keys = (ctypes.c_char_p * len(geometry))(*[k.encode() for k in geometry])
    vals = (ctypes.c_longlong * len(geometry))(*[int(v) for v in geometry.values()])
    r = L.r4dxb_kernel_covers(name.encode(), keys, vals, len(geometry))
    if r < 0:
        raise KeyError(name)
    return r == 1


def covering(op: str, **geometry: int) -> List[str]:
    """Names of the kernels that implement ``op`` and whose constraints hold for the geometry."""
    return [k["name"] for k in kernels() if k["op"] == op and covers(k["name"], **geometry)]
