"""numpy front end of the CPU checker (oracle/linf_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the CPU
baseline leg of bench.py.  The product package never imports this module.

Every function takes and returns C-contiguous numpy arrays in the reference's layout
(input [B, CI, HW], weight [CO, CI/G], output / pos / grad_output [B, CO, HW]).
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_F = ctypes.POINTER(ctypes.c_float)
_I = ctypes.POINTER(ctypes.c_int32)


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liblinf_oracle.so")
        if not os.path.exists(path):
            from . import build as _build
            _build.build_oracle()
        _LIB = ctypes.CDLL(path)
    return _LIB


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_F)


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_I)


def _dims(x, w, group):
    B, CI, HW = x.shape
    CO = w.shape[0]
    assert w.shape[1] * group == CI and CO % group == 0
    return B, CO, CI, group, HW


def inf_dist_forward(x, w, group=1):
    """Returns (y float32 [B,CO,HW], pos int32 [B,CO,HW])."""
    x, px = _f(x); w, pw = _f(w)
    B, CO, CI, G, HW = _dims(x, w, group)
    y = np.empty((B, CO, HW), np.float32); pos = np.empty((B, CO, HW), np.int32)
    _lib().oracle_inf_dist_forward(px, pw, B, CO, CI, G, HW, y.ctypes.data_as(_F), pos.ctypes.data_as(_I))
    return y, pos


def inf_dist_bound(xl, xu, w, group=1):
    """Returns (lower, upper) float32 [B,CO,HW]."""
    xl, pl = _f(xl); xu, pu = _f(xu); w, pw = _f(w)
    B, CO, CI, G, HW = _dims(xl, w, group)
    yl = np.empty((B, CO, HW), np.float32); yu = np.empty((B, CO, HW), np.float32)
    _lib().oracle_inf_dist_bound_forward(pl, pu, pw, B, CO, CI, G, HW, yl.ctypes.data_as(_F), yu.ctypes.data_as(_F))
    return yl, yu


def inf_dist_backward(grad_out, pos, CI, group=1):
    """Ordered scatter.  Returns (grad_input [B,CI,HW], grad_weight [CO,CI/G])."""
    g, pg = _f(grad_out); pos, pp = _i(pos)
    B, CO, HW = g.shape
    gx = np.empty((B, CI, HW), np.float32); gw = np.empty((CO, CI // group), np.float32)
    _lib().oracle_inf_dist_backward_input(pg, pp, B, CO, CI, group, HW, gx.ctypes.data_as(_F))
    _lib().oracle_inf_dist_backward_weight(pg, pp, B, CO, CI, group, HW, gw.ctypes.data_as(_F))
    return gx, gw


def norm_dist_forward(x, w, group, p):
    x, px = _f(x); w, pw = _f(w)
    B, CO, CI, G, HW = _dims(x, w, group)
    y = np.empty((B, CO, HW), np.float32)
    _lib().oracle_norm_dist_forward(px, pw, B, CO, CI, G, HW, ctypes.c_float(p), y.ctypes.data_as(_F))
    return y


def norm_dist_backward(grad_out, x, w, y, group, p):
    """Returns (grad_input, grad_weight) computed in double precision from fp32 inputs."""
    g, pg = _f(grad_out); x, px = _f(x); w, pw = _f(w); y, py = _f(y)
    B, CO, CI, G, HW = _dims(x, w, group)
    gx = np.empty_like(x); gw = np.empty_like(w)
    _lib().oracle_norm_dist_backward_input(pg, px, pw, py, B, CO, CI, G, HW, ctypes.c_float(p), gx.ctypes.data_as(_F))
    _lib().oracle_norm_dist_backward_weight(pg, px, pw, py, B, CO, CI, G, HW, ctypes.c_float(p), gw.ctypes.data_as(_F))
    return gx, gw
