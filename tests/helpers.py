"""Test-side helpers: C-ABI calls on torch CUDA tensors and seeded inputs."""
import ctypes
import os

import numpy as np
import torch

import linfdist_b200
from linfdist_b200 import _lib

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def stream():
    return torch.cuda.current_stream().cuda_stream


def dev(a, device="cuda:0"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def make_inputs(B, CI, CO, HW, G, seed, x_dist="uniform"):
    """Seeded CPU tensors in the reference layout: x [B,CI,HW], w [CO,CI/G], g [B,CO,HW]."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.rand(B, CI, HW, generator=gen) if x_dist == "uniform" else torch.randn(B, CI, HW, generator=gen)
    w = torch.randn(CO, CI // G, generator=gen)
    g = torch.randn(B, CO, HW, generator=gen)
    return x.numpy(), w.numpy(), g.numpy()


def c_inf_forward(x, w, G, use_ws=True):
    lib = _lib.load()
    B, CI, HW = x.shape; CO = w.shape[0]
    y = torch.empty(B, CO, HW, device=x.device); pos = torch.empty(B, CO, HW, device=x.device, dtype=torch.int32)
    need = lib.linf_inf_dist_forward_workspace_bytes(B, CO, CI, G, HW) if use_ws else 0
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        rc = lib.linf_inf_dist_forward_ws(x.data_ptr(), w.data_ptr(), B, CO, CI, G, HW, y.data_ptr(),
                                          pos.data_ptr(), ws.data_ptr(), need, stream())
    else:
        rc = lib.linf_inf_dist_forward(x.data_ptr(), w.data_ptr(), B, CO, CI, G, HW, y.data_ptr(),
                                       pos.data_ptr(), stream())
    assert rc == 0, lib.linf_error_string(rc)
    return y, pos


def c_inf_bound(lo, up, w, G):
    lib = _lib.load()
    B, CI, HW = lo.shape; CO = w.shape[0]
    yl = torch.empty(B, CO, HW, device=lo.device); yu = torch.empty_like(yl)
    rc = lib.linf_inf_dist_bound_forward(lo.data_ptr(), up.data_ptr(), w.data_ptr(), B, CO, CI, G, HW,
                                         yl.data_ptr(), yu.data_ptr(), stream())
    assert rc == 0, lib.linf_error_string(rc)
    return yl, yu


def c_inf_backward(g, pos, CI, G, mode="ordered"):
    lib = _lib.load()
    B, CO, HW = g.shape
    if mode == "ordered":
        # poison the outputs: the ordered kernels must overwrite every element
        gx = torch.full((B, CI, HW), float("nan"), device=g.device)
        gw = torch.full((CO, CI // G), float("nan"), device=g.device)
        rc = lib.linf_inf_dist_backward_input(g.data_ptr(), pos.data_ptr(), B, CO, CI, G, HW, gx.data_ptr(), stream())
        assert rc == 0, lib.linf_error_string(rc)
        rc = lib.linf_inf_dist_backward_weight(g.data_ptr(), pos.data_ptr(), B, CO, CI, G, HW, gw.data_ptr(), stream())
        assert rc == 0, lib.linf_error_string(rc)
    elif mode == "both":
        gx = torch.full((B, CI, HW), float("nan"), device=g.device)
        gw = torch.full((CO, CI // G), float("nan"), device=g.device)
        rc = lib.linf_inf_dist_backward(g.data_ptr(), pos.data_ptr(), B, CO, CI, G, HW, gx.data_ptr(), gw.data_ptr(), stream())
        assert rc == 0, lib.linf_error_string(rc)
    else:
        gx = torch.zeros(B, CI, HW, device=g.device); gw = torch.zeros(CO, CI // G, device=g.device)
        rc = lib.linf_inf_dist_backward_atomic(g.data_ptr(), pos.data_ptr(), B, CO, CI, G, HW,
                                               gx.data_ptr(), gw.data_ptr(), stream())
        assert rc == 0, lib.linf_error_string(rc)
    return gx, gw


def c_lp_forward(x, w, G, p):
    lib = _lib.load()
    B, CI, HW = x.shape; CO = w.shape[0]
    y = torch.empty(B, CO, HW, device=x.device)
    rc = lib.linf_norm_dist_forward(x.data_ptr(), w.data_ptr(), B, CO, CI, G, HW, y.data_ptr(), float(p), stream())
    assert rc == 0, lib.linf_error_string(rc)
    return y


def c_lp_backward(g, x, w, y, G, p):
    lib = _lib.load()
    B, CI, HW = x.shape; CO = w.shape[0]
    gx = torch.full_like(x, float("nan")); gw = torch.full_like(w, float("nan"))
    rc = lib.linf_norm_dist_backward_input(g.data_ptr(), x.data_ptr(), w.data_ptr(), y.data_ptr(),
                                           B, CO, CI, G, HW, gx.data_ptr(), float(p), stream())
    assert rc == 0, lib.linf_error_string(rc)
    rc = lib.linf_norm_dist_backward_weight(g.data_ptr(), x.data_ptr(), w.data_ptr(), y.data_ptr(),
                                            B, CO, CI, G, HW, gw.data_ptr(), float(p), stream())
    assert rc == 0, lib.linf_error_string(rc)
    return gx, gw


def bits(a):
    """float32 array -> uint32 view, for bit-exact comparison (distinguishes -0 from +0)."""
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bits_equal(a, b, what):
    a = a.detach().cpu().numpy() if torch.is_tensor(a) else np.asarray(a)
    b = b.detach().cpu().numpy() if torch.is_tensor(b) else np.asarray(b)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    if a.dtype == np.float32:
        bad = bits(a) != bits(b)
    else:
        bad = a != b
    n = int(bad.sum())
    if n:
        idx = np.argwhere(bad)[:5]
        raise AssertionError(f"{what}: {n} of {a.size} elements differ, first at {idx.tolist()}: "
                             f"{[a[tuple(i)] for i in idx]} vs {[b[tuple(i)] for i in idx]}")


# Tolerance of the finite-p path (stated by the task: 1e-5 relative).  Forward values are
# compared elementwise (floor=0).  Gradient entries are signed sums with cancellation -- an entry
# near zero still carries the rounding of terms as large as the largest entry -- so their error
# is measured against the largest entry of the tensor: |a - b| <= LP_RTOL * max|b| (floor=1).
# For scale: the reference's own fp32 PyTorch branch sits 6e-7 (p=8), 1e-6 (p=16), 3.5e-6 (p=64)
# from double precision under this measure, and up to 2e-4 on individual small entries.
# Two more measures are REPORTED for every gradient comparison (and collected in LP_REPORT): the
# mixed one, |a - b| / max(|b|, 1e-2 * max|b|), and the plain elementwise one over the entries
# with |b| >= 1e-3 * max|b|.
LP_RTOL = 1e-5
LP_FLOOR = 1.0
LP_REPORT = []


def lp_errors(a, b):
    """(normwise, mixed with floor 1e-2, elementwise over entries >= 1e-3 of the largest) relative errors."""
    a = a.detach().cpu().numpy() if torch.is_tensor(a) else np.asarray(a)
    b = b.detach().cpu().numpy() if torch.is_tensor(b) else np.asarray(b)
    a = a.astype(np.float64); b = b.astype(np.float64)
    if b.size == 0:
        return 0.0, 0.0, 0.0
    top = max(float(np.abs(b).max()), 1e-300)
    err = np.abs(a - b)
    big = np.abs(b) >= 1e-3 * top
    return (float(err.max() / top), float((err / np.maximum(np.abs(b), 1e-2 * top)).max()),
            float((err[big] / np.abs(b[big])).max()) if big.any() else 0.0)


def assert_lp_close(a, b, what, floor=LP_FLOOR, rtol=LP_RTOL):
    a = a.detach().cpu().numpy() if torch.is_tensor(a) else np.asarray(a)
    b = b.detach().cpu().numpy() if torch.is_tensor(b) else np.asarray(b)
    a = a.astype(np.float64); b = b.astype(np.float64)
    scale = np.maximum(np.abs(b), floor * np.abs(b).max())
    err = np.abs(a - b) / np.maximum(scale, 1e-300)
    worst = float(err.max()) if err.size else 0.0
    norm, mixed, elem = lp_errors(a, b)
    LP_REPORT.append((what, norm, mixed, elem))
    print(f"[lp] {what}: normwise {norm:.2e}, mixed(floor 1e-2) {mixed:.2e}, elementwise(|b| >= 1e-3 max) {elem:.2e}")
    assert worst <= rtol, f"{what}: max scaled error {worst:.3e} > {rtol}"
    return worst
