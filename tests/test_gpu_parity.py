"""GPU parity: the CUDA library, called through its C ABI, against the CPU oracle on the same
seeded inputs, against the golden fixtures of the reference's PyTorch branch, and (when the
prebuilt library is present) against the reference's own CUDA kernels."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import ROOT
from helpers import (GOLDEN, assert_bits_equal, assert_lp_close, c_inf_backward, c_inf_bound,
                     c_inf_forward, c_lp_backward, c_lp_forward, dev, make_inputs)

pytestmark = pytest.mark.gpu

# (B, CI, CO, HW, G): tiny and ragged shapes (generic path), dense aligned shapes (tiled path,
# with and without k-splitting), grouped and conv-shaped ones.
SHAPES = [
    (1, 1, 1, 1, 1), (1, 15, 1, 1, 1), (1, 16, 10, 1, 1), (1, 17, 17, 1, 1), (7, 17, 10, 1, 1),
    (3, 18, 12, 5, 3), (2, 8, 6, 4, 2), (5, 784, 10, 1, 1), (6, 32, 48, 1, 4),
    (33, 100, 65, 1, 1), (64, 128, 128, 1, 1), (130, 784, 200, 1, 1), (16, 64, 256, 1, 4),
    (70, 36, 300, 1, 1), (9, 3072, 129, 1, 1), (4, 27, 32, 9, 1), (200, 20, 1000, 1, 1),
    # few output channels: lanes split the reduction (classifier layer 5120 -> 10 and neighbours)
    (37, 5120, 10, 1, 1), (5, 256, 3, 1, 1), (11, 512, 31, 1, 1), (6, 1024, 40, 1, 4), (3, 128, 17, 1, 1),
]


def _ids(s):
    return "B{}_CI{}_CO{}_HW{}_G{}".format(*s)


@pytest.mark.parametrize("shape", SHAPES, ids=_ids)
@pytest.mark.parametrize("use_ws", [True, False], ids=["ws", "nows"])
def test_inf_forward_bit_exact(cuda, lib, shape, use_ws):
    B, CI, CO, HW, G = shape
    x, w, _ = make_inputs(B, CI, CO, HW, G, seed=100 + B + CI)
    y_ref, pos_ref = oracle.inf_dist_forward(x, w, G)
    y, pos = c_inf_forward(dev(x), dev(w), G, use_ws=use_ws)
    assert_bits_equal(y, y_ref, "values")
    assert_bits_equal(pos, pos_ref, "arg-max")


@pytest.mark.parametrize("shape", SHAPES, ids=_ids)
def test_inf_forward_quantised_inputs_many_ties(cuda, lib, shape):
    """Inputs on a coarse grid produce many exactly tied maxima: the lowest index must win."""
    B, CI, CO, HW, G = shape
    rng = np.random.default_rng(7)
    x = rng.integers(0, 4, (B, CI, HW)).astype(np.float32)
    w = rng.integers(0, 4, (CO, CI // G)).astype(np.float32)
    y_ref, pos_ref = oracle.inf_dist_forward(x, w, G)
    y, pos = c_inf_forward(dev(x), dev(w), G)
    assert_bits_equal(y, y_ref, "values")
    assert_bits_equal(pos, pos_ref, "arg-max")


def test_inf_forward_special_values(cuda, lib):
    B, CI, CO = 70, 64, 130
    x, w, _ = make_inputs(B, CI, CO, 1, 1, seed=5)
    x[0, :, 0] = w[0]                  # all-zero differences against output 0
    x[1, 3, 0] = np.nan                # NaN terms are skipped
    x[2, 5, 0] = np.inf
    w[7, 9] = -np.inf
    x[3, :, 0] = 1e-42                 # subnormals survive (no flush to zero)
    w[11] = 3e-42
    y_ref, pos_ref = oracle.inf_dist_forward(x, w, 1)
    y, pos = c_inf_forward(dev(x), dev(w), 1)
    assert_bits_equal(y, y_ref, "values")
    assert_bits_equal(pos, pos_ref, "arg-max")
    assert y_ref[0, 0, 0] == 0 and pos_ref[0, 0, 0] == 0
    assert 0 < y_ref[3, 11, 0] < 1e-38


def test_inf_forward_config1_full_size(cuda, lib):
    """B=512, Din=784, Dout=5120 (x ~ U[0,1), w ~ N(0,1)): values and arg-max bit-exact."""
    x, w, g = make_inputs(512, 784, 5120, 1, 1, seed=2020)
    y_ref, pos_ref = oracle.inf_dist_forward(x, w, 1)
    for use_ws in (True, False):
        y, pos = c_inf_forward(dev(x), dev(w), 1, use_ws=use_ws)
        assert_bits_equal(y, y_ref, "values")
        assert_bits_equal(pos, pos_ref, "arg-max")
    assert lib.linf_tune_set(2, 0) == 0          # no bounded wait of the TMA loader has ever run out
    gx_ref, gw_ref = oracle.inf_dist_backward(g, pos_ref, 784, 1)
    gx, gw = c_inf_backward(dev(g), dev(pos_ref), 784, 1, "ordered")
    assert_bits_equal(gx, gx_ref, "grad_input"); assert_bits_equal(gw, gw_ref, "grad_weight")
    gx2, gw2 = c_inf_backward(dev(g), dev(pos_ref), 784, 1, "ordered")
    assert_bits_equal(gx2, gx, "grad_input run-to-run"); assert_bits_equal(gw2, gw, "grad_weight run-to-run")
    gxa, gwa = c_inf_backward(dev(g), dev(pos_ref), 784, 1, "atomic")
    np.testing.assert_allclose(gxa.cpu().numpy(), gx_ref, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(gwa.cpu().numpy(), gw_ref, rtol=1e-4, atol=2e-4)


@pytest.mark.parametrize("shape", SHAPES, ids=_ids)
def test_inf_backward(cuda, lib, shape):
    B, CI, CO, HW, G = shape
    x, w, g = make_inputs(B, CI, CO, HW, G, seed=300 + B + CO)
    _, pos = oracle.inf_dist_forward(x, w, G)
    gx_ref, gw_ref = oracle.inf_dist_backward(g, pos, CI, G)
    gx, gw = c_inf_backward(dev(g), dev(pos), CI, G, "ordered")
    assert_bits_equal(gx, gx_ref, "ordered grad_input"); assert_bits_equal(gw, gw_ref, "ordered grad_weight")
    gxb, gwb = c_inf_backward(dev(g), dev(pos), CI, G, "both")
    assert_bits_equal(gxb, gx_ref, "side-by-side grad_input"); assert_bits_equal(gwb, gw_ref, "side-by-side grad_weight")
    gxa, gwa = c_inf_backward(dev(g), dev(pos), CI, G, "atomic")
    np.testing.assert_allclose(gxa.cpu().numpy(), gx_ref, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(gwa.cpu().numpy(), gw_ref, rtol=1e-4, atol=1e-4)


def test_inf_backward_atomic_exact_when_sums_are_exact(cuda, lib):
    """With small-integer gradients every partial sum is exact, so any order gives the same bits."""
    B, CI, CO = 64, 40, 96
    x, w, _ = make_inputs(B, CI, CO, 1, 1, seed=11)
    g = np.random.default_rng(3).integers(-8, 9, (B, CO, 1)).astype(np.float32)
    _, pos = oracle.inf_dist_forward(x, w, 1)
    gx_ref, gw_ref = oracle.inf_dist_backward(g, pos, CI, 1)
    gxa, gwa = c_inf_backward(dev(g), dev(pos), CI, 1, "atomic")
    assert np.array_equal(gxa.cpu().numpy(), gx_ref) and np.array_equal(gwa.cpu().numpy(), gw_ref)


BOUND_SHAPES = SHAPES + [(512, 3072, 256, 1, 1), (64, 3072, 512, 1, 4)]


@pytest.mark.parametrize("shape", BOUND_SHAPES, ids=_ids)
def test_inf_bound_bit_exact(cuda, lib, shape):
    B, CI, CO, HW, G = shape
    x, w, _ = make_inputs(B, CI, CO, HW, G, seed=500 + CI)
    eps = np.float32(8.0 / 255.0)
    lo = np.clip(x - eps, 0, 1).astype(np.float32); up = np.clip(x + eps, 0, 1).astype(np.float32)
    yl_ref, yu_ref = oracle.inf_dist_bound(lo, up, w, G)
    yl, yu = c_inf_bound(dev(lo), dev(up), dev(w), G)
    assert_bits_equal(yl, yl_ref, "lower"); assert_bits_equal(yu, yu_ref, "upper")
    assert (yl_ref <= yu_ref).all()


@pytest.mark.parametrize("CI", [64, 2048], ids=["short_rows", "rows_split_over_two_ctas"])
@pytest.mark.parametrize("kind", ["swapped", "nan", "inf", "degenerate"])
def test_inf_bound_irregular_inputs(cuda, lib, kind, CI):
    """lower > upper, NaN and infinities leave the fast rule's domain: the result must still be
    the literal rule's, bit for bit (also when two CTAs share a tile's reduction and merge in memory)."""
    B, CO = 130, 200
    x, w, _ = make_inputs(B, CI, CO, 1, 1, seed=77)
    lo = (x - 0.05).astype(np.float32); up = (x + 0.05).astype(np.float32)
    if kind == "swapped":
        lo[5, 7, 0], up[5, 7, 0] = up[5, 7, 0], lo[5, 7, 0]
        lo[100, :, 0], up[100, :, 0] = up[100, :, 0].copy(), lo[100, :, 0].copy()
    elif kind == "nan":
        lo[3, 2, 0] = np.nan; up[70, 9, 0] = np.nan; w[4, 4] = np.nan
    elif kind == "inf":
        up[1, 1, 0] = np.inf; lo[66, 3, 0] = -np.inf; w[9, 0] = np.inf; w[10, 1] = -np.inf
    else:
        up[:] = lo                      # zero-width intervals
        w[0] = lo[0, :, 0]              # and a weight row equal to an input row
    yl_ref, yu_ref = oracle.inf_dist_bound(lo, up, w, 1)
    yl, yu = c_inf_bound(dev(lo), dev(up), dev(w), 1)
    assert_bits_equal(yl, yl_ref, "lower"); assert_bits_equal(yu, yu_ref, "upper")


LP_SHAPES = [(1, 1, 1, 1, 1), (7, 17, 10, 1, 1), (3, 18, 12, 5, 3), (6, 32, 48, 1, 4),
             (33, 100, 65, 1, 1), (64, 128, 128, 1, 1), (40, 784, 96, 1, 1),
             # few outputs per group, long rows: the forward spreads the reduction over a CTA
             (70, 2048, 10, 1, 1), (33, 512, 24, 1, 2), (9, 1024, 3, 1, 1), (5, 640, 31, 1, 1)]


@pytest.mark.parametrize("shape", LP_SHAPES, ids=_ids)
@pytest.mark.parametrize("p", [8.0, 16.0, 64.0, 11.3, 1.5, 333.25])
def test_lp_against_oracle(cuda, lib, shape, p):
    B, CI, CO, HW, G = shape
    x, w, g = make_inputs(B, CI, CO, HW, G, seed=900 + CI, x_dist="normal")
    y_ref = oracle.norm_dist_forward(x, w, G, p)
    y = c_lp_forward(dev(x), dev(w), G, p)
    assert_lp_close(y, y_ref, "forward", floor=0.0)
    # gradients from the SAME fp32 output, so only the backward arithmetic is compared
    gx_ref, gw_ref = oracle.norm_dist_backward(g, x, w, y_ref, G, p)
    gx, gw = c_lp_backward(dev(g), dev(x), dev(w), dev(y_ref), G, p)
    # beyond p = 64 the rounding of |t|/y alone, amplified by p - 1, exceeds 1e-5
    rtol = 1e-5 if p <= 64 else 1e-5 * p / 64
    assert_lp_close(gx, gx_ref, "grad_input", rtol=rtol)
    assert_lp_close(gw, gw_ref, "grad_weight", rtol=rtol)


@pytest.mark.parametrize("shape", [(64, 128, 128, 1, 1), (40, 784, 96, 1, 1), (70, 256, 100, 1, 1), (130, 64, 52, 1, 1),
                                   (33, 128, 192, 1, 4)], ids=_ids)
@pytest.mark.parametrize("p", [8.0, 64.0, 11.3])
def test_lp_forward_tile_widths(cuda, lib, shape, p):
    """The finite-p forward picks 64- or 48-wide output tiles by the shape.  Every output is summed over the inputs
    in the same order either way: forced to one width or the other the bits are the same, and they agree with the
    checker."""
    B, CI, CO, HW, G = shape
    x, w, _ = make_inputs(B, CI, CO, HW, G, seed=1200 + CO, x_dist="normal")
    y_ref = oracle.norm_dist_forward(x, w, G, p)
    ys = []
    try:
        for width in (1, 2):
            assert lib.linf_tune_set(6, width) == 0
            ys.append(c_lp_forward(dev(x), dev(w), G, p))
    finally:
        lib.linf_tune_set(6, 0)
    assert_bits_equal(ys[0], ys[1].cpu().numpy(), "48-wide against 64-wide tiles")
    assert_lp_close(ys[1], y_ref, "forward, 48-wide tiles", floor=0.0)


def test_lp_against_golden(cuda, lib):
    z = np.load(os.path.join(GOLDEN, "lp.npz"))
    cases = sorted({k.split("_")[0] for k in z.files if k.startswith("c")})
    for c in cases:
        G = int(z[c + "_shape"][4])
        x, w, g = z[c + "_x"], z[c + "_w"], z[c + "_g"]
        for p in (8.0, 16.0, 64.0):
            tag = f"{c}_p{p:g}"
            y = c_lp_forward(dev(x), dev(w), G, p)
            assert_lp_close(y, z[tag + "_y"], f"forward {tag}", floor=0.0)
            gx, gw = c_lp_backward(dev(g), dev(x), dev(w), y, G, p)
            assert_lp_close(gx, z[tag + "_gx"], f"grad_input {tag}")
            assert_lp_close(gw, z[tag + "_gw"], f"grad_weight {tag}")


def test_golden_inf_and_bound(cuda, lib):
    z = np.load(os.path.join(GOLDEN, "inf_forward.npz"))
    for c in sorted({k.split("_")[0] for k in z.files}):
        G = int(z[c + "_shape"][4])
        y, _ = c_inf_forward(dev(z[c + "_x"]), dev(z[c + "_w"]), G)
        assert_bits_equal(y, z[c + "_y"], f"inf forward {c}")
    z = np.load(os.path.join(GOLDEN, "inf_bound.npz"))
    for c in sorted({k.split("_")[0] for k in z.files}):
        G = int(z[c + "_shape"][4])
        yl, yu = c_inf_bound(dev(z[c + "_lo"]), dev(z[c + "_up"]), dev(z[c + "_w"]), G)
        assert_bits_equal(yl, z[c + "_yl"], f"bound lower {c}"); assert_bits_equal(yu, z[c + "_yu"], f"bound upper {c}")


def test_lp_config2_slice_and_annealing_points(cuda, lib):
    """Din = Dout = 5120 as in config 2, on a batch slice the CPU oracle finishes in seconds."""
    B, CI, CO = 16, 5120, 5120
    x, w, g = make_inputs(B, CI, CO, 1, 1, seed=2021, x_dist="normal")
    for p in (8.0, 16.0, 64.0):
        y_ref = oracle.norm_dist_forward(x, w, 1, p)
        y = c_lp_forward(dev(x), dev(w), 1, p)
        assert_lp_close(y, y_ref, f"forward p={p}", floor=0.0)
        gx_ref, gw_ref = oracle.norm_dist_backward(g, x, w, y_ref, 1, p)
        gx, gw = c_lp_backward(dev(g), dev(x), dev(w), dev(y_ref), 1, p)
        assert_lp_close(gx, gx_ref, f"grad_input p={p}"); assert_lp_close(gw, gw_ref, f"grad_weight p={p}")


# ---- the reference's own CUDA kernels, when their prebuilt library travelled along ----------
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_norm_dist.so")


def _ref_lib():
    return ctypes.CDLL(REF_LIB) if os.path.exists(REF_LIB) else None


@pytest.mark.parametrize("p", [8.0, 16.0, 64.0])
def test_lp_config2_full_size(cuda, lib, p):
    """B = 512, Din = Dout = 5120 (x, w, grad_out ~ N(0,1)) at full size on the GPU.  The double-precision
    checker is run on samples that keep it cheap and still cover every reduction at its full length:
    forward and grad_input on 8 batch rows (they depend on that row only), grad_weight on 8 output channels
    (they depend on that channel over all 512 rows).  The whole forward is also compared with the
    reference's own CUDA kernel."""
    B, CI, CO = 512, 5120, 5120
    x, w, g = make_inputs(B, CI, CO, 1, 1, seed=2021, x_dist="normal")
    xd, wd, gd = dev(x), dev(w), dev(g)
    y = c_lp_forward(xd, wd, 1, p)
    gx, gw = c_lp_backward(gd, xd, wd, y, 1, p)
    torch.cuda.synchronize()
    yh = y.cpu().numpy()
    rng = np.random.default_rng(int(p))
    rows = np.sort(rng.choice(B, 8, replace=False)); cols = np.sort(rng.choice(CO, 8, replace=False))
    y_rows = oracle.norm_dist_forward(x[rows], w, 1, p)
    assert_lp_close(yh[rows], y_rows, f"forward rows p={p}", floor=0.0)
    # gradients from the GPU's own fp32 output, so that only the backward arithmetic is compared
    gx_rows, _ = oracle.norm_dist_backward(g[rows], x[rows], w, yh[rows], 1, p)
    assert_lp_close(gx.cpu().numpy()[rows], gx_rows, f"grad_input rows p={p}")
    _, gw_cols = oracle.norm_dist_backward(np.ascontiguousarray(g[:, cols]), x, np.ascontiguousarray(w[cols]),
                                           np.ascontiguousarray(yh[:, cols]), 1, p)
    assert_lp_close(gw.cpu().numpy()[cols], gw_cols, f"grad_weight channels p={p}")
    ref = _ref_lib()
    if ref is not None:
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        y_r = torch.empty_like(y)
        ref.ref_norm_dist_forward(P(xd), P(wd), B, CO, CI, 1, 1, P(y_r), ctypes.c_float(p))
        torch.cuda.synchronize()
        torch.testing.assert_close(y, y_r, rtol=2e-5, atol=0)


@pytest.mark.parametrize("G", [1, 4])
def test_inf_bound_config3_full_size(cuda, lib, G):
    """B = 512, Din = 3072, Dout = 5120 (x ~ U[0,1), box of 8/255 clamped to [0,1]), groups 1 and 4: lower and
    upper bit-exact against the reference's own CUDA kernel over the whole output, and against the CPU
    checker on 8 sampled batch rows."""
    B, CI, CO = 512, 3072, 5120
    x, w, _ = make_inputs(B, CI, CO, 1, G, seed=2022)
    eps = np.float32(8.0 / 255.0)
    lo = np.clip(x - eps, 0, 1).astype(np.float32); up = np.clip(x + eps, 0, 1).astype(np.float32)
    lod, upd, wd = dev(lo), dev(up), dev(w)
    yl, yu = c_inf_bound(lod, upd, wd, G)
    torch.cuda.synchronize()
    rows = np.sort(np.random.default_rng(G).choice(B, 8, replace=False))
    yl_rows, yu_rows = oracle.inf_dist_bound(lo[rows], up[rows], w, G)
    assert_bits_equal(yl.cpu().numpy()[rows], yl_rows, "lower rows"); assert_bits_equal(yu.cpu().numpy()[rows], yu_rows, "upper rows")
    ref = _ref_lib()
    if ref is not None:
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        yl_r = torch.empty_like(yl); yu_r = torch.empty_like(yu)
        ref.ref_inf_dist_bound_forward(P(lod), P(upd), P(wd), B, CO, CI, G, 1, P(yl_r), P(yu_r))
        torch.cuda.synchronize()
        assert_bits_equal(yl, yl_r, "lower vs reference kernel"); assert_bits_equal(yu, yu_r, "upper vs reference kernel")
    # the value path at the same shape: forward + arg-max against the reference kernel and the sampled rows
    y, pos = c_inf_forward(dev(x), wd, G)
    y_rows, pos_rows = oracle.inf_dist_forward(x[rows], w, G)
    assert_bits_equal(y.cpu().numpy()[rows], y_rows, "values rows"); assert_bits_equal(pos.cpu().numpy()[rows], pos_rows, "arg-max rows")
    if ref is not None:
        y_r = torch.empty_like(y); pos_r = torch.empty_like(pos)
        ref.ref_inf_dist_forward(P(dev(x)), P(wd), B, CO, CI, G, 1, P(y_r), P(pos_r))
        torch.cuda.synchronize()
        assert_bits_equal(y, y_r, "values vs reference kernel"); assert_bits_equal(pos, pos_r, "arg-max vs reference kernel")


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="reference kernels were not prebuilt")
@pytest.mark.parametrize("shape", [(33, 100, 65, 1, 1), (130, 784, 200, 1, 1), (16, 64, 256, 1, 4),
                                   (3, 18, 12, 5, 3), (512, 784, 5120, 1, 1)], ids=_ids)
def test_against_reference_kernels(cuda, lib, shape):
    ref = ctypes.CDLL(REF_LIB)
    B, CI, CO, HW, G = shape
    x, w, g = make_inputs(B, CI, CO, HW, G, seed=40 + CO)
    xd, wd, gd = dev(x), dev(w), dev(g)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    torch.cuda.synchronize()
    # forward + arg-max
    y_r = torch.empty(B, CO, HW, device="cuda"); pos_r = torch.empty(B, CO, HW, device="cuda", dtype=torch.int32)
    ref.ref_inf_dist_forward(P(xd), P(wd), B, CO, CI, G, HW, P(y_r), P(pos_r))
    torch.cuda.synchronize()
    y, pos = c_inf_forward(xd, wd, G)
    assert_bits_equal(y, y_r, "values vs reference kernel"); assert_bits_equal(pos, pos_r, "arg-max vs reference kernel")
    # bounds
    lo = (xd - 0.03).clamp(0, 1); up = (xd + 0.03).clamp(0, 1)
    yl_r = torch.empty_like(y_r); yu_r = torch.empty_like(y_r)
    ref.ref_inf_dist_bound_forward(P(lo), P(up), P(wd), B, CO, CI, G, HW, P(yl_r), P(yu_r))
    torch.cuda.synchronize()
    yl, yu = c_inf_bound(lo, up, wd, G)
    assert_bits_equal(yl, yl_r, "lower vs reference kernel"); assert_bits_equal(yu, yu_r, "upper vs reference kernel")
    # backward: the reference's atomics are unordered; equal up to summation order
    gx_r = torch.zeros(B, CI, HW, device="cuda"); gw_r = torch.zeros(CO, CI // G, device="cuda")
    ref.ref_inf_dist_backward_input(P(gd), P(pos_r), B, CO, CI, G, HW, P(gx_r))
    ref.ref_inf_dist_backward_weight(P(gd), P(pos_r), B, CO, CI, G, HW, P(gw_r))
    torch.cuda.synchronize()
    gx, gw = c_inf_backward(gd, pos, CI, G, "ordered")
    torch.testing.assert_close(gx, gx_r, rtol=1e-4, atol=2e-4); torch.testing.assert_close(gw, gw_r, rtol=1e-4, atol=2e-4)
    # finite p: both sides approximate; the reference uses lg2/ex2 approximations
    xn = dev(make_inputs(B, CI, CO, HW, G, seed=41, x_dist="normal")[0])
    for p in (8.0, 16.0):
        yp_r = torch.empty_like(y_r)
        ref.ref_norm_dist_forward(P(xn), P(wd), B, CO, CI, G, HW, P(yp_r), ctypes.c_float(p))
        torch.cuda.synchronize()
        yp = c_lp_forward(xn, wd, G, p)
        torch.testing.assert_close(yp, yp_r, rtol=2e-5, atol=0)


@pytest.mark.parametrize("p_norm", [float("inf"), 8.0, 23.7, None])
def test_fused_adamw_matches_torch_rule(cuda, lib, p_norm):
    """The fused optimiser kernel against the same step written with torch ops on the CPU (the
    host-side rule that also runs when tensors are not on a GPU)."""
    import linfdist_b200 as L

    def make(dev):
        torch.manual_seed(9)
        if p_norm is None:
            m = torch.nn.Linear(300, 37)                 # a module without a norm: plain decay
        else:
            m = L.NormDist(300, 37, bias=True)
            m.weight.data = torch.randn(37, 300, 1, 1)   # identity init would plant -10 entries
            m.bias.data = torch.randn(37)
            L.set_p_norm(m, p_norm)
        return m.to(dev)

    cpu, gpu = make("cpu"), make("cuda")
    oc = L.AdamW(cpu, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
    og = L.AdamW(gpu, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
    gen = torch.Generator().manual_seed(1)
    for _ in range(3):
        for prm_c, prm_g in zip(cpu.parameters(), gpu.parameters()):
            g = torch.randn(prm_c.shape, generator=gen)
            prm_c.grad = g.clone(); prm_g.grad = g.cuda()
        oc.step(); og.step()
    for prm_c, prm_g in zip(cpu.parameters(), gpu.parameters()):
        torch.testing.assert_close(prm_g.detach().cpu(), prm_c.detach(), rtol=2e-5, atol=2e-6)


def test_pipelined_step_equals_plain_step(cuda, lib):
    """The hand-scheduled step (optimiser on a side stream, forward waiting per layer) must leave
    exactly the parameters that forward -> backward -> optimizer.step() leaves."""
    import linfdist_b200 as L
    from linfdist_b200.train_step import DataParallelStep, MarginLoss, hinge

    def run(pipelined):
        torch.manual_seed(3)
        net = L.Model(L.MLP(3, 1, (3, 8, 8), num_classes=10), L.BoundFinalIdentity(), eps=8 / 255).cuda()
        L.set_p_norm(net, float("inf"))
        opt = L.AdamW(net, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
        model = DataParallelStep(net, opt) if pipelined else net
        loss_fn = MarginLoss(hinge(0.75), 1.0)
        gen = torch.Generator().manual_seed(5)
        for _ in range(4):
            x = torch.rand(64, 3, 8, 8, generator=gen).cuda(); t = torch.randint(0, 10, (64,), generator=gen).cuda()
            out, worst = model(x, targets=t)
            loss = loss_fn(out, worst, t)
            opt.zero_grad(set_to_none=True)
            loss.backward()
            if pipelined:
                model.finish_step()
            else:
                opt.step()
        if pipelined:
            model.synchronize()
        torch.cuda.synchronize()
        return [p.detach().clone() for p in net.parameters()]

    for a, b in zip(run(False), run(True)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("shape", [(4, 36, 64, 25, 1), (3, 32, 96, 9, 2), (2, 27, 40, 16, 1), (5, 64, 128, 4, 4)],
                         ids=_ids)
@pytest.mark.parametrize("p", [float("inf"), 8.0])
def test_python_operator_conv_shapes(cuda, lib, shape, p):
    """DistF / inf_dist_bound on conv-shaped inputs (HW > 1), incl. the shapes that are routed
    through the dense kernels as B*HW rows: same results as the checker on the original layout."""
    import linfdist_b200 as L
    B, CI, CO, HW, G = shape
    x, w, g = make_inputs(B, CI, CO, HW, G, seed=60 + CI, x_dist="uniform" if p == float("inf") else "normal")
    xd = dev(x).requires_grad_(True); wd = dev(w).requires_grad_(True)
    y = L.norm_dist(xd, wd, G, p)
    y.backward(dev(g))
    if p == float("inf"):
        y_ref, pos_ref = oracle.inf_dist_forward(x, w, G)
        gx_ref, gw_ref = oracle.inf_dist_backward(g, pos_ref, CI, G)
        assert_bits_equal(y.detach(), y_ref, "values")
        assert_bits_equal(xd.grad, gx_ref, "grad_input"); assert_bits_equal(wd.grad, gw_ref, "grad_weight")
        lo = np.clip(x - 0.03, 0, 1).astype(np.float32); up = np.clip(x + 0.03, 0, 1).astype(np.float32)
        yl, yu = L.inf_dist_bound(dev(lo), dev(up), dev(w), G)
        yl_ref, yu_ref = oracle.inf_dist_bound(lo, up, w, G)
        assert_bits_equal(yl, yl_ref, "lower"); assert_bits_equal(yu, yu_ref, "upper")
    else:
        y_ref = oracle.norm_dist_forward(x, w, G, p)
        assert_lp_close(y.detach(), y_ref, "forward", floor=0.0)
        gx_ref, gw_ref = oracle.norm_dist_backward(g, x, w, y_ref, G, p)
        assert_lp_close(xd.grad, gx_ref, "grad_input"); assert_lp_close(wd.grad, gw_ref, "grad_weight")


def test_norm_dist_conv_module(cuda, lib):
    """NormDistConv (3x3, padding, stride) end to end against the checker on unfolded patches."""
    import linfdist_b200 as L
    import torch.nn.functional as F
    torch.manual_seed(0)
    m = L.NormDistConv(8, 32, 3, stride=2, padding=1, bias=True, mean_normalize=False).cuda()
    L.set_p_norm(m, float("inf"))
    x = torch.rand(3, 8, 9, 9, device="cuda")
    y, _, _ = m(x)
    cols = F.unfold(x, 3, 1, 1, 2)
    y_ref, _ = oracle.inf_dist_forward(cols.cpu().numpy(), m.weight.detach().view(32, -1).cpu().numpy(), 1)
    assert y.shape == (3, 32, 5, 5)
    assert_bits_equal((y - m.bias.view(1, -1, 1, 1)).reshape(3, 32, 25), y_ref, "conv layer values")
    m.eval()
    lo = (x - 0.01).clamp(0, 1); up = (x + 0.01).clamp(0, 1)
    y2, l2, u2 = m(x, lo, up)
    assert (l2 <= y2 + 1e-6).all() and (y2 <= u2 + 1e-6).all()


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="reference kernels were not prebuilt")
def test_faster_than_reference_kernels(cuda, lib):
    """Config-1 layer (B=512, Din=784, Dout=5120): forward + backward of this library against the
    reference's own CUDA kernels compiled for sm_100a, same inputs, CUDA events, L2 flushed.  The
    measured times are written to ref_gpu_timing.json in the folder LINF_REPORT_DIR names, if set."""
    import json
    from linfdist_b200 import _lib
    from helpers import stream
    ref = ctypes.CDLL(REF_LIB)
    B, CI, CO = 512, 784, 5120
    x, w, g = make_inputs(B, CI, CO, 1, 1, seed=2020)
    xd, wd, gd = dev(x), dev(w), dev(g)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    y = torch.empty(B, CO, 1, device="cuda"); pos = torch.empty(B, CO, 1, device="cuda", dtype=torch.int32)
    gx = torch.empty_like(xd); gw = torch.empty_like(wd)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    L = _lib.load()

    def ours():
        rc = L.linf_inf_dist_forward(xd.data_ptr(), wd.data_ptr(), B, CO, CI, 1, 1, y.data_ptr(), pos.data_ptr(), stream())
        rc |= L.linf_inf_dist_backward_input(gd.data_ptr(), pos.data_ptr(), B, CO, CI, 1, 1, gx.data_ptr(), stream())
        rc |= L.linf_inf_dist_backward_weight(gd.data_ptr(), pos.data_ptr(), B, CO, CI, 1, 1, gw.data_ptr(), stream())
        assert rc == 0

    def theirs():
        ref.ref_inf_dist_forward(P(xd), P(wd), B, CO, CI, 1, 1, P(y), P(pos))
        gx.zero_(); gw.zero_()
        ref.ref_inf_dist_backward_input(P(gd), P(pos), B, CO, CI, 1, 1, P(gx))
        ref.ref_inf_dist_backward_weight(P(gd), P(pos), B, CO, CI, 1, 1, P(gw))

    def time_ms(fn, n=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            flush.zero_()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    t_ours, t_ref = time_ms(ours), time_ms(theirs)
    terms = B * CI * CO
    report = {"workload": "inf-dist layer fwd+bwd, B=512, Din=784, Dout=5120", "ours_ms": t_ours, "reference_kernels_ms": t_ref,
              "ours_terms_per_s": terms / (t_ours * 1e-3), "reference_terms_per_s": terms / (t_ref * 1e-3),
              "speedup": t_ref / t_ours}
    out_dir = os.environ.get("LINF_REPORT_DIR")
    if out_dir:
        try:
            os.makedirs(out_dir, exist_ok=True)
            json.dump(report, open(os.path.join(out_dir, "ref_gpu_timing.json"), "w"), indent=1)
        except OSError:
            pass
    assert t_ours < t_ref, report


def test_workspace_errors_and_determinism(cuda, lib):
    """A workspace that is too small or misaligned is refused with a code (no launch); a split-k
    forward gives the same bits on every run although the last-arriving CTA differs."""
    from helpers import stream
    B, CI, CO = 512, 5120, 2048
    need = lib.linf_inf_dist_forward_workspace_bytes(B, CO, CI, 1, 1)
    assert need > 0
    x = torch.rand(B, CI, 1, device="cuda"); w = torch.randn(CO, CI, device="cuda")
    y = torch.empty(B, CO, 1, device="cuda"); pos = torch.empty(B, CO, 1, device="cuda", dtype=torch.int32)
    ws = torch.empty(need + 512, dtype=torch.uint8, device="cuda")
    args = (x.data_ptr(), w.data_ptr(), B, CO, CI, 1, 1, y.data_ptr(), pos.data_ptr())
    assert lib.linf_inf_dist_forward_ws(*args, ws.data_ptr(), need - 1, stream()) == 6          # too small
    assert lib.linf_inf_dist_forward_ws(*args, ws.data_ptr() + 4, need, stream()) == 6          # misaligned
    assert lib.linf_inf_dist_forward_ws(*args, None, 0, stream()) == 6                          # missing
    runs = []
    for _ in range(3):
        assert lib.linf_inf_dist_forward_ws(*args, ws.data_ptr(), need, stream()) == 0
        torch.cuda.synchronize()
        runs.append((y.clone(), pos.clone()))
    for yy, pp in runs[1:]:
        assert torch.equal(yy, runs[0][0]) and torch.equal(pp, runs[0][1])
    y0, p0 = c_inf_forward(x, w, 1, use_ws=False)
    assert torch.equal(y0, runs[0][0]) and torch.equal(p0, runs[0][1])


def test_lp_shapes_that_leave_the_tiled_path(cuda, lib):
    """Channel counts that are not multiples of 4, and p beyond the tiled instantiations, take the
    generic kernels: same tolerance."""
    for (B, CI, CO, p) in [(9, 66, 34, 8.0), (5, 64, 33, 16.0), (70, 128, 96, 1500.5), (33, 100, 64, 2.5)]:
        x, w, g = make_inputs(B, CI, CO, 1, 1, seed=31 + CO, x_dist="normal")
        y_ref = oracle.norm_dist_forward(x, w, 1, p)
        y = c_lp_forward(dev(x), dev(w), 1, p)
        assert_lp_close(y, y_ref, f"forward {B,CI,CO,p}", floor=0.0)
        gx_ref, gw_ref = oracle.norm_dist_backward(g, x, w, y_ref, 1, p)
        gx, gw = c_lp_backward(dev(g), dev(x), dev(w), dev(y_ref), 1, p)
        rtol = 1e-5 if p <= 64 else 1e-5 * p / 64
        assert_lp_close(gx, gx_ref, f"grad_input {p}", rtol=rtol); assert_lp_close(gw, gw_ref, f"grad_weight {p}", rtol=rtol)


@pytest.mark.parametrize("pattern", ["one_bin", "two_bins", "uniform", "out_of_range", "runs"])
@pytest.mark.parametrize("shape", [(1100, 785, 96, 1), (40, 784, 1300, 1), (64, 60, 2048, 2), (513, 36, 520, 1),
                                   (300, 4100, 1024, 1), (64, 8192, 1030, 2)],
                         ids=lambda s: "B{}_CI{}_CO{}_G{}".format(*s))
def test_inf_backward_synthetic_positions(cuda, lib, pattern, shape):
    """The ordered scatter on position patterns a forward pass rarely produces: every source of a
    row in one bin, two alternating bins, indices outside the group (dropped), long runs; row
    lengths that are not multiples of 32, of the staging block or of 4."""
    B, CI, CO, G = shape
    CIg = CI // G
    rng = np.random.default_rng(len(pattern) * 100 + B)
    if pattern == "one_bin":
        idx = np.full((B, CO, 1), CIg - 1, dtype=np.int64)
    elif pattern == "two_bins":
        idx = (np.arange(B)[:, None, None] + np.arange(CO)[None, :, None]) % 2 * (CIg - 1)
    elif pattern == "uniform":
        idx = rng.integers(0, CIg, (B, CO, 1))
    elif pattern == "out_of_range":
        idx = rng.integers(0, CIg + 40, (B, CO, 1))
    else:
        idx = (np.arange(B)[:, None, None] // 37 + np.arange(CO)[None, :, None] // 45) % CIg
    sign = rng.integers(0, 2, (B, CO, 1)).astype(np.uint32) << 31
    pos = (idx.astype(np.uint32) | sign).view(np.int32)
    g = rng.standard_normal((B, CO, 1)).astype(np.float32)
    gx_ref, gw_ref = oracle.inf_dist_backward(g, pos, CI, G)
    for mode in ("ordered", "both"):
        gx, gw = c_inf_backward(dev(g), dev(pos), CI, G, mode)
        assert_bits_equal(gx, gx_ref, f"{mode} grad_input"); assert_bits_equal(gw, gw_ref, f"{mode} grad_weight")


@pytest.mark.parametrize("shape", [(512, 784, 5120), (96, 3072, 1024), (64, 5120, 1024), (40, 2048, 1536), (300, 100, 65)],
                         ids=lambda s: "B{}_CI{}_CO{}".format(*s))
def test_inf_backward_with_mostly_zero_grad_output(cuda, lib, shape):
    """In a training step most of grad_output is exactly zero (whole columns of it).  The kernels drop such sources
    instead of adding +-0; the sums must still be the checker's bits, signed zeros included."""
    B, CI, CO = shape
    x, w, _ = make_inputs(B, CI, CO, 1, 1, seed=4000 + CO)
    _, pos = oracle.inf_dist_forward(x, w, 1)
    rng = np.random.default_rng(B + CO)
    g = rng.standard_normal((B, CO, 1)).astype(np.float32)
    g[:, rng.random(CO) < 0.9, :] = 0.0                      # nine columns in ten are zero
    g[rng.random((B, CO, 1)) < 0.3] *= 0.0                   # and a third of the rest, as +0 or -0
    gx_ref, gw_ref = oracle.inf_dist_backward(g, pos, CI, 1)
    for mode in ("ordered", "both"):
        gx, gw = c_inf_backward(dev(g), dev(pos), CI, 1, mode)
        assert_bits_equal(gx, gx_ref, f"{mode} grad_input"); assert_bits_equal(gw, gw_ref, f"{mode} grad_weight")


@pytest.mark.parametrize("pattern", ["hot", "spread", "mixed"])
def test_inf_backward_input_kernel_choice(cuda, lib, pattern):
    """grad_input of a wide dense layer runs on the direct-accumulation kernel or on the sort kernel, as a probe of
    the arg-max positions decides (many sources of a row in few bins: the sort).  Whatever the probe says, and with
    either kernel forced, the bits are the checker's."""
    B, CI, CO = 40, 2048, 1536
    rng = np.random.default_rng(7 + len(pattern))
    if pattern == "hot":            # three quarters of every row's sources in a dozen bins
        idx = np.where(rng.random((B, CO, 1)) < 0.75, rng.integers(0, 12, (B, CO, 1)) * 97, rng.integers(0, CI, (B, CO, 1)))
    elif pattern == "spread":
        idx = rng.integers(0, CI, (B, CO, 1))
    else:                           # only some rows are contested (the probe samples rows: either answer must be right)
        idx = rng.integers(0, CI, (B, CO, 1))
        idx[::5] = rng.integers(0, 3, (len(idx[::5]), CO, 1)) * 11
    sign = rng.integers(0, 2, (B, CO, 1)).astype(np.uint32) << 31
    pos = (idx.astype(np.uint32) | sign).view(np.int32)
    g = rng.standard_normal((B, CO, 1)).astype(np.float32)
    gx_ref, gw_ref = oracle.inf_dist_backward(g, pos, CI, 1)
    try:
        for path in (0, 1, 2):
            assert lib.linf_tune_set(3, path) == 0
            for mode in ("ordered", "both"):
                gx, gw = c_inf_backward(dev(g), dev(pos), CI, 1, mode)
                assert_bits_equal(gx, gx_ref, f"path {path} {mode} grad_input")
                assert_bits_equal(gw, gw_ref, f"path {path} {mode} grad_weight")
    finally:
        lib.linf_tune_set(3, 0)


@pytest.mark.parametrize("shape", [(64, 64, 64, 1, 1), (33, 100, 65, 1, 1), (130, 784, 200, 1, 1), (16, 64, 256, 1, 4),
                                   (70, 1000, 96, 1, 1), (512, 784, 640, 1, 1), (64, 3072, 512, 1, 4), (9, 36, 40, 1, 1)], ids=_ids)
@pytest.mark.parametrize("variant", [4, 1, 2, 3], ids=["tma_padded", "cp_async_32", "cp_async_16", "window_16"])
def test_inf_forward_other_loader_variants(cuda, lib, shape, variant):
    """The default forward fetches its operand tiles by TMA (tiled bulk copies with the 128-byte swizzle,
    completion on mbarriers).  The other variants of the same kernel -- TMA with padded boxes, cp.async
    with 32- or 16-term k-tiles, one tracking window per k-tile -- must give the same bits.  Ragged
    k-tiles, rows and channels past the end arrive as zeros from the copy engine; the bounded waits
    of the TMA loaders must never have run out."""
    B, CI, CO, HW, G = shape
    x, w, _ = make_inputs(B, CI, CO, HW, G, seed=77 + CI)
    y_ref, pos_ref = oracle.inf_dist_forward(x, w, G)
    assert lib.linf_tune_set(0, variant) == 0
    try:
        for use_ws in (False, True):
            y, pos = c_inf_forward(dev(x), dev(w), G, use_ws=use_ws)
            assert_bits_equal(y, y_ref, "values"); assert_bits_equal(pos, pos_ref, "arg-max")
        assert lib.linf_tune_set(2, 0) == 0
    finally:
        lib.linf_tune_set(0, 0)


@pytest.mark.parametrize("shape", [(64, 64, 64, 1, 1), (33, 100, 65, 1, 1), (130, 784, 200, 1, 1), (16, 64, 256, 1, 4),
                                   (70, 1000, 96, 1, 1), (512, 784, 640, 1, 1), (64, 3072, 512, 1, 4), (9, 36, 40, 1, 1),
                                   (200, 256, 48, 1, 1), (65, 160, 49, 1, 1), (300, 1024, 1100, 1, 1),
                                   # rows of 2048 terms and more: 16-term tracking windows
                                   (70, 2304, 130, 1, 1), (33, 4100, 96, 1, 1), (40, 4096, 128, 1, 2)], ids=_ids)
@pytest.mark.parametrize("width", [1, 2], ids=["tiles_64", "tiles_48"])
def test_inf_forward_tile_widths(cuda, lib, shape, width):
    """The library picks between output tiles of 64 x 64 and 64 x 48 (and k-splitting) by the shape; forced either
    way, with and without scratch, the bits must be those of the checker -- including channel counts that are
    no multiple of either width and grouped layers."""
    B, CI, CO, HW, G = shape
    x, w, _ = make_inputs(B, CI, CO, HW, G, seed=99 + CO)
    y_ref, pos_ref = oracle.inf_dist_forward(x, w, G)
    assert lib.linf_tune_set(5, width) == 0
    try:
        for windows in ((0, 1) if CI // G >= 2048 else (0,)):
            assert lib.linf_tune_set(7, windows) == 0
            for split in (2, 0, 1):
                assert lib.linf_tune_set(4, split) == 0
                for use_ws in (False, True):
                    y, pos = c_inf_forward(dev(x), dev(w), G, use_ws=use_ws)
                    assert_bits_equal(y, y_ref, "values"); assert_bits_equal(pos, pos_ref, "arg-max")
        assert lib.linf_tune_set(2, 0) == 0
    finally:
        lib.linf_tune_set(5, 0); lib.linf_tune_set(4, 0); lib.linf_tune_set(7, 0)


def test_adamw_step_rows_equals_whole_tensor_step(cuda, lib):
    """Updating a weight matrix in row blocks, each block with moments of its own (what the sharded
    data-parallel steps do on every rank), leaves exactly the bits of one update of the whole matrix."""
    import linfdist_b200 as L

    def make():
        torch.manual_seed(5)
        m = L.NormDist(256, 64, bias=False).cuda()
        m.weight.data = torch.randn(64, 256, 1, 1, device="cuda")
        return m

    whole, parts = make(), make()
    ow = L.AdamW(whole, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
    op = L.AdamW(parts, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
    gen = torch.Generator(device="cuda").manual_seed(2)
    for _ in range(3):
        g = torch.randn(64, 256, 1, 1, device="cuda", generator=gen)
        whole.weight.grad = g.clone()
        ow.step()
        for r0 in range(0, 64, 16):
            op.step_rows(parts.weight, r0, 16, g.view(64, 256)[r0:r0 + 16].contiguous())
    torch.cuda.synchronize()
    assert torch.equal(whole.weight.data, parts.weight.data)


def test_certify_config4_shape_bit_exact(cuda, lib):
    """The certification pass (eval mode, clamped eps box, five distance layers 3072-5120x4-10 with their
    eval-mode mean shift / bias, margins) on the GPU against the CPU checker chained layer by layer."""
    import linfdist_b200 as L
    from linfdist_b200.train_step import build_cifar_net
    B, eps = 48, 8.0 / 255.0
    net = build_cifar_net(torch.device("cuda:0"))
    gen = torch.Generator().manual_seed(77)
    for m in net.modules():
        if isinstance(m, L.MeanNorm):
            m.running_mean.copy_(torch.randn(m.running_mean.shape, generator=gen).cuda() + 9.0)
    net.feature.fc_last.bias.data = torch.randn(10, generator=gen).cuda()
    x = torch.rand(B, 3, 32, 32, generator=gen); t = torch.randint(0, 10, (B,), generator=gen)
    ok, margins = L.certify(net, x.cuda(), t.cuda(), eps, torch.ones((), device="cuda"), torch.zeros((), device="cuda"))
    lo = torch.max(x - eps, torch.zeros(())).reshape(B, -1).numpy(); up = torch.min(x + eps, torch.ones(())).reshape(B, -1).numpy()
    layers = list(net.feature.fc) + [net.feature.fc_last]
    for layer in layers:
        w = layer.weight.detach().view(layer.weight.size(0), -1).cpu().numpy()
        lo, up = oracle.inf_dist_bound(lo[:, :, None], up[:, :, None], w, 1)
        lo, up = lo[:, :, 0], up[:, :, 0]
        if layer.normalize is not None:
            rm = layer.normalize.running_mean.cpu().numpy()
            lo, up = lo - rm, up - rm
        if layer.bias is not None:
            b = layer.bias.detach().cpu().numpy()
            lo, up = lo + b, up + b
    lo, up = -up, -lo                                         # a small distance means "this class"
    tn = t.numpy()
    ref = up - lo[np.arange(B), tn][:, None]
    ref[np.arange(B), tn] = 0.0
    assert_bits_equal(margins, ref.astype(np.float32), "worst-case margins")
    assert np.array_equal(ok.cpu().numpy(), ref.argmax(axis=1) == tn)
    # with the value path run as well (the reference's loop), and with the torch epilogue: the same margins
    _, m2 = L.certify(net, x.cuda(), t.cuda(), eps, torch.ones((), device="cuda"), torch.zeros((), device="cuda"), values=True)
    assert_bits_equal(m2, margins, "margins with the value path")
    L.set_fused_epilogue(False)
    try:
        _, m3 = L.certify(net, x.cuda(), t.cuda(), eps, torch.ones((), device="cuda"), torch.zeros((), device="cuda"), values=True)
    finally:
        L.set_fused_epilogue(True)
    assert_bits_equal(m3, margins, "margins with separate elementwise passes")


def test_pgd_runs_the_input_gradient_only(cuda, lib):
    """AttackPGD freezes the parameters, so the backward of every distance layer produces grad_input
    alone; that gradient must be the one a full backward gives, and one step of `find` must be the
    sign step projected onto the eps ball and the data range."""
    import torch.nn.functional as F
    import linfdist_b200 as L
    torch.manual_seed(1)
    net = L.Model(L.MLP(3, 1, (3, 8, 8), num_classes=10), L.BoundFinalIdentity(), eps=8 / 255).cuda()
    L.set_p_norm(net, float("inf"))
    net.eval()
    x = torch.rand(32, 3, 8, 8, device="cuda"); t = torch.randint(0, 10, (32,), device="cuda")
    xa = x.clone().requires_grad_(True)
    F.cross_entropy(net(xa), t, reduction="sum").backward()
    assert all(q.grad is not None for q in net.parameters())
    full = xa.grad.clone()
    net.zero_grad(set_to_none=True)
    eps, step = 8 / 255, 2 / 255
    up, down = torch.ones((), device="cuda"), torch.zeros((), device="cuda")
    adv = L.AttackPGD(net, eps, step, 1, up, down, random_start=False).find(x, t)
    assert all(q.grad is None for q in net.parameters()) and all(q.requires_grad for q in net.parameters())
    want = torch.min(torch.max(torch.min(torch.max(x + step * torch.sign(full), x - eps), x + eps), down), up)
    assert torch.equal(adv, want)
    adv = L.AttackPGD(net, eps, step, 5, up, down, random_start=True).find(x, t)
    assert float((adv - x).abs().max()) <= eps + 1e-6 and float(adv.min()) >= 0 and float(adv.max()) <= 1


@pytest.mark.parametrize("shape", [(512, 5120), (7, 33), (64, 100), (513, 31)])
def test_mean_shift_one_launch(cuda, lib, shape):
    """Training-mode mean shift in one launch: the mean agrees with torch's reduction to fp32 rounding (the
    summation order differs), and GIVEN that mean the subtraction and the running-mean update are the
    torch sequence of model/norm_dist.py:85-97 bit for bit.  Its backward is the same map on the gradient."""
    import linfdist_b200 as L
    from helpers import stream
    rows, cols = shape
    gen = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=gen) * 3 + 10).cuda()
    rm0 = torch.randn(cols, generator=gen).cuda()
    rm = rm0.clone(); out = torch.empty_like(x); mean = torch.empty(cols, device="cuda")
    assert lib.linf_mean_shift(x.data_ptr(), rows, cols, rm.data_ptr(), 0.1, out.data_ptr(), mean.data_ptr(), stream()) == 0
    torch.cuda.synchronize()
    exact = x.double().mean(dim=0)
    assert float((mean.double() - exact).abs().max()) <= 2e-6 * float(x.abs().max())
    assert float((mean - x.mean(dim=0)).abs().max()) <= 4e-6 * float(x.abs().max())
    assert torch.equal(out, x - mean)
    assert torch.equal(rm, rm0.clone().mul_(1 - 0.1).add_(mean, alpha=0.1))
    # in place, and without a running mean
    y = x.clone()
    assert lib.linf_mean_shift(y.data_ptr(), rows, cols, None, 0.0, y.data_ptr(), None, stream()) == 0
    assert torch.equal(y, out)
    # the module: fused and torch paths agree to rounding, forward and backward
    m_f, m_t = L.MeanNorm(cols).cuda(), L.MeanNorm(cols).cuda()
    xa = x.clone().requires_grad_(True); xb = x.clone().requires_grad_(True)
    g = torch.randn(rows, cols, generator=gen).cuda()
    ya = m_f(xa); ya.backward(g)
    L.set_fused_epilogue(False)
    try:
        yb = m_t(xb); yb.backward(g)
    finally:
        L.set_fused_epilogue(True)
    torch.testing.assert_close(ya, yb, rtol=0, atol=4e-6 * float(x.abs().max()))
    torch.testing.assert_close(xa.grad, xb.grad, rtol=0, atol=4e-6 * float(g.abs().max()))
    torch.testing.assert_close(m_f.running_mean, m_t.running_mean, rtol=0, atol=1e-6 * float(x.abs().max()))


@pytest.mark.parametrize("case", [(64, 784, 5120, True, False, False), (37, 5120, 10, False, True, True), (130, 100, 65, True, True, False),
                                  (9, 18, 7, True, True, True), (512, 3072, 640, True, False, False), (33, 256, 96, False, False, True)],
                         ids=lambda c: "B{}_CI{}_CO{}_mn{}_bias{}_neg{}".format(*[int(v) for v in c]))
def test_eval_epilogue_in_kernel_bit_exact(cuda, lib, case):
    """Eval mode: mean shift by the running mean, bias and sign flip applied inside the forward and bound
    kernels (tiled, few-output and generic paths) against the same steps as separate torch operations
    (model/norm_dist.py:137-140, :150-155, model/mlp.py:22): identical bits for value, lower and upper."""
    import linfdist_b200 as L
    B, CI, CO, mean_normalize, bias, negate = case
    torch.manual_seed(CI + CO)
    layer = L.NormDist(CI, CO, bias=bias, mean_normalize=mean_normalize).cuda()
    L.set_p_norm(layer, float("inf"))
    if mean_normalize:
        layer.normalize.running_mean.copy_(torch.randn(CO).cuda() + 5)
    if bias:
        layer.bias.data = torch.randn(CO).cuda()
    layer.eval()
    x = torch.rand(B, CI, device="cuda"); lo = (x - 0.02).clamp(0, 1); up = (x + 0.02).clamp(0, 1)
    with torch.no_grad():
        fused = layer(x, lo, up, negate=negate)
        L.set_fused_epilogue(False)
        try:
            plain = layer(x, lo, up, negate=negate)
        finally:
            L.set_fused_epilogue(True)
    for a, b, name in zip(fused, plain, ("value", "lower", "upper")):
        assert_bits_equal(a, b, name)
    assert bool((fused[1] <= fused[2]).all())
    # with gradients required the value takes the arg-max path and the torch steps: same numbers
    xg = x.clone().requires_grad_(True)
    yg, _, _ = layer(xg, negate=negate)
    assert_bits_equal(yg.detach(), fused[0], "value with autograd")
    yg.sum().backward()
    assert xg.grad is not None


def test_training_step_with_and_without_fused_mean_shift(cuda, lib):
    """Two optimisation steps of a small net with the one-launch mean shift and with the torch sequence:
    the same parameters up to the rounding of the batch means."""
    import linfdist_b200 as L
    from linfdist_b200.train_step import MarginLoss, hinge

    def run(fused):
        L.set_fused_epilogue(fused)
        torch.manual_seed(3)
        net = L.Model(L.MLP(3, 1, (3, 8, 8), num_classes=10), L.BoundFinalIdentity(), eps=8 / 255).cuda()
        for m in net.modules():
            if isinstance(m, L.NormDist):
                m.weight.data.normal_()
        L.set_p_norm(net, 8.0)
        opt = L.AdamW(net, lr=0.02, betas=(0.9, 0.99), eps=1e-3, weight_decay=5e-3)
        loss_fn = MarginLoss(hinge(0.75), 1.0)
        gen = torch.Generator().manual_seed(5)
        for _ in range(2):
            x = torch.rand(64, 3, 8, 8, generator=gen).cuda(); t = torch.randint(0, 10, (64,), generator=gen).cuda()
            out, worst = net(x, targets=t)
            loss = loss_fn(out, worst, t)
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
        torch.cuda.synchronize()
        return [q.detach().clone() for q in net.parameters()] + [b.clone() for b in net.buffers()]

    try:
        a, b = run(True), run(False)
    finally:
        L.set_fused_epilogue(True)
    for qa, qb in zip(a, b):
        torch.testing.assert_close(qa, qb, rtol=1e-4, atol=1e-5)


def test_launch_count_counts_the_library_kernels(cuda, lib):
    """linf_launch_count: what bench.py reports as gpu_launches.  A forward and the two backward kernels of the
    headline layer are three launches; a call that is refused launches nothing."""
    x, w, g = make_inputs(64, 784, 256, 1, 1, seed=5)
    n0 = lib.linf_launch_count()
    y, pos = c_inf_forward(dev(x), dev(w), 1, use_ws=False)
    n1 = lib.linf_launch_count()
    c_inf_backward(dev(g), pos, 784, 1, "both")
    n2 = lib.linf_launch_count()
    assert 1 <= n1 - n0 <= 2 and n2 - n1 == 2, (n0, n1, n2)
    assert lib.linf_inf_dist_forward(None, None, 1, 1, 1, 1, 1, None, None, None) != 0
    assert lib.linf_launch_count() == n2
