"""CPU: the oracle (oracle/linf_oracle.c) against the fixtures produced by the reference's own
pure-PyTorch branch (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

import oracle
from helpers import GOLDEN, assert_bits_equal, assert_lp_close


def _cases(npz):
    return sorted({k.split("_")[0] for k in npz.files if k.startswith("c")}, key=lambda s: int(s[1:]))


def test_inf_forward_values_bit_exact():
    z = np.load(os.path.join(GOLDEN, "inf_forward.npz"))
    for c in _cases(z):
        B, CI, CO, HW, G = z[c + "_shape"]
        y, pos = oracle.inf_dist_forward(z[c + "_x"], z[c + "_w"], int(G))
        assert_bits_equal(y, z[c + "_y"], f"inf forward {c}")
        # the index must point at a term that attains the maximum, with the right sign
        x, w = z[c + "_x"], z[c + "_w"]
        idx = pos & 0x7fffffff
        for b in range(B):
            for o in range(CO):
                g = o // (CO // G)
                for hw in range(HW):
                    i = idx[b, o, hw]
                    t = np.float32(x[b, g * (CI // G) + i, hw]) - np.float32(w[o, i])
                    assert abs(t) == y[b, o, hw]
                    assert (pos[b, o, hw] < 0) == (t < 0)


def test_inf_backward_close_to_autograd():
    """Autograd of the reference branch rescales each contribution by n/n and splits ties, so it
    is not bit-comparable; without ties it must agree to rounding."""
    z = np.load(os.path.join(GOLDEN, "inf_forward.npz"))
    for c in _cases(z):
        B, CI, CO, HW, G = z[c + "_shape"]
        y, pos = oracle.inf_dist_forward(z[c + "_x"], z[c + "_w"], int(G))
        gx, gw = oracle.inf_dist_backward(z[c + "_g"], pos, int(CI), int(G))
        np.testing.assert_allclose(gx, z[c + "_gx"], rtol=2e-5, atol=2e-5)
        np.testing.assert_allclose(gw, z[c + "_gw"], rtol=2e-5, atol=2e-5)


def test_inf_bound_bit_exact():
    z = np.load(os.path.join(GOLDEN, "inf_bound.npz"))
    for c in _cases(z):
        G = int(z[c + "_shape"][4])
        yl, yu = oracle.inf_dist_bound(z[c + "_lo"], z[c + "_up"], z[c + "_w"], G)
        assert_bits_equal(yl, z[c + "_yl"], f"bound lower {c}")
        assert_bits_equal(yu, z[c + "_yu"], f"bound upper {c}")


def test_lp_within_tolerance():
    z = np.load(os.path.join(GOLDEN, "lp.npz"))
    for c in _cases(z):
        G = int(z[c + "_shape"][4])
        x, w, g = z[c + "_x"], z[c + "_w"], z[c + "_g"]
        for p in z["ps"]:
            tag = f"{c}_p{p:g}"
            y = oracle.norm_dist_forward(x, w, G, float(p))
            assert_lp_close(y, z[tag + "_y"], f"lp forward {tag}", floor=0.0)
            gx, gw = oracle.norm_dist_backward(g, x, w, y, G, float(p))
            # the fp32 autograd of the reference carries about (p-1) * 6e-8 of rounding itself
            rtol = max(1e-5, 1e-7 * float(p))
            assert_lp_close(gx, z[tag + "_gx"], f"lp grad_input {tag}", rtol=rtol)
            assert_lp_close(gw, z[tag + "_gw"], f"lp grad_weight {tag}", rtol=rtol)


def test_tie_break_and_zero_row():
    x = np.zeros((2, 4, 1), np.float32); w = np.zeros((3, 4), np.float32)
    # row 0: |t| = 2 at i = 1 (t = -2) and i = 3 (t = +2): lowest index wins, sign bit set
    x[0, :, 0] = [0, 1, 0, 5]; w[0] = [0, 3, 0, 3]
    y, pos = oracle.inf_dist_forward(x, w, 1)
    assert y[0, 0, 0] == 2 and pos[0, 0, 0] == np.int32(-2 ** 31 + 1)
    # an all-zero difference gives value 0, pos 0
    assert y[1, 1, 0] == 0 and pos[1, 1, 0] == 0


def test_ordered_scatter_definition():
    """grad cells are sequential fp32 sums in ascending source order, starting from +0."""
    rng = np.random.default_rng(0)
    B, CO, CI = 3, 50, 4
    g = (rng.standard_normal((B, CO, 1)) * 1e3).astype(np.float32)
    pos = rng.integers(0, CI, (B, CO, 1)).astype(np.int32)
    pos[:, ::3] |= np.int32(-2 ** 31)
    gx, gw = oracle.inf_dist_backward(g, pos, CI, 1)
    exp_x = np.zeros((B, CI, 1), np.float32); exp_w = np.zeros((CO, CI), np.float32)
    for b in range(B):
        for o in range(CO):
            i = pos[b, o, 0] & 0x7fffffff
            s = np.float32(1) if pos[b, o, 0] >= 0 else np.float32(-1)
            exp_x[b, i, 0] = np.float32(exp_x[b, i, 0] + s * g[b, o, 0])
            exp_w[o, i] = np.float32(exp_w[o, i] - s * g[b, o, 0])
    assert_bits_equal(gx, exp_x, "grad_input"); assert_bits_equal(gw, exp_w, "grad_weight")
