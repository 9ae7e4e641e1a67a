"""GPU: the drop-in proof.  The reference's own, unmodified model/norm_dist.py (staged by oracle/build.py
under baseline/_ref/, outside the repository's history) is imported with the ctypes stand-in for its
compiled extension `norm_dist_cpp` (l_inf-dist-net_b200/shim/norm_dist_cpp.py) first on sys.path, and its
DistF / norm_dist / inf_dist_bound / NormDist are run against the CPU checker."""
import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from conftest import ROOT
from helpers import assert_bits_equal, assert_lp_close, dev, make_inputs

pytestmark = pytest.mark.gpu

REF_FILE = os.path.join(ROOT, "baseline", "_ref", "model", "norm_dist.py")
SHIM_DIR = os.path.join(ROOT, "l_inf-dist-net_b200", "shim")


@pytest.fixture(scope="module")
def ref(cuda, lib):
    if not os.path.exists(REF_FILE):
        pytest.skip("the reference's model/norm_dist.py was not staged (oracle/build.py --reference ...)")
    sys.modules.pop("norm_dist_cpp", None)
    sys.path.insert(0, SHIM_DIR)
    try:
        spec = importlib.util.spec_from_file_location("reference_norm_dist", REF_FILE)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)                       # runs `import norm_dist_cpp`: the stand-in
    finally:
        sys.path.remove(SHIM_DIR)
    assert sys.modules["norm_dist_cpp"].__file__.startswith(SHIM_DIR)
    return mod


@pytest.mark.parametrize("shape", [(33, 100, 65, 1, 1), (130, 784, 200, 1, 1), (16, 64, 256, 1, 4), (3, 18, 12, 5, 3),
                                   (256, 784, 1024, 1, 1)], ids=lambda s: "B{}_CI{}_CO{}_HW{}_G{}".format(*s))
def test_reference_distf_on_this_library(ref, shape):
    B, CI, CO, HW, G = shape
    x, w, g = make_inputs(B, CI, CO, HW, G, seed=800 + CO)
    xd = dev(x).requires_grad_(True); wd = dev(w).requires_grad_(True)
    y = ref.DistF.apply(xd, wd, G, float("inf"), None)
    y.backward(dev(g))
    y_ref, pos_ref = oracle.inf_dist_forward(x, w, G)
    gx_ref, gw_ref = oracle.inf_dist_backward(g, pos_ref, CI, G)
    assert_bits_equal(y.detach(), y_ref, "values")
    assert_bits_equal(xd.grad, gx_ref, "grad_input"); assert_bits_equal(wd.grad, gw_ref, "grad_weight")
    # finite p through the same reference code path
    xn = make_inputs(B, CI, CO, HW, G, seed=801, x_dist="normal")[0]
    xd = dev(xn).requires_grad_(True); wd = dev(w).requires_grad_(True)
    y = ref.norm_dist(xd, wd, G, 8.0)
    y.backward(dev(g))
    y8 = oracle.norm_dist_forward(xn, w, G, 8.0)
    assert_lp_close(y.detach(), y8, "L_8 forward", floor=0.0)
    gx8, gw8 = oracle.norm_dist_backward(g, xn, w, y.detach().cpu().numpy(), G, 8.0)
    assert_lp_close(xd.grad, gx8, "L_8 grad_input"); assert_lp_close(wd.grad, gw8, "L_8 grad_weight")
    # interval bounds
    lo = np.clip(x - 0.03, 0, 1).astype(np.float32); up = np.clip(x + 0.03, 0, 1).astype(np.float32)
    yl, yu = ref.inf_dist_bound(dev(lo), dev(up), dev(w), G)
    yl_ref, yu_ref = oracle.inf_dist_bound(lo, up, w, G)
    assert_bits_equal(yl, yl_ref, "lower"); assert_bits_equal(yu, yu_ref, "upper")


def test_reference_module_and_errors(ref):
    torch.manual_seed(0)
    layer = ref.NormDist(96, 40, bias=True, mean_normalize=True).cuda()
    ref.set_p_norm(layer, float("inf"))
    layer.eval()
    x = torch.rand(12, 96, device="cuda")
    y, lo, up = layer(x, x - 0.01, x + 0.01)
    w = layer.weight.detach().view(40, 96).cpu().numpy()
    y_ref, _ = oracle.inf_dist_forward(x.cpu().numpy()[:, :, None], w, 1)
    assert_bits_equal((y - layer.bias).detach().cpu().numpy(), y_ref[:, :, 0] - layer.normalize.running_mean.cpu().numpy(), "layer values")
    assert bool((lo <= y + 1e-6).all()) and bool((y <= up + 1e-6).all())
    with pytest.raises(RuntimeError):                      # the binding's contiguity check (model/norm_dist.cpp:3-5)
        ref.norm_dist(torch.rand(4, 8, 6, device="cuda").transpose(1, 2), torch.rand(5, 6, device="cuda"), 1, float("inf"))
    with pytest.raises(RuntimeError):                      # a CPU tensor
        ref.norm_dist(torch.rand(4, 6, 1), torch.rand(5, 6, device="cuda"), 1, float("inf"))
