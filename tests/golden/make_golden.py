"""Generates the golden fixtures of this folder from the REFERENCE implementation.

Run in a container that has the reference checkout (it is not needed to run the tests):

    python tests/golden/make_golden.py --reference <checkout of zbh2047/L_inf-dist-net>

The script imports the reference's model/norm_dist.py (after registering an empty stand-in
for its CUDA extension `norm_dist_cpp`, which that file imports unconditionally) and calls its
pure-PyTorch branch (`use_custom_cuda_func=False`, model/norm_dist.py:52-57 and :66-75) on
seeded inputs on the CPU.  Inputs and reference outputs are stored together, so the tests do
not depend on a random-number generator reproducing the same stream.

Files written:
    inf_forward.npz  p = inf forward values and autograd gradients
    inf_bound.npz    interval bounds (lower, upper)
    lp.npz           finite-p forward values and autograd gradients
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (B, CI, CO, HW, G)
SHAPES = [
    (1, 1, 1, 1, 1),
    (5, 20, 12, 1, 1),
    (7, 17, 10, 1, 1),
    (6, 32, 48, 1, 4),
    (3, 18, 12, 5, 3),
    (33, 100, 65, 1, 1),
    (4, 64, 40, 1, 1),
    (2, 8, 6, 4, 2),
]
LP_PS = [8.0, 16.0, 64.0, 11.3, 1.5, 200.0]


def load_reference(path):
    sys.modules.setdefault("norm_dist_cpp", types.ModuleType("norm_dist_cpp"))
    sys.path.insert(0, path)
    from model import norm_dist as ref  # noqa: E402
    return ref


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LINF_REFERENCE"), required=os.environ.get("LINF_REFERENCE") is None,
                    help="checkout of zbh2047/L_inf-dist-net (or set LINF_REFERENCE)")
    args = ap.parse_args()
    ref = load_reference(args.reference)
    torch.set_num_threads(1)
    gen = torch.Generator().manual_seed(2020)

    inf_fw, bound, lp = {}, {}, {}
    for n, (B, CI, CO, HW, G) in enumerate(SHAPES):
        x = torch.rand(B, CI, HW, generator=gen)
        w = torch.randn(CO, CI // G, generator=gen)
        g = torch.randn(B, CO, HW, generator=gen)

        # ---- p = inf forward + autograd gradients -------------------------------------
        xr = x.clone().requires_grad_(True)
        wr = w.clone().requires_grad_(True)
        y = ref.norm_dist(xr, wr, G, float("inf"), use_custom_cuda_func=False)
        y.backward(g)
        key = f"c{n}"
        inf_fw[key + "_shape"] = np.array([B, CI, CO, HW, G])
        inf_fw[key + "_x"] = x.numpy(); inf_fw[key + "_w"] = w.numpy(); inf_fw[key + "_g"] = g.numpy()
        inf_fw[key + "_y"] = y.detach().numpy()
        inf_fw[key + "_gx"] = xr.grad.numpy(); inf_fw[key + "_gw"] = wr.grad.numpy()

        # ---- interval bounds: an eps box, plus planted degenerate intervals ---------------
        eps = 8.0 / 255.0
        lo = (x - eps).clamp(0, 1)
        up = (x + eps).clamp(0, 1)
        if B * CI * HW >= 4:
            lo.view(-1)[1] = up.view(-1)[1]                      # lower == upper
        w2 = w.clone()
        if CI // G >= 2:
            w2[0, 0] = lo[0, 0, 0]                               # lower == weight
            w2[0, 1] = up[0, 1, 0]                               # upper == weight
        yl, yu = ref.inf_dist_bound(lo, up, w2, G, use_custom_cuda_func=False)
        bound[key + "_shape"] = np.array([B, CI, CO, HW, G])
        bound[key + "_lo"] = lo.numpy(); bound[key + "_up"] = up.numpy(); bound[key + "_w"] = w2.numpy()
        bound[key + "_yl"] = yl.numpy(); bound[key + "_yu"] = yu.numpy()

        # ---- finite p ------------------------------------------------------------------
        xn = torch.randn(B, CI, HW, generator=gen)
        lp[key + "_shape"] = np.array([B, CI, CO, HW, G])
        lp[key + "_x"] = xn.numpy(); lp[key + "_w"] = w.numpy(); lp[key + "_g"] = g.numpy()
        for p in LP_PS:
            xr = xn.clone().requires_grad_(True)
            wr = w.clone().requires_grad_(True)
            y = ref.norm_dist(xr, wr, G, p, use_custom_cuda_func=False)
            y.backward(g)
            tag = f"{key}_p{p:g}"
            lp[tag + "_y"] = y.detach().numpy()
            lp[tag + "_gx"] = xr.grad.numpy(); lp[tag + "_gw"] = wr.grad.numpy()
    lp["ps"] = np.array(LP_PS)

    np.savez_compressed(os.path.join(HERE, "inf_forward.npz"), **inf_fw)
    np.savez_compressed(os.path.join(HERE, "inf_bound.npz"), **bound)
    np.savez_compressed(os.path.join(HERE, "lp.npz"), **lp)
    for f in ("inf_forward.npz", "inf_bound.npz", "lp.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
