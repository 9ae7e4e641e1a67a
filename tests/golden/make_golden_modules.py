"""Generates golden fixtures for the host-side modules from the REFERENCE implementation.

Run in a container that has the reference checkout (it is not needed to run the tests):

    python tests/golden/make_golden_modules.py --reference <checkout of zbh2047/L_inf-dist-net>

Everything is computed by the reference's own Python on the CPU:
    adamw.npz          adamw.py:30-86 -- three optimisation steps of one layer from seeded weights and
                       gradients, for p_norm in {inf, 8, 23.7} (a NormDist layer with bias) and for a
                       module without a norm (torch.nn.Linear): parameters after every step
    bound_modules.npz  model/bound_module.py:5-116 -- BoundLinear (with / without bias), BoundFinalLinear
                       (non-zero bias, targets), BoundMeanNorm (train twice, then eval; 2-D and 4-D),
                       BoundFinalIdentity, BoundReLU / BoundTanh, Predictor: inputs, parameters, outputs
    small_nets.npz     model/model.py + model/mlp.py + adamw.py -- two optimisation steps of a small
                       distance net (MLP 192-64-64-10 with BoundFinalIdentity, hinge loss; and MLPFeature
                       192-64-64 + Predictor(64, 32, 20), cross entropy) at p = inf and p = 8, through the
                       reference's pure-PyTorch distance branch (model/norm_dist.py:52-57; the modules
                       call norm_dist with the CUDA branch as default, so the script binds
                       use_custom_cuda_func=False).  The layer width unit (model/mlp.py: net_width)
                       is set to 64 so that the fixture stays small; weights are plain N(0,1) draws.
                       For the p = inf runs also the certification pass of main.py:166-194 on the
                       state after the two steps (eval mode, bounds through every layer, margins).
The reference file model/norm_dist.py imports its CUDA extension unconditionally; an empty stand-in
module named norm_dist_cpp is registered first.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
HYPER = dict(lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)


def load_reference(path):
    sys.modules.setdefault("norm_dist_cpp", types.ModuleType("norm_dist_cpp"))
    sys.path.insert(0, path)
    import adamw as ref_adamw                                   # noqa: E402
    from model import bound_module, mlp, model, norm_dist      # noqa: E402
    cpu_branch = norm_dist.norm_dist
    norm_dist.norm_dist = lambda i, w, g, p, use_custom_cuda_func=True, tag=None: cpu_branch(i, w, g, p, False, tag)
    cpu_bound = norm_dist.inf_dist_bound
    norm_dist.inf_dist_bound = lambda lo, up, w, g, use_custom_cuda_func=True, tag=None: cpu_bound(lo, up, w, g, False, tag)
    return ref_adamw, bound_module, mlp, model, norm_dist


def hinge_loss(outputs, worst, targets, mix=0.75):
    """mix * mean_b max_j relu(m_bj) + (1 - mix) * mean_bj relu(m_bj) on the worst-case margins."""
    pos = worst.clamp(min=0)
    return mix * pos.max(dim=1)[0].mean() + (1 - mix) * pos.mean()


def ce_loss(outputs, worst, targets):
    return torch.nn.functional.cross_entropy(worst, targets)


def make_adamw(ref_adamw, nd, out):
    gen = torch.Generator().manual_seed(7)
    rows, cols = 37, 300
    for name, p_norm in (("inf", float("inf")), ("p8", 8.0), ("p23", 23.7), ("none", None)):
        w0 = torch.randn(rows, cols, generator=gen)
        b0 = torch.randn(rows, generator=gen)
        if p_norm is None:
            m = torch.nn.Linear(cols, rows)
            m.weight.data = w0.clone(); m.bias.data = b0.clone()
        else:
            m = nd.NormDist(cols, rows, bias=True)
            m.weight.data = w0.clone().view(rows, cols, 1, 1); m.bias.data = b0.clone()
            nd.set_p_norm(m, p_norm)
        opt = ref_adamw.AdamW(m, **HYPER)
        out[f"{name}_w0"] = w0.numpy(); out[f"{name}_b0"] = b0.numpy()
        for step in range(3):
            gw = torch.randn(rows, cols, generator=gen); gb = torch.randn(rows, generator=gen)
            m.weight.grad = gw.clone().view_as(m.weight); m.bias.grad = gb.clone()
            opt.step()
            out[f"{name}_gw{step}"] = gw.numpy(); out[f"{name}_gb{step}"] = gb.numpy()
            out[f"{name}_w{step + 1}"] = m.weight.detach().reshape(rows, cols).numpy().copy()
            out[f"{name}_b{step + 1}"] = m.bias.detach().numpy().copy()


def make_bound_modules(bm, out):
    gen = torch.Generator().manual_seed(11)
    R = lambda *s: torch.randn(*s, generator=gen)
    x = R(9, 64); rad = R(9, 64).abs() * 0.1
    lo, up = x - rad, x + rad
    out["x"] = x.numpy(); out["lo"] = lo.numpy(); out["up"] = up.numpy()
    with torch.no_grad():
        for tag, bias in (("lin", True), ("linnb", False)):
            m = bm.BoundLinear(64, 48, bias=bias)
            m.weight.data = R(48, 64)
            if bias:
                m.bias.data = R(48)
                out[tag + "_b"] = m.bias.numpy().copy()
            out[tag + "_w"] = m.weight.numpy().copy()
            y, l, u = m(x, lo, up)
            out[tag + "_y"] = y.numpy(); out[tag + "_l"] = l.numpy(); out[tag + "_u"] = u.numpy()
            y2, l2, u2 = m(x)
            assert l2 is None and u2 is None and torch.equal(y2, y)
        h, hl, hu = out["lin_y"], out["lin_l"], out["lin_u"]
        h, hl, hu = (torch.from_numpy(t) for t in (h, hl, hu))
        for cls, tag in ((bm.BoundReLU, "relu"), (bm.BoundTanh, "tanh")):
            y, l, u = cls()(h, hl, hu)
            out[tag + "_y"] = y.numpy(); out[tag + "_l"] = l.numpy(); out[tag + "_u"] = u.numpy()
        f = bm.BoundFinalLinear(48, 10)
        f.weight.data = R(10, 48); f.bias.data = R(10)
        targets = torch.randint(0, 10, (9,), generator=gen)
        y, res = f(torch.tanh(h), torch.tanh(hl), torch.tanh(hu), targets=targets)
        out["fin_w"] = f.weight.numpy().copy(); out["fin_b"] = f.bias.numpy().copy()
        out["targets"] = targets.numpy(); out["fin_y"] = y.numpy(); out["fin_res"] = res.numpy()
        assert torch.equal(f(torch.tanh(h)), y)
        ident = bm.BoundFinalIdentity()
        o = R(9, 10); ol = o - 0.3; ou = o + 0.2
        y, res = ident(o, ol, ou, targets=targets)
        out["id_x"] = o.numpy(); out["id_l"] = ol.numpy(); out["id_u"] = ou.numpy(); out["id_res"] = res.numpy()
        for tag, shape in (("mn2", (9, 16)), ("mn4", (4, 16, 3, 3))):
            mn = bm.BoundMeanNorm(16)
            mn.train()
            for call in range(2):
                a = R(*shape); r = R(*shape).abs() * 0.2
                y, l, u = mn(a, a - r, a + r)
                out[f"{tag}_x{call}"] = a.numpy(); out[f"{tag}_r{call}"] = r.numpy()
                out[f"{tag}_y{call}"] = y.numpy(); out[f"{tag}_l{call}"] = l.numpy(); out[f"{tag}_u{call}"] = u.numpy()
                out[f"{tag}_rm{call}"] = mn.running_mean.numpy().copy()
            mn.eval()
            y, l, u = mn(a, a - r, a + r)
            out[f"{tag}_ye"] = y.numpy(); out[f"{tag}_le"] = l.numpy(); out[f"{tag}_ue"] = u.numpy()
        pr = bm.Predictor(64, 32, 10)
        pr.fc1.bias.data = R(32); pr.fc2.bias.data = R(10)
        for k, v in pr.state_dict().items():
            out["pred_sd_" + k] = v.numpy().copy()
        y, res = pr(x, lo, up, targets=targets)
        out["pred_y"] = y.numpy(); out["pred_res"] = res.numpy()


def make_small_nets(ref_adamw, bm, mlp, model, nd, out):
    mlp.net_width = 64
    gen = torch.Generator().manual_seed(21)
    B = 24
    x = torch.rand(B, 3, 8, 8, generator=gen)
    out["x"] = x.numpy()
    for kind in ("mlp", "feat"):
        classes = 10 if kind == "mlp" else 20
        targets = torch.randint(0, classes, (B,), generator=gen)
        out[f"{kind}_targets"] = targets.numpy()
        for pname, p in (("inf", float("inf")), ("p8", 8.0)):
            torch.manual_seed(5)
            if kind == "mlp":
                net = model.Model(mlp.MLP(3, 1, (3, 8, 8), num_classes=classes), bm.BoundFinalIdentity(), eps=8 / 255)
                loss_fn = hinge_loss
            else:
                net = model.Model(mlp.MLPFeature(2, 1, (3, 8, 8)), bm.Predictor(64, 32, classes), eps=1 / 255)
                loss_fn = ce_loss
            # plain random weights: the identity initialisation (a -10 on the diagonal of square layers) makes
            # every sample pick the same input, and behind a mean shift the weight gradient is then rounding
            # noise, which Adam's normalisation turns into steps of +-lr -- nothing a comparison could pin
            for m in net.modules():
                if isinstance(m, nd.NormDist):
                    m.weight.data.normal_()
            nd.set_p_norm(net, p)
            net.train()
            tag = f"{kind}_{pname}"
            for k, v in net.state_dict().items():
                out[f"{tag}_sd0_{k}"] = v.numpy().copy()
            opt = ref_adamw.AdamW(net, **HYPER)
            for step in range(2):
                outputs, worst = net(x, targets=targets)
                loss = loss_fn(outputs, worst, targets)
                opt.zero_grad()
                loss.backward()
                if step == 0:
                    out[f"{tag}_out0"] = outputs.detach().numpy().copy()
                    out[f"{tag}_worst0"] = worst.detach().numpy().copy()
                    for k, q in net.named_parameters():
                        out[f"{tag}_grad0_{k}"] = q.grad.numpy().copy()
                out[f"{tag}_loss{step}"] = np.float32(loss.item())
                opt.step()
            for k, v in net.state_dict().items():
                out[f"{tag}_sd2_{k}"] = v.numpy().copy()
            if pname == "inf":
                # certification pass of main.py:166-194 on the trained state: eval mode, clamped eps box,
                # bounds through every layer, worst-case margins
                net.eval()
                eps = 8 / 255 if kind == "mlp" else 1 / 255
                with torch.no_grad():
                    lower = torch.max(x - eps, torch.zeros(())); upper = torch.min(x + eps, torch.ones(()))
                    outputs, margins = net(x, lower=lower, upper=upper, targets=targets)
                out[f"{tag}_cert_outputs"] = outputs.numpy().copy()
                out[f"{tag}_cert_margins"] = margins.numpy().copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LINF_REFERENCE"), required=os.environ.get("LINF_REFERENCE") is None)
    args = ap.parse_args()
    ref_adamw, bm, mlp, model, nd = load_reference(args.reference)
    torch.set_num_threads(1)
    for name, fn in (("adamw.npz", lambda o: make_adamw(ref_adamw, nd, o)),
                     ("bound_modules.npz", lambda o: make_bound_modules(bm, o)),
                     ("small_nets.npz", lambda o: make_small_nets(ref_adamw, bm, mlp, model, nd, o))):
        out = {}
        fn(out)
        path = os.path.join(HERE, name)
        np.savez_compressed(path, **out)
        print(name, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
