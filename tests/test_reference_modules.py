"""Host-side modules and optimiser against outputs of the REFERENCE's own Python (fixtures written by
tests/golden/make_golden_modules.py from adamw.py, model/bound_module.py, model/mlp.py and model/model.py
of zbh2047/L_inf-dist-net, run on the CPU).  The CPU variants run everywhere (the distance operator is
then the CPU checker); the `gpu` variants run the same comparisons through the CUDA library."""
import math
import os

import numpy as np
import pytest
import torch

import linfdist_b200 as L
from helpers import GOLDEN

HYPER = dict(lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def T(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def close(a, b, what, rtol, atol):
    a = a.detach().cpu().double(); b = torch.as_tensor(np.asarray(b)).double()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    err = (a - b).abs()
    bad = err > atol + rtol * b.abs()
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {bad.numel()} entries beyond rtol {rtol}, atol {atol}; "
                                 f"max |a-b| = {float(err.max()):.3e}")


# ---------------------------------------------------------------------------------------------
# AdamW with l_p row decay (adamw.py:30-86)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name,p_norm", [("inf", float("inf")), ("p8", 8.0), ("p23", 23.7), ("none", None)])
def test_adamw_trajectory_matches_reference(device, name, p_norm, request):
    if device == "cuda":
        request.getfixturevalue("cuda"); request.getfixturevalue("lib")
    z = np.load(os.path.join(GOLDEN, "adamw.npz"))
    rows, cols = z[name + "_w0"].shape
    if p_norm is None:
        m = torch.nn.Linear(cols, rows)
        m.weight.data = T(z[name + "_w0"], "cpu"); m.bias.data = T(z[name + "_b0"], "cpu")
    else:
        m = L.NormDist(cols, rows, bias=True)
        m.weight.data = T(z[name + "_w0"], "cpu").view(rows, cols, 1, 1); m.bias.data = T(z[name + "_b0"], "cpu")
        L.set_p_norm(m, p_norm)
    m = m.to(device)
    opt = L.AdamW(m, **HYPER)
    for step in range(3):
        m.weight.grad = T(z[f"{name}_gw{step}"], device).view_as(m.weight)
        m.bias.grad = T(z[f"{name}_gb{step}"], device)
        opt.step()
        # one step moves an entry by about lr = 0.02; the comparison is to rounding of that arithmetic
        close(m.weight.reshape(rows, cols), z[f"{name}_w{step + 1}"], f"weight after step {step + 1}", 2e-5, 2e-6)
        close(m.bias, z[f"{name}_b{step + 1}"], f"bias after step {step + 1}", 2e-5, 2e-6)


# ---------------------------------------------------------------------------------------------
# interval modules (model/bound_module.py:5-116)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
def test_bound_modules_match_reference(device, request):
    if device == "cuda":
        request.getfixturevalue("cuda")
    z = np.load(os.path.join(GOLDEN, "bound_modules.npz"))
    x, lo, up = (T(z[k], device) for k in ("x", "lo", "up"))
    tol = dict(rtol=2e-5, atol=2e-5)           # fp32 GEMMs of length 64 in a different summation order
    with torch.no_grad():
        for tag, bias in (("lin", True), ("linnb", False)):
            m = L.BoundLinear(64, 48, bias=bias).to(device)
            m.weight.data = T(z[tag + "_w"], device)
            if bias:
                m.bias.data = T(z[tag + "_b"], device)
            y, l, u = m(x, lo, up)
            close(y, z[tag + "_y"], tag + " value", **tol); close(l, z[tag + "_l"], tag + " lower", **tol)
            close(u, z[tag + "_u"], tag + " upper", **tol)
            y2, l2, u2 = m(x)
            assert l2 is None and u2 is None
            close(y2, z[tag + "_y"], tag + " value without bounds", **tol)
        h, hl, hu = (T(z[k], device) for k in ("lin_y", "lin_l", "lin_u"))
        for cls, tag in ((L.BoundReLU, "relu"), (L.BoundTanh, "tanh")):
            y, l, u = cls()(h, hl, hu)
            close(y, z[tag + "_y"], tag, 1e-6, 1e-7); close(l, z[tag + "_l"], tag, 1e-6, 1e-7); close(u, z[tag + "_u"], tag, 1e-6, 1e-7)
        f = L.BoundFinalLinear(48, 10).to(device)
        f.weight.data = T(z["fin_w"], device); f.bias.data = T(z["fin_b"], device)
        targets = T(z["targets"], device)
        y, res = f(torch.tanh(h), torch.tanh(hl), torch.tanh(hu), targets=targets)
        close(y, z["fin_y"], "final linear value", **tol); close(res, z["fin_res"], "final linear margins", **tol)
        close(f(torch.tanh(h)), z["fin_y"], "final linear value without bounds", **tol)
        y, res = L.BoundFinalIdentity()(T(z["id_x"], device), T(z["id_l"], device), T(z["id_u"], device), targets=targets)
        close(res, z["id_res"], "identity margins", 0, 0)
        assert torch.equal(y.cpu(), T(z["id_x"], "cpu"))
        for tag in ("mn2", "mn4"):
            mn = L.BoundMeanNorm(16).to(device)
            mn.train()
            for call in range(2):
                a, r = T(z[f"{tag}_x{call}"], device), T(z[f"{tag}_r{call}"], device)
                y, l, u = mn(a, a - r, a + r)
                close(y, z[f"{tag}_y{call}"], f"{tag} value {call}", 1e-5, 1e-6)
                close(l, z[f"{tag}_l{call}"], f"{tag} lower {call}", 1e-5, 1e-6)
                close(u, z[f"{tag}_u{call}"], f"{tag} upper {call}", 1e-5, 1e-6)
                close(mn.running_mean, z[f"{tag}_rm{call}"], f"{tag} running mean {call}", 1e-5, 1e-7)
            mn.eval()
            y, l, u = mn(a, a - r, a + r)
            close(y, z[f"{tag}_ye"], tag + " eval value", 1e-5, 1e-6); close(l, z[f"{tag}_le"], tag + " eval lower", 1e-5, 1e-6)
            close(u, z[f"{tag}_ue"], tag + " eval upper", 1e-5, 1e-6)
        pr = L.Predictor(64, 32, 10).to(device)
        pr.load_state_dict({k[len("pred_sd_"):]: T(z[k], device) for k in z.files if k.startswith("pred_sd_")}, strict=True)
        y, res = pr(x, lo, up, targets=targets)
        close(y, z["pred_y"], "predictor value", **tol); close(res, z["pred_res"], "predictor margins", **tol)


# ---------------------------------------------------------------------------------------------
# two optimisation steps of small nets (model/model.py, model/mlp.py, adamw.py)
# ---------------------------------------------------------------------------------------------
def hinge_loss(outputs, worst, targets, mix=0.75):
    pos = worst.clamp(min=0)
    return mix * pos.max(dim=1)[0].mean() + (1 - mix) * pos.mean()


def ce_loss(outputs, worst, targets):
    return torch.nn.functional.cross_entropy(worst, targets)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("kind", ["mlp", "feat"])
@pytest.mark.parametrize("pname,p", [("inf", float("inf")), ("p8", 8.0)])
def test_small_net_steps_match_reference(device, kind, pname, p, request, monkeypatch):
    """Same start, same batch, two steps of forward / loss / backward / AdamW: activations, gradients,
    losses and parameters follow the reference's CPU run.  The reference's CPU branch differentiates
    y = ||t / n||_p * n with autograd (contributions (g * n) / n, ties split evenly), the CUDA rule is
    a scatter of exactly +-g to the lowest arg-max index: the two agree to rounding on inputs without
    exact ties, which is what the tolerances below state."""
    import linfdist_b200.nets as nets
    monkeypatch.setattr(nets, "UNIT", 64)
    if device == "cuda":
        request.getfixturevalue("cuda"); request.getfixturevalue("lib")
    else:
        import cpu_ops
        cpu_ops.patch(monkeypatch)
    z = np.load(os.path.join(GOLDEN, "small_nets.npz"))
    tag = f"{kind}_{pname}"
    classes = 10 if kind == "mlp" else 20
    if kind == "mlp":
        net = L.Model(L.MLP(3, 1, (3, 8, 8), num_classes=classes), L.BoundFinalIdentity(), eps=8 / 255)
        loss_fn = hinge_loss
    else:
        net = L.Model(L.MLPFeature(2, 1, (3, 8, 8)), L.Predictor(64, 32, classes), eps=1 / 255)
        loss_fn = ce_loss
    sd0 = {k[len(tag) + 5:]: T(z[k], "cpu") for k in z.files if k.startswith(tag + "_sd0_")}
    net.load_state_dict(sd0, strict=True)
    net = net.to(device)
    L.set_p_norm(net, p)
    net.train()
    x = T(z["x"], device); targets = T(z[f"{kind}_targets"], device)
    opt = L.AdamW(net, **HYPER)
    for step in range(2):
        outputs, worst = net(x, targets=targets)
        loss = loss_fn(outputs, worst, targets)
        opt.zero_grad()
        loss.backward()
        if step == 0:
            close(outputs, z[tag + "_out0"], "outputs", 1e-5, 1e-5)
            close(worst, z[tag + "_worst0"], "worst-case margins", 1e-5, 1e-5)
            # gradients: to 1e-6 of the largest gradient entry of the net (entries are signed sums)
            scale = max(float(np.abs(z[f"{tag}_grad0_{k}"]).max()) for k, _ in net.named_parameters())
            for k, q in net.named_parameters():
                close(q.grad, z[f"{tag}_grad0_{k}"], "gradient of " + k, 0.0, 1e-6 * scale)
            assert abs(float(loss.detach()) - float(z[f"{tag}_loss0"])) <= 1e-6 * max(1.0, abs(float(z[f"{tag}_loss0"])))
        else:
            assert abs(float(loss.detach()) - float(z[f"{tag}_loss1"])) <= 1e-4 * max(1.0, abs(float(z[f"{tag}_loss1"])))
        opt.step()
    if device == "cuda":
        torch.cuda.synchronize()
    sd2 = net.state_dict()
    for k in sd0:
        a = sd2[k].detach().cpu().double(); b = torch.from_numpy(z[f"{tag}_sd2_{k}"]).double()
        err = (a - b).abs()
        if math.isinf(p):
            # With eps = 1e-10 Adam moves every entry whose gradient is not exactly zero by about lr per step.
            # A cell whose contributions cancel to exactly zero in one summation order and to rounding noise
            # in the other (the reference's CPU branch multiplies and divides every contribution by the
            # distance first) therefore ends up to 2 * lr apart, and drags the next step's batch means along.
            # Such cells must stay a vanishing fraction; all others agree to rounding.
            off = err > 1e-4
            # (a channel's batch mean moves with ANY entry of its weight row: half of the means may show it)
            limit = 0.5 if "running_mean" in k else 5e-3
            assert off.double().mean() <= limit, f"{k}: {int(off.sum())} of {off.numel()} entries differ by more than 1e-4"
            assert float(err.max()) <= (5e-3 if "running_mean" in k else 5 * HYPER["lr"]), (k, float(err.max()))
        else:
            assert float(err.max()) <= 1e-4, (k, float(err.max()))


# ---------------------------------------------------------------------------------------------
# certification pass (main.py:166-194)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("kind", ["mlp", "feat"])
def test_certify_matches_reference(device, kind, request, monkeypatch):
    """certify() on the reference's trained small net: bounds through every distance layer (fused
    lower/upper kernel), eval-mode mean shift, bias, final margins.  The distance layers are exact
    (max / min of exactly rounded differences), so for the pure distance net the margins must be
    the reference's bit for bit; the dense head of the other net is a GEMM in another order."""
    import linfdist_b200.nets as nets
    monkeypatch.setattr(nets, "UNIT", 64)
    if device == "cuda":
        request.getfixturevalue("cuda"); request.getfixturevalue("lib")
    else:
        import cpu_ops
        cpu_ops.patch(monkeypatch)
    z = np.load(os.path.join(GOLDEN, "small_nets.npz"))
    tag = f"{kind}_inf"
    classes = 10 if kind == "mlp" else 20
    eps = 8 / 255 if kind == "mlp" else 1 / 255
    if kind == "mlp":
        net = L.Model(L.MLP(3, 1, (3, 8, 8), num_classes=classes), L.BoundFinalIdentity(), eps=0.5)
    else:
        net = L.Model(L.MLPFeature(2, 1, (3, 8, 8)), L.Predictor(64, 32, classes), eps=0.5)
    net.load_state_dict({k[len(tag) + 5:]: T(z[k], "cpu") for k in z.files if k.startswith(tag + "_sd2_")}, strict=True)
    net = net.to(device)
    L.set_p_norm(net, 8.0)
    net.train()
    x = T(z["x"], device); targets = T(z[f"{kind}_targets"], device)
    ok, margins = L.certify(net, x, targets, eps, torch.ones((), device=device), torch.zeros((), device=device))
    assert net.training and L.get_p_norm(net) == 8.0 and L.get_eps(net) == 0.5      # state restored
    ref = z[f"{tag}_cert_margins"]
    if kind == "mlp":
        assert np.array_equal(margins.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    else:
        close(margins, ref, "margins", 2e-5, 2e-5)
    assert torch.equal(ok.cpu(), torch.from_numpy(ref).max(dim=1)[1] == T(z[f"{kind}_targets"], "cpu"))
    acc = L.certified_accuracy(net, [(x[:10], targets[:10]), (x[10:], targets[10:])], eps,
                               torch.ones((), device=device), torch.zeros((), device=device))
    assert abs(acc - float(ok.float().mean())) < 1e-6
