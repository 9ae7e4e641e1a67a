"""CPU: the host side above the C ABI -- module surface, state_dict layout, error behaviour,
interval modules, optimiser semantics, and the data-parallel path on two gloo ranks.  Where a
distance layer has to run, the CPU checker stands in for the CUDA operator (tests/cpu_ops.py)."""
import math
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

import linfdist_b200 as L
import cpu_ops


def test_public_surface_matches_reference_names():
    for name in ["DistF", "norm_dist", "inf_dist_bound", "MeanNorm", "NormDistConv", "NormDist", "set_p_norm",
                 "get_p_norm", "BoundReLU", "BoundTanh", "BoundLinear", "BoundFinalLinear", "BoundMeanNorm",
                 "BoundFinalIdentity", "Predictor", "MLP", "MLPFeature", "Model", "set_eps", "get_eps", "AdamW"]:
        assert hasattr(L, name), name


def test_state_dict_layout_and_identity_init():
    torch.manual_seed(0)
    m = L.NormDistConv(6, 10, 3, group=2, bias=True, mean_normalize=True)
    sd = m.state_dict()
    assert sd["weight"].shape == (10, 3, 3, 3) and sd["bias"].shape == (10,)
    assert sd["normalize.running_mean"].shape == (10,)
    # identity init: row i has -10 at channel i % (CI/G), kernel centre
    for i in range(10):
        assert m.weight[i, i % 3, 1, 1].item() == -10.0
    d = L.NormDist(8, 4, bias=False)                  # CI > CO: no identity init
    assert list(d.state_dict().keys()) == ["weight"] and d.weight.shape == (4, 8, 1, 1)
    assert not (d.weight == -10).any()


def test_p_norm_plumbing():
    net = L.MLP(3, 1, (2, 2, 2), num_classes=5)
    assert L.get_p_norm(net) == 0
    L.set_p_norm(net, 11.5)
    assert all(m.p == 11.5 for m in net.modules() if isinstance(m, L.NormDist))
    L.set_p_norm(net, float("inf"))
    assert math.isinf(L.get_p_norm(net))
    assert L.get_p_norm(nn.Linear(2, 2)) is None


def test_errors_without_gpu():
    x, w = torch.rand(2, 4, 1), torch.randn(3, 4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        L.norm_dist(x, w, 1, float("inf"))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        L.inf_dist_bound(x, x, w, 1)
    with pytest.raises(RuntimeError, match="not available"):
        L.norm_dist(x, w, 1, 8.0, use_custom_cuda_func=False)
    with pytest.raises(ValueError):
        L.set_backward_mode("fastest")
    with pytest.raises(ValueError):
        L.AdamW(nn.Linear(2, 2), lr=-1.0)


def test_mean_norm_train_and_eval():
    mn = L.MeanNorm(3, momentum=0.1)
    x = torch.tensor([[1.0, 2.0, 3.0], [3.0, 6.0, 9.0]])
    y = mn(x)
    assert torch.allclose(y.mean(0), torch.zeros(3), atol=1e-6)
    assert torch.allclose(mn.running_mean, torch.tensor([0.2, 0.4, 0.6]))
    mn.eval()
    assert torch.allclose(mn(x), x - mn.running_mean)
    x4 = torch.rand(2, 3, 4, 4)
    mn.train()
    assert torch.allclose(mn(x4).mean(dim=(0, 2, 3)), torch.zeros(3), atol=1e-6)


def test_bound_linear_contains_all_corners():
    torch.manual_seed(1)
    lin = L.BoundLinear(5, 4)
    x = torch.randn(3, 5); lo = x - 0.1; up = x + 0.1
    y, yl, yu = lin(x, lo, up)
    assert (yl <= y + 1e-6).all() and (y <= yu + 1e-6).all()
    for _ in range(50):
        z = lo + (up - lo) * torch.randint(0, 2, x.shape).float()
        yz = lin(z)[0]
        assert (yl <= yz + 1e-5).all() and (yz <= yu + 1e-5).all()
    assert lin(x)[1] is None
    t = L.BoundTanh()
    a, b, c = t(x, lo, up)
    assert torch.equal(b, torch.tanh(lo)) and torch.equal(c, torch.tanh(up))


def test_bound_final_modules():
    torch.manual_seed(2)
    B, C = 4, 6
    x = torch.randn(B, C); lo = x - 0.2; up = x + 0.2
    t = torch.tensor([0, 5, 2, 2])
    out, worst = L.BoundFinalIdentity()(x, lo, up, t)
    assert torch.equal(out, x)
    for b in range(B):
        for j in range(C):
            exp = 0.0 if j == t[b] else (up[b, j] - lo[b, t[b]]).item()
            assert abs(worst[b, j].item() - exp) < 1e-6
    fin = L.BoundFinalLinear(C, 3)
    t3 = torch.tensor([0, 1, 2, 1])
    y, worst = fin(x, lo, up, t3)
    # worst-case margin dominates the margin at any corner of the box; the target row is 0
    for _ in range(30):
        z = lo + (up - lo) * torch.randint(0, 2, x.shape).float()
        yz = fin(z)
        margin = yz - yz.gather(1, t3.view(-1, 1))
        assert (margin <= worst + 1e-5).all()
    assert torch.allclose(worst.gather(1, t3.view(-1, 1)), torch.zeros(B, 1), atol=1e-6)
    assert torch.is_tensor(fin(x))


def test_adamw_decay_rules():
    torch.manual_seed(3)
    net = L.NormDist(6, 4, bias=True)
    lin = nn.Linear(3, 2)
    model = nn.Sequential(net, lin)
    opt = L.AdamW(model, lr=0.1, betas=(0.9, 0.99), eps=1e-10, weight_decay=0.5)
    for p in model.parameters():
        p.grad = torch.zeros_like(p)                  # isolates the decay: Adam's own update is 0
    w0 = net.weight.detach().clone(); b0 = net.bias.detach().clone() + 1.0
    net.bias.data += 1.0
    lw0 = lin.weight.detach().clone()
    # p = inf: only the entry of largest magnitude in each row shrinks by lr*wd
    L.set_p_norm(model, float("inf"))
    opt.step()
    rows = w0.view(4, -1)
    exp = rows.clone()
    idx = rows.abs().argmax(dim=1)
    exp[torch.arange(4), idx] *= (1 - 0.05)
    assert torch.allclose(net.weight.view(4, -1), exp, atol=1e-7)
    assert torch.allclose(net.bias, b0 * (1 - 0.05), atol=1e-7)        # 1-element rows: plain decay
    assert torch.allclose(lin.weight, lw0 * (1 - 0.05), atol=1e-7)     # module without p: uniform decay
    # finite p: x_i -= lr*wd * (|x_i| / ||x||_p)^(p-2) * x_i
    L.set_p_norm(model, 8.0)
    w1 = net.weight.detach().clone().view(4, -1).double()
    opt.step()
    norm = (w1.abs() ** 8).sum(dim=1, keepdim=True) ** (1 / 8)
    exp = w1 - 0.05 * (w1.abs() / norm) ** 6 * w1
    assert torch.allclose(net.weight.view(4, -1).double(), exp, rtol=1e-4, atol=1e-6)


def test_adam_update_matches_torch():
    """With weight_decay = 0 the step is plain Adam with torch's bias correction."""
    torch.manual_seed(4)
    a = nn.Linear(5, 3); b = nn.Linear(5, 3); b.load_state_dict(a.state_dict())
    oa = L.AdamW(a, lr=0.01, betas=(0.9, 0.99), eps=1e-10, weight_decay=0.0)
    ob = torch.optim.Adam(b.parameters(), lr=0.01, betas=(0.9, 0.99), eps=1e-10)
    x = torch.randn(7, 5)
    for _ in range(3):
        for m, o in ((a, oa), (b, ob)):
            o.zero_grad(); m(x).pow(2).sum().backward(); o.step()
    assert torch.allclose(a.weight, b.weight, atol=1e-6) and torch.allclose(a.bias, b.bias, atol=1e-6)


def test_mlp_and_model_wiring(monkeypatch):
    cpu_ops.patch(monkeypatch)
    torch.manual_seed(5)
    net = L.Model(L.MLP(3, 1, (1, 4, 4), num_classes=5), L.BoundFinalIdentity(), eps=0.1)
    L.set_p_norm(net, float("inf"))
    x = torch.rand(6, 1, 4, 4); t = torch.randint(0, 5, (6,))
    net.train()
    out, worst = net(x, targets=t)
    assert out.shape == (6, 5) and worst.shape == (6, 5)
    # training: the box at the output is [out - eps, out + eps]; MLP negates its last layer
    col = t.view(-1, 1)
    exp = ((out + 0.1) - (out - 0.1).gather(1, col)).scatter(1, col, 0.0)
    assert torch.allclose(worst, exp, atol=1e-6)
    # certification: bounds propagated layer by layer enclose the clean output and the eps box is tighter nowhere
    net.eval()
    lo = (x - 0.02).clamp(0, 1); up = (x + 0.02).clamp(0, 1)
    y, ylo, yup = net.feature(x, lo, up)
    assert (ylo <= y + 1e-6).all() and (y <= yup + 1e-6).all()
    for _ in range(5):
        z = lo + (up - lo) * torch.rand_like(x)
        yz = net.feature(z)[0]
        assert (ylo <= yz + 1e-5).all() and (yz <= yup + 1e-5).all()
    assert torch.is_tensor(net(x))                     # no targets: plain logits
    L.set_eps(net, 0.3); assert L.get_eps(net) == 0.3


def test_train_step_decreases_loss_on_cpu(monkeypatch):
    cpu_ops.patch(monkeypatch)
    from linfdist_b200.train_step import MarginLoss, hinge
    torch.manual_seed(6)
    net = L.Model(L.MLP(2, 1, (1, 3, 3), num_classes=3), L.BoundFinalIdentity(), eps=0.01)
    L.set_p_norm(net, 8.0)
    opt = L.AdamW(net, lr=0.05, betas=(0.9, 0.99), eps=1e-10, weight_decay=0.0)
    loss_fn = MarginLoss(hinge(0.75), kappa=1.0)
    x = torch.rand(16, 1, 3, 3); t = torch.randint(0, 3, (16,))
    losses = []
    for _ in range(6):
        out, worst = net(x, targets=t)
        loss = loss_fn(out, worst, t)
        opt.zero_grad(); loss.backward(); opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]


def _ddp_worker(rank, world, port, out, overlapped):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import importlib
    nd = importlib.import_module("linfdist_b200.norm_dist")
    nd.norm_dist = cpu_ops.cpu_norm_dist
    from linfdist_b200.train_step import MarginLoss, hinge
    torch.manual_seed(7)                               # same initial weights on every rank
    net = L.Model(L.MLP(2, 1, (1, 3, 3), num_classes=3), L.BoundFinalIdentity(), eps=0.01)
    L.set_p_norm(net, float("inf"))
    opt = L.AdamW(net, lr=0.05, betas=(0.9, 0.99), eps=1e-10, weight_decay=1e-3)
    if overlapped:
        from linfdist_b200.train_step import DataParallelStep
        ddp = DataParallelStep(net, opt)               # all-reduce + optimiser per parameter inside backward
    else:
        ddp = nn.parallel.DistributedDataParallel(net)
    gen = torch.Generator().manual_seed(100 + rank)    # every rank its own batch shard
    x = torch.rand(8, 1, 3, 3, generator=gen); t = torch.randint(0, 3, (8,), generator=gen)
    loss_fn = MarginLoss(hinge(0.75), kappa=1.0)
    for _ in range(2):
        o, wst = ddp(x, targets=t)
        loss = loss_fn(o, wst, t)
        opt.zero_grad(set_to_none=True); loss.backward()
        if not overlapped:
            opt.step()
        else:
            ddp.finish_step(); ddp.synchronize()
    flat = torch.cat([p.detach().flatten() for p in net.parameters()])
    gathered = [torch.zeros_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    bufs = torch.cat([b.detach().flatten() for b in net.buffers()])
    all_bufs = [torch.zeros_like(bufs) for _ in range(world)]
    dist.all_gather(all_bufs, bufs)
    if rank == 0:
        out.put((bool(all(torch.equal(gathered[0], g) for g in gathered)), gathered[0].numpy().copy(), torch.stack(all_bufs).numpy().copy()))   # plain arrays: the process may exit before the parent reads
    dist.destroy_process_group()


def _run_two_ranks(overlapped):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + (os.getpid() % 400) + (50 if overlapped else 0)
    procs = [ctx.Process(target=_ddp_worker, args=(r, 2, port, out, overlapped)) for r in range(2)]
    for p in procs:
        p.start()
    same, params, bufs = out.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same is True
    return torch.from_numpy(params), torch.from_numpy(bufs)


def test_data_parallel_two_ranks_gloo():
    """Two CPU ranks, different batch shards: parameters stay identical across ranks, and applying
    the optimiser parameter by parameter inside backward gives what a plain DDP step gives."""
    plain, plain_bufs = _run_two_ranks(False)
    overlapped, over_bufs = _run_two_ranks(True)
    assert torch.allclose(plain, overlapped, rtol=1e-6, atol=1e-7)
    # MeanNorm running means: every step starts from rank 0's values and adds the rank's own batch
    # statistics.  DistributedDataParallel broadcasts rank 0's buffers at the start of the NEXT forward, so its
    # ranks end a step with different values; the hand-scheduled step sends them right after the forward
    # (they are then in place long before the next step needs them), so every replica ends the step with
    # rank 0's values -- the values DDP's rank 0 holds, and the ones every rank would start the next step from.
    assert not torch.equal(plain_bufs[0], plain_bufs[1])
    assert torch.allclose(plain_bufs[0], over_bufs[0], rtol=1e-6, atol=1e-7)
    assert torch.equal(over_bufs[0], over_bufs[1])


def test_bench_sharding_inputs():
    import bench
    x0, w0, g0 = bench.seeded_inputs(0)
    x1, w1, g1 = bench.seeded_inputs(1)
    assert x0.shape == (512, 784, 1) and w0.shape == (5120, 784) and g0.shape == (512, 5120, 1)
    assert torch.equal(w0, w1) and not torch.equal(x0, x1)          # weight replicas, distinct batch shards
    assert 0 <= x0.min() and x0.max() < 1
