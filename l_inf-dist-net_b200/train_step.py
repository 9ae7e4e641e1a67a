"""CIFAR-shape training step of an L_inf-dist net on top of the distance layers: forward with the
eps box at the feature output, hinge loss on the worst-case margins, backward, l_p-decay AdamW
(step semantics of main.py:60-105 and :239-260 of zbh2047/L_inf-dist-net, hyper-parameters of
command/ell_inf_dist_net_cifar10.sh).  Data are synthetic: images ~ U[0,1) of shape 3x32x32,
labels uniform over 10 classes."""
import math

import torch
import torch.nn as nn

from .adamw import AdamW
from .bound_module import BoundFinalIdentity
from .nets import MLP, Model
from .norm_dist import set_p_norm


def hinge(mix=0.75):
    """mix * mean_b max_j relu(m_bj) + (1 - mix) * mean_bj relu(m_bj) on margin vectors m."""
    def fn(margins, targets):
        pos = margins.clamp(min=0)
        return mix * pos.max(dim=1)[0].mean() + (1 - mix) * pos.mean()
    return fn


class MarginLoss:
    """kappa * loss(worst-case margins) + (1 - kappa) * loss(clean margins)."""

    def __init__(self, loss, kappa):
        self.loss, self.kappa = loss, kappa

    def __call__(self, outputs, worst, targets):
        clean = outputs - outputs.gather(1, targets.view(-1, 1))
        return self.kappa * self.loss(worst, targets) + (1 - self.kappa) * self.loss(clean, targets)


def build_cifar_net(device, depth=5, width=5, p=float("inf"), eps=8.0 / 255.0, seed=2020):
    torch.manual_seed(seed)
    net = Model(MLP(depth, width, (3, 32, 32), num_classes=10), BoundFinalIdentity(), eps).to(device)
    set_p_norm(net, p)
    return net


def bench_train_step(device, world, rank, steps=8, warmup=3, batch=512, p=float("inf")):
    """Times `steps` optimisation steps (after `warmup`), inputs copied from pinned host memory
    every step.  Returns a dict with samples/s over all ranks (max step time over ranks)."""
    import torch.distributed as dist
    net = build_cifar_net(device, p=p)
    model = nn.parallel.DistributedDataParallel(net, device_ids=[device.index]) if world > 1 else net
    opt = AdamW(net, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
    loss_fn = MarginLoss(hinge(0.75), kappa=1.0)
    gen = torch.Generator().manual_seed(4040 + rank)
    images = torch.rand(batch, 3, 32, 32, generator=gen).pin_memory()
    labels = torch.randint(0, 10, (batch,), generator=gen).pin_memory()
    net.train()

    def step():
        x = images.to(device, non_blocking=True)
        t = labels.to(device, non_blocking=True)
        outputs, worst = model(x, targets=t)
        loss = loss_fn(outputs, worst, t)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    for _ in range(warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    last = float(loss.item())
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    params = sum(q.numel() for q in net.parameters())
    return {"metric": "CIFAR-shape L_inf-dist net train samples/s", "value": world * batch / (ms * 1e-3),
            "unit": "samples/s", "ms_per_step": ms, "steps": steps, "batch_per_gpu": batch, "n_gpus": world,
            "p": "inf" if math.isinf(p) else p, "loss": last, "parameters": params,
            "config": "MLP 3072-5120x4-10, MeanNorm, eps 8/255, hinge(0.75), AdamW lr .02 wd 5e-3; "
                      "DDP gradient all-reduce when n_gpus > 1; backward mode as --backward"}
