"""CIFAR-shape training step of an L_inf-dist net on top of the distance layers: forward with the
eps box at the feature output, hinge loss on the worst-case margins, backward, l_p-decay AdamW
(step semantics of main.py:60-105 and :239-260 of zbh2047/L_inf-dist-net, hyper-parameters of
command/ell_inf_dist_net_cifar10.sh).  Data are synthetic: images ~ U[0,1) of shape 3x32x32,
labels uniform over 10 classes."""
import math

import torch
import torch.nn as nn

from .adamw import AdamW
from .bound_module import BoundFinalIdentity, Predictor
from .nets import MLP, MLPFeature, Model
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


def build_tiny_net(device, depth=5, width=5, hidden=512, p=float("inf"), eps=1.0 / 255.0, seed=2020):
    """The '++' variant on TinyImageNet-shaped inputs (3x64x64 = 12288 features, 200 classes): `depth`
    distance layers as feature extractor, then the reference's BoundLinear -> tanh -> BoundFinalLinear
    head (model/bound_module.py:105-116; the reference head uses tanh, not ReLU)."""
    torch.manual_seed(seed)
    feat = MLPFeature(depth, width, (3, 64, 64))
    net = Model(feat, Predictor(feat.out_features, hidden, 200), eps).to(device)
    set_p_norm(net, p)
    return net


def cross_entropy():
    return torch.nn.functional.cross_entropy


class DataParallelStep:
    """Training step of one model replica per GPU, scheduled by hand on top of stock
    torch.distributed collectives (no DistributedDataParallel wrapper):
      * parameters are broadcast from rank 0 once; the MeanNorm running means are broadcast from
        rank 0 at the start of every step (what DDP's broadcast_buffers does);
      * when autograd has accumulated the gradient of a parameter, its all-reduce (average) is
        issued asynchronously and, on a side stream that waits for exactly that all-reduce, the
        optimiser updates that parameter; the next forward waits, layer by layer, only for the
        update of the layer it is about to run;
      * gradients become ready last layer first, but the next forward needs the first layer
        first.  `eager_bytes` (off by default) caps what is sent while the backward still runs; the
        rest is then held back until the parameter that the forward needs first is on the wire and
        follows in forward order behind the next forward pass.  Measured on B200 this loses: the
        forward kernels fill every SM, so a collective queued behind them starts only when they
        end (6.09 ms vs 5.64 ms per step on 2 GPUs), hence the default sends everything at once.
    The arithmetic is that of a plain data-parallel step (every parameter is updated with its
    averaged gradient before its next use); only the order of launches differs.  With one rank
    there is no communication and the same schedule overlaps the optimiser with the passes."""

    def __init__(self, net, optimizer, eager_bytes=None):
        import torch.distributed as dist
        self.net, self.opt = net, optimizer
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.world = self.dist.get_world_size() if self.dist else 1
        self.avg = self.dist.ReduceOp.AVG if (self.dist and self.dist.get_backend() == "nccl") else None
        self.cuda = next(net.parameters()).is_cuda
        self.side = torch.cuda.Stream() if self.cuda else None
        self.eager_bytes = eager_bytes
        self.params = [p for p in net.parameters() if p.requires_grad]      # forward (registration) order
        self.first = self.params[0]
        if self.world > 1:
            for p in net.parameters():
                self.dist.broadcast(p.data, src=0)
        self.buffers = list(net.buffers()) if self.world > 1 else []
        self.events = {}
        self.sent, self.held = 0, []
        for p in self.params:
            p.register_post_accumulate_grad_hook(self._on_grad)
        if self.cuda:
            for m in net.modules():
                own = [q for q in m.parameters(recurse=False) if q.requires_grad]
                if own:
                    m.register_forward_pre_hook(self._make_wait(own))

    def _make_wait(self, own):
        def wait(module, inputs):
            cur = torch.cuda.current_stream()
            for q in own:
                ev = self.events.get(id(q))
                if ev is not None:
                    cur.wait_event(ev)
        return wait

    def _issue(self, p):
        """All-reduce (if any) and optimiser update of one parameter, behind the current stream."""
        if not self.cuda:
            if self.world > 1:
                p.grad.div_(self.world)
                self.dist.all_reduce(p.grad)
            self.opt.step_params([p])
            return
        work = None
        if self.world > 1:
            work = self.dist.all_reduce(p.grad, op=self.avg, async_op=True)
        else:
            self.side.wait_stream(torch.cuda.current_stream())
        p.grad.record_stream(self.side)
        with torch.cuda.stream(self.side):
            if work is not None:
                work.wait()                       # stream-side wait: the host does not block
            self.opt.step_params([p])
            ev = self.events.get(id(p))
            if ev is None:
                ev = self.events[id(p)] = torch.cuda.Event()
            ev.record(self.side)

    def _on_grad(self, p):
        nbytes = p.grad.numel() * p.grad.element_size()
        if p is self.first:
            self._issue(p)
            order = {id(q): k for k, q in enumerate(self.params)}
            for q in sorted(self.held, key=lambda t: order[id(t)]):
                self._issue(q)
            self.held = []
        elif self.world == 1 or self.eager_bytes is None or self.sent + nbytes <= self.eager_bytes:
            self.sent += nbytes
            self._issue(p)
        else:
            self.held.append(p)

    def __call__(self, *a, **k):
        for b in self.buffers:
            self.dist.broadcast(b, src=0, async_op=self.cuda)
        self.sent = 0
        return self.net(*a, **k)

    def finish_step(self):
        """Call after loss.backward().  Parameters whose gradient never arrived through the hook of
        the first parameter (a net whose first parameter got no gradient) are flushed here."""
        for q in self.held:
            self._issue(q)
        self.held = []

    def synchronize(self):
        """Makes the current stream wait for every update issued so far."""
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.side)


def bench_train_step(device, world, rank, steps=8, warmup=3, batch=None, p=float("inf"), config="cifar"):
    """Times `steps` optimisation steps (after `warmup`), inputs copied from pinned host memory
    every step.  Returns a dict with samples/s over all ranks (max step time over ranks).
    config "cifar": 3x32x32 inputs, 5 distance layers 3072-5120x4-10, batch 512 per GPU, hinge loss;
    config "tiny" : 3x64x64 inputs, 5 distance layers of width 5120 + tanh MLP head 5120-512-200,
                    batch 256 per GPU, cross entropy on the worst-case margins."""
    import torch.distributed as dist
    if config == "cifar":
        batch = batch or 512
        net = build_cifar_net(device, p=p)
        opt = AdamW(net, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
        loss_fn = MarginLoss(hinge(0.75), kappa=1.0)
        side, classes = 32, 10
        what = "MLP 3072-5120x4-10, MeanNorm, eps 8/255, hinge(0.75), fused AdamW lr .02 wd 5e-3"
    else:
        batch = batch or 256
        net = build_tiny_net(device, p=p)
        opt = AdamW(net, lr=0.04, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
        loss_fn = MarginLoss(cross_entropy(), kappa=1.0)
        side, classes = 64, 200
        what = ("MLPFeature 12288-5120x5 + head 5120-512(tanh)-200, MeanNorm, eps 1/255, cross entropy, "
                "fused AdamW lr .04 wd 5e-3")
    model = DataParallelStep(net, opt)
    gen = torch.Generator().manual_seed(4040 + rank)
    images = torch.rand(batch, 3, side, side, generator=gen).pin_memory()
    labels = torch.randint(0, classes, (batch,), generator=gen).pin_memory()
    net.train()

    def step():
        x = images.to(device, non_blocking=True)
        t = labels.to(device, non_blocking=True)
        outputs, worst = model(x, targets=t)
        loss = loss_fn(outputs, worst, t)
        opt.zero_grad(set_to_none=True)
        loss.backward()                   # all-reduce + optimiser run per parameter inside
        model.finish_step()
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
    model.synchronize()
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
    name = "CIFAR-shape L_inf-dist net" if config == "cifar" else "TinyImageNet-shape L_inf-dist net+MLP"
    return {"metric": name + " train samples/s", "value": world * batch / (ms * 1e-3),
            "unit": "samples/s", "ms_per_step": ms, "steps": steps, "batch_per_gpu": batch, "n_gpus": world,
            "p": "inf" if math.isinf(p) else p, "loss": last, "parameters": params,
            "config": what + "; "
                      "n_gpus > 1: data parallel, one NCCL all-reduce (avg) per parameter issued as its gradient is "
                      "ready, optimiser applied per parameter as it arrives; backward mode as --backward"}
