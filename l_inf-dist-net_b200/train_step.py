"""CIFAR-shape training step of an L_inf-dist net on top of the distance layers: forward with the
eps box at the feature output, hinge loss on the worst-case margins, backward, l_p-decay AdamW
(step semantics of main.py:60-105 and :239-260 of zbh2047/L_inf-dist-net, hyper-parameters of
command/ell_inf_dist_net_cifar10.sh).  Data are synthetic: images ~ U[0,1) of shape 3x32x32,
labels uniform over 10 classes."""
import math

import torch
import torch.nn as nn

from . import _lib
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
        self.handles = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params]
        if self.cuda:
            for m in net.modules():
                own = [q for q in m.parameters(recurse=False) if q.requires_grad]
                if own:
                    self.handles.append(m.register_forward_pre_hook(self._make_wait(own)))

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

    def close(self):
        """Takes the hooks off the network (the hooks hold this object, the object holds the network)."""
        for h in self.handles:
            h.remove()
        self.handles = []


class ShardedNcclStep(DataParallelStep):
    """Data-parallel step with the optimiser sharded by rows: for every large weight matrix (rows
    divisible by the world size) the all-reduce of the base class is split into its two halves --
    a reduce-scatter (average) that leaves rank r with rows [r*s, (r+1)*s) of the gradient, and an
    all-gather of the updated rows -- and the fused optimiser kernel runs in between on those rows
    only, with the Adam moments of those rows only.  Same bytes on the wire as the all-reduce, 1/W of
    the optimiser's HBM traffic and state per rank (0.47 ms of a 4.9 ms step on one GPU).  Every row
    is updated by exactly one rank and then gathered, so the replicas stay bit-identical.  Small
    parameters keep the all-reduce."""

    MIN_BYTES = 1 << 20

    def __init__(self, net, optimizer):
        super().__init__(net, optimizer)
        if not (self.cuda and self.world > 1 and self.avg is not None):
            raise RuntimeError("ShardedNcclStep needs CUDA tensors, NCCL and more than one rank")
        self.rank = self.dist.get_rank()
        self.big = {}
        for p in self.params:
            if p.dim() >= 2 and p.size(0) % self.world == 0 and p.numel() * 4 >= self.MIN_BYTES:
                s = p.size(0) // self.world
                cols = p.numel() // p.size(0)
                self.big[id(p)] = {"s": s, "cols": cols,
                                   "reduced": torch.empty(s, cols, dtype=torch.float32, device=p.device),
                                   "rows": torch.empty(s, cols, dtype=torch.float32, device=p.device)}

    def _issue(self, p):
        b = self.big.get(id(p))
        if b is None:
            return super()._issue(p)
        r, s, cols = self.rank, b["s"], b["cols"]
        work = self.dist.reduce_scatter_tensor(b["reduced"].view(-1), p.grad.view(-1), op=self.avg, async_op=True)
        p.grad.record_stream(self.side)
        with torch.cuda.stream(self.side):
            work.wait()                           # stream-side wait: the host does not block
            self.opt.step_rows(p, r * s, s, b["reduced"])
            b["rows"].copy_(p.data.view(self.world, s, cols)[r], non_blocking=True)
            gather = self.dist.all_gather_into_tensor(p.data.view(-1), b["rows"].view(-1), async_op=True)
            gather.wait()
            ev = self.events.get(id(p))
            if ev is None:
                ev = self.events[id(p)] = torch.cuda.Event()
            ev.record(self.side)


class ShardedCopyEngineStep(DataParallelStep):
    """Data-parallel step for one replica per GPU on an NVLink/NVSwitch node in which the gradient
    exchange of the large weight matrices uses no SM at all:

      * every large parameter (rows divisible by the world size) lives in symmetric memory, so that
        peers can write into it; rank r owns rows [r*s, (r+1)*s) of it together with the Adam moments
        of those rows only (the optimiser state and work are sharded, the row-wise l_p decay makes
        rows the natural unit);
      * when the gradient of such a parameter is ready, rank r PUSHES chunk j of it into a staging
        area on rank j with peer-to-peer copies (copy engines over NVLink) and then raises a flag in
        rank j's memory with a stream memory operation; rank r waits -- again with stream memory
        operations, not kernels -- for the W-1 chunks addressed to it, adds the W chunks in rank
        order, divides by W, runs the fused optimiser kernel on its rows and pushes the updated rows
        into every peer's copy of the parameter, raising a second flag;
      * the next forward waits, layer by layer, for its own update and the W-1 flags of that layer.

    Why not NCCL here: the forward kernels of the wide layers fill every SM for hundreds of
    microseconds per CTA, so a collective kernel launched while they run starts only when they
    end; with all-reduce kernels the exchange of the layers that finish their backward last ends up
    exposed (6.3 ms per step on 8 GPUs against 5.0 ms on one).  Copies and flag operations need no
    SM and run under the forward pass.  Small parameters (biases) keep the NCCL all-reduce of the
    base class.  Every shard is reduced by exactly one rank in a fixed order and then copied, so all
    replicas hold bit-identical parameters.

    A rank that dies leaves its peers waiting on a flag (as a dead rank leaves NCCL waiting): run it
    under a job-level timeout."""

    MIN_BYTES = 1 << 20

    def __init__(self, net, optimizer):
        import torch.distributed as dist
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        super().__init__(net, optimizer)
        if not (self.cuda and self.world > 1):
            raise RuntimeError("ShardedCopyEngineStep needs CUDA tensors and more than one rank")
        self.lib = _lib.load()
        self.rank = dist.get_rank()
        self.copy = torch.cuda.Stream()      # gradient chunks to their owners
        self.push = torch.cuda.Stream()      # updated rows to every replica
        group = dist.group.WORLD.group_name
        W, r = self.world, self.rank
        self.big = {}
        for p in self.params:
            if p.dim() < 2 or p.size(0) % W or p.numel() * 4 < self.MIN_BYTES:
                continue
            rows, cols = p.size(0), p.numel() // p.size(0)
            s = rows // W
            store = symm_mem.empty(p.numel(), dtype=torch.float32, device=p.device)
            stage = symm_mem.empty(p.numel(), dtype=torch.float32, device=p.device)      # [W][s * cols]
            flags = symm_mem.empty(2 * W, dtype=torch.int32, device=p.device)
            flags.zero_()
            store.copy_(p.data.reshape(-1))
            hs, hg, hf = (symm_mem.rendezvous(t, group) for t in (store, stage, flags))
            p.data = store.view(p.shape)
            self.big[id(p)] = {
                "rows": rows, "cols": cols, "s": s, "step": 0, "others": [(r + k) % W for k in range(1, W)],
                "store": store.view(rows, cols), "stage": stage.view(W, s * cols), "flags": flags,
                "peer_store": [hs.get_buffer(j, (rows, cols), torch.float32) for j in range(W)],
                "peer_stage": [hg.get_buffer(j, (W, s * cols), torch.float32) for j in range(W)],
                "peer_flags": [hf.get_buffer(j, (2 * W,), torch.int32) for j in range(W)],
                "reduced": torch.empty(s, cols, dtype=torch.float32, device=p.device),
                "updated": torch.cuda.Event(), "pushed": torch.cuda.Event(),
            }
            b = self.big[id(p)]
            chunk = s * cols * 4
            b["chunk_bytes"] = chunk
            b["bytes"] = (ctypes.c_size_t * (W - 1))(*([chunk] * (W - 1)))
            # gradient chunk r lands in slot r of the owner's staging area; its flag is word r there
            b["d_rs"] = self._ptrs([b["peer_stage"][j][r].data_ptr() for j in b["others"]])
            b["f_rs"] = self._ptrs([b["peer_flags"][j].data_ptr() + 4 * r for j in b["others"]])
            b["f_wait"] = self._ptrs([flags.data_ptr() + 4 * j for j in b["others"]])
            # updated rows of this rank into every replica; flag word W + r there
            b["s_ag"] = self._ptrs([b["store"][r * s:(r + 1) * s].data_ptr()] * (W - 1))
            b["d_ag"] = self._ptrs([b["peer_store"][j][r * s:(r + 1) * s].data_ptr() for j in b["others"]])
            b["f_ag"] = self._ptrs([b["peer_flags"][j].data_ptr() + 4 * (W + r) for j in b["others"]])
            b["f_fwd"] = self._ptrs([flags.data_ptr() + 4 * (W + j) for j in b["others"]])
        torch.cuda.synchronize()
        dist.barrier()

    # ---- grouped peer copies and flag operations: one call into the library per group (no kernel,
    # no SM; csrc/peer_push.cu) ----
    @staticmethod
    def _ptrs(values):
        import ctypes
        return (ctypes.c_void_p * len(values))(*values)

    def _make_wait(self, own):
        base = super()._make_wait(own)

        def wait(module, inputs):
            base(module, inputs)
            cur = torch.cuda.current_stream()
            for q in own:
                b = self.big.get(id(q))
                if b is not None and b["step"] > 0:
                    cur.wait_event(b["updated"])
                    _lib.check(self.lib.linf_flags_wait(self.world - 1, b["f_fwd"], b["step"], cur.cuda_stream), "flags_wait")
        return wait

    def _issue(self, p):
        b = self.big.get(id(p))
        if b is None:
            return super()._issue(p)
        W, r, s, cols = self.world, self.rank, b["s"], b["cols"]
        n = W - 1
        b["step"] += 1
        t = b["step"]
        grad = p.grad.view(W, s * cols)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        p.grad.record_stream(self.copy)
        p.grad.record_stream(self.side)
        # 1. chunks of this rank's gradient to their owners, then the "chunk from r has landed" flags
        self.copy.wait_event(ready)
        g0 = p.grad.data_ptr()
        src = self._ptrs([g0 + j * b["chunk_bytes"] for j in b["others"]])
        _lib.check(self.lib.linf_peer_push(n, b["d_rs"], src, b["bytes"], n, b["f_rs"], t, self.copy.cuda_stream), "peer_push")
        # 2. own shard: wait for the W-1 chunks, add in rank order, average, update the rows
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            if t > 1:
                self.side.wait_event(b["pushed"])     # last step's pushes have read the rows about to change
            b["stage"][r].copy_(grad[r], non_blocking=True)
            _lib.check(self.lib.linf_flags_wait(n, b["f_wait"], t, self.side.cuda_stream), "flags_wait")
            torch.sum(b["stage"].view(W, s, cols), dim=0, out=b["reduced"])
            b["reduced"].mul_(1.0 / W)
            self.opt.step_rows(p, r * s, s, b["reduced"])
            b["updated"].record(self.side)
        # 3. the updated rows to every replica, on a stream of their own so that the next
        #    parameter's reduction does not queue behind these copies
        self.push.wait_event(b["updated"])
        _lib.check(self.lib.linf_peer_push(n, b["d_ag"], b["s_ag"], b["bytes"], n, b["f_ag"], t, self.push.cuda_stream), "peer_push")
        b["pushed"].record(self.push)

    def synchronize(self):
        super().synchronize()
        torch.cuda.current_stream().wait_stream(self.copy)
        torch.cuda.current_stream().wait_stream(self.push)


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
    exchange = "one NCCL all-reduce (avg) per parameter issued as its gradient is ready, optimiser applied per parameter as it arrives"
    model = None
    if world > 1 and device.type == "cuda":
        import os
        kind = os.environ.get("LINF_EXCHANGE", "allreduce")
        if kind == "sharded":
            model = ShardedNcclStep(net, opt)
            exchange = ("per weight matrix a NCCL reduce-scatter (avg) as its gradient is ready, the fused optimiser on this "
                        "rank's rows only, a NCCL all-gather of the updated rows; biases by all-reduce")
        elif kind == "copy":
            try:
                model = ShardedCopyEngineStep(net, opt)
                exchange = ("weight gradients pushed shard by shard over NVLink by the copy engines, flags by stream memory "
                            "operations, optimiser sharded by rows, updated rows pushed back (no SM used by the exchange); "
                            "biases by NCCL all-reduce")
            except Exception as exc:                   # no symmetric memory on this system: NCCL path
                exchange += " (copy-engine exchange unavailable: %r)" % (exc,)
    if model is None:
        model = DataParallelStep(net, opt)
    gen = torch.Generator().manual_seed(4040 + rank)
    images = torch.rand(batch, 3, side, side, generator=gen).pin_memory()
    labels = torch.randint(0, classes, (batch,), generator=gen).pin_memory()
    net.train()

    # Every step copies its batch from pinned host memory; the copy of the NEXT batch is issued on a
    # stream of its own at the start of a step, so that it runs under this step's kernels instead of
    # in front of the first layer (with the copy-engine exchange it would otherwise also queue behind
    # the last parameter pushes of the previous step).
    h2d = torch.cuda.Stream() if device.type == "cuda" else None
    nxt = {}

    def fetch():
        if h2d is None:
            nxt["x"], nxt["t"], nxt["ev"] = images.to(device), labels.to(device), None
            return
        with torch.cuda.stream(h2d):
            nxt["x"] = images.to(device, non_blocking=True)
            nxt["t"] = labels.to(device, non_blocking=True)
            nxt["ev"] = torch.cuda.Event()
            nxt["ev"].record(h2d)

    fetch()

    def step():
        x, t, ev = nxt["x"], nxt["t"], nxt["ev"]
        if ev is not None:
            cur = torch.cuda.current_stream()
            cur.wait_event(ev)
            x.record_stream(cur); t.record_stream(cur)
        fetch()
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
    # give the memory of this leg back before the next one (another model in the same process)
    model.close()
    del model, opt, loss
    if device.type == "cuda":
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    name = "CIFAR-shape L_inf-dist net" if config == "cifar" else "TinyImageNet-shape L_inf-dist net+MLP"
    return {"metric": name + " train samples/s", "value": world * batch / (ms * 1e-3),
            "unit": "samples/s", "ms_per_step": ms, "steps": steps, "batch_per_gpu": batch, "n_gpus": world,
            "p": "inf" if math.isinf(p) else p, "loss": last, "parameters": params,
            "config": what + "; "
                      "n_gpus > 1: data parallel, " + exchange + "; backward mode as --backward"}
