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
from .norm_dist import NormDistConv, get_p_norm, set_p_norm


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
      * parameters are broadcast from rank 0 once; the MeanNorm running means (views of one flat tensor)
        are broadcast from rank 0 right after the forward that updated them and waited for at the start of
        the next step: the same values at the start of every step as DDP's broadcast_buffers gives;
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

    def __init__(self, net, optimizer, eager_bytes=None, urgent_group=True):
        import torch.distributed as dist
        self.net, self.opt = net, optimizer
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.world = self.dist.get_world_size() if self.dist else 1
        self.avg = self.dist.ReduceOp.AVG if (self.dist and self.dist.get_backend() == "nccl") else None
        self.cuda = next(net.parameters()).is_cuda
        self.side = torch.cuda.Stream() if self.cuda else None
        self.side_first = torch.cuda.Stream() if self.cuda else None     # optimiser of the first layer: see below
        self.eager_bytes = eager_bytes
        self.params = [p for p in net.parameters() if p.requires_grad]      # forward (registration) order
        self.first = self.params[0]
        # The gradient of the FIRST layer is ready last and needed first: on the communicator that carries
        # the other layers' all-reduces it would wait behind all of them, and the next forward behind it.
        # It therefore travels on a communicator of its own (every rank issues the collectives of both
        # communicators in the same order, the order of the backward pass), sharing the links with
        # whatever is still in flight instead of queueing, and its optimiser update runs on a stream of
        # its own instead of behind the updates of the other layers (which wait for their all-reduces).
        self.urgent = None
        if self.world > 1 and self.cuda and urgent_group and self.avg is not None:
            opts = self.dist.ProcessGroupNCCL.Options()
            opts.is_high_priority_stream = True
            self.urgent = self.dist.new_group(backend="nccl", pg_options=opts)
        if self.world > 1:
            for p in net.parameters():
                self.dist.broadcast(p.data, src=0)
        # the MeanNorm running means of all layers as views of ONE tensor: one broadcast per step
        self.buffers, self.flat_buffers, self.buffer_work = [], None, None
        if self.world > 1:
            self.buffers = [b for b in net.buffers() if b.dtype == torch.float32]
            if self.buffers:
                self.flat_buffers = torch.cat([b.detach().reshape(-1) for b in self.buffers])
                off = 0
                for b in self.buffers:
                    b.data = self.flat_buffers[off:off + b.numel()].view_as(b)
                    off += b.numel()
        self.events = {}
        self.trace = None               # set to a list to record, per waiting layer, how long the forward stalled
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
            marks = None
            if self.trace is not None:
                marks = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                marks[0].record(cur)
            for q in own:
                ev = self.events.get(id(q))
                if ev is not None:
                    cur.wait_event(ev)
            if marks is not None:
                marks[1].record(cur)
                self.trace.append((type(module).__name__ + str(tuple(own[0].shape)), marks))
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
        side = self.side_first if p is self.first else self.side
        if self.world > 1:
            group = self.urgent if (p is self.first and self.urgent is not None) else None
            work = self.dist.all_reduce(p.grad, op=self.avg, group=group, async_op=True)
        else:
            side.wait_stream(torch.cuda.current_stream())
        p.grad.record_stream(side)
        with torch.cuda.stream(side):
            if work is not None:
                work.wait()                       # stream-side wait: the host does not block
            self.opt.step_params([p])
            ev = self.events.get(id(p))
            if ev is None:
                ev = self.events[id(p)] = torch.cuda.Event()
            ev.record(side)

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
        # Rank 0's running means reach every replica BEFORE the forward touches them (the forward updates
        # them in place).  The broadcast for step t + 1 is queued right after the forward of step t (nothing
        # changes the running means in between), so that it has long landed when step t + 1 begins; the
        # compute stream waits for it there (a stream-side wait, the host does not block).
        if self.flat_buffers is not None:
            if self.buffer_work is None:
                self.buffer_work = self.dist.broadcast(self.flat_buffers, src=0, async_op=self.cuda)
            if self.cuda:
                self.buffer_work.wait()
            self.buffer_work = None
        self.sent = 0
        out = self.net(*a, **k)
        if self.flat_buffers is not None and self.net.training:
            if self.cuda:
                # the collective runs on the communicator's stream: it must see this forward's updates
                self.flat_buffers.record_stream(torch.cuda.current_stream())
            self.buffer_work = self.dist.broadcast(self.flat_buffers, src=0, async_op=self.cuda)
        return out

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
            torch.cuda.current_stream().wait_stream(self.side_first)

    def close(self):
        """Takes the hooks off the network (the hooks hold this object, the object holds the network)."""
        if self.buffer_work is not None and self.cuda:
            self.buffer_work.wait()
        self.buffer_work = None
        for h in self.handles:
            h.remove()
        self.handles = []


class SparseRowsStep(DataParallelStep):
    """Data-parallel step whose p = inf distance layers exchange their gradients as lists of non-zeros,
    read from the peers' memory by a kernel -- no collective, no dense traffic.

    A row of an inf-dist weight gradient has at most B non-zeros (every sample adds to ONE column,
    model/inf_dist_cuda.cu:158-171); in the CIFAR-shape step the five weight gradients together hold a
    few hundred non-zeros in 94 M cells, and the reference's DistributedDataParallel (main.py:290-291)
    all-reduces all 378 MB of them.  Here, per weight and on a side stream behind its gradient:
    linf_grad_rows_compact lists the non-zeros of this rank's rows into symmetric memory (and leaves the
    dense gradient zero), linf_flag_publish raises this rank's flag to the step number, linf_flags_wait
    waits (bounded) for every rank's flag, linf_grad_rows_merge adds value / W of every rank's entries,
    rank by rank, into the dense gradient, and the fused optimiser runs on it.  Every rank adds the same
    numbers in the same order, so the replicas stay bit-identical; for a power-of-two W the result is the
    average an all-reduce gives.  Two lists per weight are used alternately, which makes the stream
    order of the four calls all the synchronisation the ranks need (csrc/sparse_exchange.cu).

    Everything else -- biases, the dense head of the '++' nets, every parameter while p is finite (dense
    gradients) -- takes the all-reduce of the base class.  A wait that runs out (a rank that died or
    fell more than TIMEOUT_MS behind) sets an error word instead of hanging; it is looked at, without
    blocking, at the start of every later step and in synchronize(), and raises there."""

    TIMEOUT_MS = 30000

    def __init__(self, net, optimizer, row_capacity=None):
        """row_capacity: entries a row's list can hold; default = the batch size of the first step, which is
        the most a row can have when every weight is used once per forward pass (a net that runs a layer k
        times per step, e.g. on value, lower and upper bound, needs k times the batch size)."""
        super().__init__(net, optimizer)
        if not (self.cuda and self.world > 1):
            raise RuntimeError("SparseRowsStep needs CUDA tensors and more than one rank")
        self.row_capacity = row_capacity
        import os
        # The exchange reads the peers' lists with plain loads; it never uses multimem instructions.  Keeping the
        # symmetric buffers off an NVLink multicast object means that a rank which dies leaves nothing bound that
        # its peers' GPUs could fault on (PyTorch reads this switch when it sets the allocation up).
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.symm = symm_mem
        self.lib = _lib.load()
        self.rank = self.dist.get_rank()
        self.timeout_ms = int(os.environ.get("LINF_EXCHANGE_TIMEOUT_MS", self.TIMEOUT_MS))
        dev = self.first.device
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.err_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.step_no = 0
        self.batch = 0
        self.lists = {}
        dense = {id(m.weight) for m in net.modules()
                 if isinstance(m, NormDistConv) and m.kernel_size == 1 and m.weight.requires_grad}
        self.sparse_ok = {id(p) for p in self.params if id(p) in dense and p.is_contiguous()}
        # symmetric memory works on this system?  (one small allocation now, so that a system without it
        # fails here, where the caller can still fall back to the all-reduce)
        try:
            probe = symm_mem.empty(4, dtype=torch.int32, device=dev)
            symm_mem.rendezvous(probe, self.dist.group.WORLD.group_name)
        except Exception:
            self.close()                     # take the hooks of the base class off again
            raise

    def _make_lists(self, p, cap):
        """Two lists (odd / even steps) of `cap` entries per row in symmetric memory, and the device
        arrays of every rank's pointers to them.  Collective: every rank gets here for the same
        parameter at the same step."""
        rows, W, dev = p.size(0), self.world, p.device
        group = self.dist.group.WORLD.group_name
        cnt = self.symm.empty(2 * rows, dtype=torch.int32, device=dev)
        ent = self.symm.empty(2 * rows * cap * 2, dtype=torch.int32, device=dev)
        flag = self.symm.empty(2, dtype=torch.int32, device=dev)
        hc, he, hf = (self.symm.rendezvous(t, group) for t in (cnt, ent, flag))
        flag.zero_()
        torch.cuda.synchronize(dev)
        self.dist.barrier()                  # nobody polls a flag that still holds leftovers
        st = {"cap": cap, "cnt": cnt, "ent": ent, "flag": flag, "keep": (hc, he, hf)}
        peers_c = [hc.get_buffer(q, (2, rows), torch.int32) for q in range(W)]
        peers_e = [he.get_buffer(q, (2, rows * cap * 2), torch.int32) for q in range(W)]
        peers_f = [hf.get_buffer(q, (2,), torch.int32) for q in range(W)]
        st["peers"] = (peers_c, peers_e, peers_f)
        for par in (0, 1):
            st[f"cnts{par}"] = torch.tensor([t[par].data_ptr() for t in peers_c], dtype=torch.int64, device=dev)
            st[f"ents{par}"] = torch.tensor([t[par].data_ptr() for t in peers_e], dtype=torch.int64, device=dev)
            st[f"flags{par}"] = torch.tensor([t[par:].data_ptr() for t in peers_f], dtype=torch.int64, device=dev)
        return st

    def _issue(self, p):
        if id(p) not in self.sparse_ok or not math.isinf(get_p_norm(self.net) or 0.0) or self.batch <= 0:
            return super()._issue(p)
        st = self.lists.get(id(p))
        want = self.row_capacity or self.batch
        if st is None or st["cap"] < want:
            st = self.lists[id(p)] = self._make_lists(p, want)
        rows, cols, cap, W = p.size(0), p.numel() // p.size(0), st["cap"], self.world
        par, lib = self.step_no & 1, self.lib
        side = self.side_first if p is self.first else self.side
        side.wait_stream(torch.cuda.current_stream())
        grad = p.grad
        if not grad.is_contiguous():
            return super()._issue(p)
        grad.record_stream(side)
        with torch.cuda.stream(side):
            s, err = side.cuda_stream, self.err.data_ptr()
            mine_c, mine_e = st["cnt"].view(2, rows)[par], st["ent"].view(2, rows * cap * 2)[par]
            _lib.check(lib.linf_grad_rows_compact(grad.data_ptr(), rows, cols, cap, mine_c.data_ptr(),
                                                  mine_e.data_ptr(), err, s), "grad_rows_compact")
            _lib.check(lib.linf_flag_publish(st["flag"][par:].data_ptr(), self.step_no, s), "flag_publish")
            _lib.check(lib.linf_flags_wait(st[f"flags{par}"].data_ptr(), W, self.step_no, self.timeout_ms, err, s),
                       "flags_wait")
            _lib.check(lib.linf_grad_rows_merge(grad.data_ptr(), rows, cols, cap, st[f"cnts{par}"].data_ptr(),
                                                st[f"ents{par}"].data_ptr(), W, 1.0 / W, err, s), "grad_rows_merge")
            self.opt.step_params([p])
            ev = self.events.get(id(p))
            if ev is None:
                ev = self.events[id(p)] = torch.cuda.Event()
            ev.record(side)

    def _check(self, wait=False):
        if wait:
            self.err_host.copy_(self.err)
        code = int(self.err_host[0])
        if code:
            raise RuntimeError("sparse gradient exchange failed: " +
                               ("a rank did not publish its gradient lists in time" if code == 1 else
                                "a gradient row holds more non-zeros than its list has room for (row_capacity)"))

    def __call__(self, *a, **k):
        self._check()
        if self.net.training:
            self.step_no += 1
            self.batch = int(a[0].size(0)) if a and torch.is_tensor(a[0]) else 0
        return super().__call__(*a, **k)

    def finish_step(self):
        super().finish_step()
        with torch.cuda.stream(self.side):
            self.side.wait_stream(self.side_first)
            self.err_host.copy_(self.err, non_blocking=True)      # looked at when the next step starts

    def synchronize(self):
        super().synchronize()
        torch.cuda.current_stream().synchronize()
        self._check(wait=True)


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
    dense = ("one NCCL all-reduce (avg) per parameter issued as its gradient is ready (the first layer's on a communicator of "
             "its own, so that it does not queue behind the others), fused optimiser per parameter as it arrives")
    exchange = "LINF_EXCHANGE=allreduce: " + dense
    model = None
    if world > 1 and device.type == "cuda":
        import os
        kind = os.environ.get("LINF_EXCHANGE", "sparse" if math.isinf(p) else "allreduce")
        if kind == "sharded":
            model = ShardedNcclStep(net, opt)
            exchange = ("LINF_EXCHANGE=sharded: per weight matrix a NCCL reduce-scatter (avg) as its gradient is ready, the fused optimiser on this "
                        "rank's rows only, a NCCL all-gather of the updated rows; biases by all-reduce")
        elif kind == "sparse":
            try:
                model = SparseRowsStep(net, opt)
                exchange = ("LINF_EXCHANGE=sparse: the weight gradient of every p = inf distance layer travels as per-row lists of its "
                            "non-zeros in symmetric memory, read from every peer over NVLink and added in rank order by one kernel "
                            "per weight (no collective, no dense traffic); other parameters: " + dense)
            except Exception as exc:           # no symmetric memory on this system
                exchange = f"LINF_EXCHANGE=allreduce (sparse unavailable: {type(exc).__name__}): " + dense
    if model is None:
        model = DataParallelStep(net, opt)
    gen = torch.Generator().manual_seed(4040 + rank)
    images = torch.rand(batch, 3, side, side, generator=gen).pin_memory()
    labels = torch.randint(0, classes, (batch,), generator=gen).pin_memory()
    net.train()

    # Every step copies its batch from pinned host memory; the copy of the NEXT batch is issued on a
    # stream of its own at the start of a step, so that it runs under this step's kernels instead of
    # in front of the first layer.
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
    # one event per step boundary: the step time is the MEDIAN over the timed steps (a step ends when its
    # last kernel on the compute stream has run; the optimiser updates it issued are waited for by the
    # next step's layers, so over many steps nothing is left out)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    launches = _lib.load().linf_launch_count()
    for k in range(steps):
        loss = step()
        if k == steps - 1:
            model.synchronize()
        marks[k + 1].record()
    launches = _lib.load().linf_launch_count() - launches     # kernels of the library in the timed steps (this rank)
    last = float(loss.item())
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    per_step = sorted(marks[k].elapsed_time(marks[k + 1]) for k in range(steps))
    ms = per_step[len(per_step) // 2]
    ms_mean = marks[0].elapsed_time(marks[steps]) / steps
    if world > 1:
        t = torch.tensor([ms, ms_mean], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_mean = float(t[0].item()), float(t[1].item())
    # How long the forward stood still waiting for updated weights (gradient exchange + optimiser not yet
    # done when the layer was due): a few extra steps with an event pair around every layer's wait.
    stalls = None
    if isinstance(model, DataParallelStep) and device.type == "cuda":
        model.trace = []
        n_trace = 5
        for _ in range(n_trace):
            step()
        model.synchronize()
        torch.cuda.synchronize()
        per_layer = {}
        for name, (a, b) in model.trace:
            per_layer[name] = per_layer.get(name, 0.0) + a.elapsed_time(b) / n_trace
        model.trace = None
        stalls = {"ms_per_step": sum(per_layer.values()), "per_layer_ms": per_layer,
                  "what": "time the compute stream waited at each layer for that layer's updated weights (all-reduce + optimiser), "
                          "mean of %d extra steps after the timed ones" % n_trace}
        if world > 1:
            t = torch.tensor([stalls["ms_per_step"]], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            stalls["ms_per_step_max_over_ranks"] = float(t.item())
        # Timeline of the exchange: how long after the last kernel of the backward pass the update of each
        # parameter has landed (negative: before the backward ended).  Three more steps, each followed by a
        # device synchronisation so that the events can be read; the timed steps above are not affected.
        for q in model.params:
            model.events[id(q)] = torch.cuda.Event(enable_timing=True)
        n_lag, lag, names = 3, {}, {}
        for k, (mname, m) in enumerate(net.named_modules()):
            for q in m.parameters(recurse=False):
                names[id(q)] = f"{mname}:{type(m).__name__}{tuple(q.shape)}"
        for _ in range(n_lag):
            step()
            end_bwd = torch.cuda.Event(enable_timing=True)
            end_bwd.record()
            model.synchronize()
            torch.cuda.synchronize()
            for q in model.params:
                lag[names[id(q)]] = lag.get(names[id(q)], 0.0) + end_bwd.elapsed_time(model.events[id(q)]) / n_lag
        stalls["update_landed_ms_after_backward"] = lag
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
            "unit": "samples/s", "ms_per_step": ms, "ms_per_step_mean": ms_mean, "steps": steps, "warmup": warmup,
            "gpu_launches": int(launches),
            "timing": "median over the timed steps, CUDA events, max over ranks",
            "batch_per_gpu": batch, "n_gpus": world, "exchange": exchange if world > 1 else "none (one GPU)",
            "p": "inf" if math.isinf(p) else p, "loss": last, "parameters": params, "forward_stall": stalls,
            "config": what + "; "
                      "n_gpus > 1: data parallel, " + exchange + "; backward mode as --backward"}
