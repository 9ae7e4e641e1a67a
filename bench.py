#!/usr/bin/env python
"""Benchmark of the inf-dist layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("step"): one forward + backward of a single inf-dist layer, fp32, groups = 1,
B = 512 per GPU, Din = 784, Dout = 5120 (x ~ U[0,1), w ~ N(0,1), grad_out ~ N(0,1), seeded
synthetic data standing in for MNIST-shaped inputs).  The metric is distance-terms per second,
B*Din*Dout / (t_forward + t_backward), summed over all GPUs (every rank owns its own batch
shard and a weight replica; the layer path itself has no collective).

One JSON line is printed by rank 0.  `value` is measured with inputs resident in HBM, CUDA
events around every step, an L2 flush between steps.  `e2e` repeats the measurement through the
public Python API (norm_dist + autograd) with the step's inputs copied from pinned host memory
and a scalar read back inside the timed region.  `roofline` relates the forward kernel to the
FP32 non-FMA issue peak, `cpu_baseline` times the CPU checker (oracle/) on the host cores.
Further objects of the same line (rank 0's GPU unless stated):
  `lp`            BASELINE configs[1]: L_p layer 512 x 5120 x 5120, p in {8, 16, 64}, forward and both gradients
  `bound`         BASELINE configs[2]: fused lower/upper bounds 512 x 3072 x 5120, groups 1 and 4
  `gpu_baseline`  the reference's own CUDA kernels (compiled for sm_100a) on the headline workload
  `certify`       the certification pass of the CIFAR-shape net (five layers, bounds only) and one PGD step
  `train`, `train_p8`, `train_tiny`  CIFAR-shape (p = inf and p = 8) and TinyImageNet-shape training steps
                  (BASELINE configs[3] and [4]; data parallel over all GPUs of the run, median step time)
`--metric train` makes the CIFAR-shape training samples/s the top-level metric (the layer metric has no
collective in it, so across GPUs it scales by construction; the training step is what exchanges gradients).

`--impl reference` times the CPU restatement of the reference path on the host cores only.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "inf-dist layer distance-terms/s (fwd+bwd)"
UNIT = "terms/s"
B, DIN, DOUT = 512, 784, 5120
WORKLOAD = "inf-dist layer fwd+bwd fp32 G=1: B=512/GPU, Din=784, Dout=5120 (BASELINE configs[0])"
TRAIN_WORKLOAD = ("CIFAR-shape L_inf-dist net training step fp32: 3072-5120x4-10, MeanNorm, eps 8/255, batch 512/GPU, "
                  "p = inf, data parallel (BASELINE configs[3])")
SEED = 2020


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--backward", default="ordered", choices=["ordered", "atomic"],
                    help="ordered = reproducible scatter (bit-exact to the checker); atomic = fused atomics")
    ap.add_argument("--no-train", action="store_true", help="skip the CIFAR-shape training-step measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the lp / bound / gpu_baseline / certify legs")
    ap.add_argument("--train-steps", type=int, default=50)
    ap.add_argument("--train-warmup", type=int, default=10)
    ap.add_argument("--metric", default="layer", choices=["layer", "train"],
                    help="layer: inf-dist layer terms/s is the top-level metric (default); train: CIFAR-shape train samples/s")
    return ap.parse_args()


def seeded_inputs(rank):
    import torch
    gen = torch.Generator().manual_seed(SEED + rank)
    x = torch.rand(B, DIN, 1, generator=gen)
    g = torch.randn(B, DOUT, 1, generator=gen)
    wgen = torch.Generator().manual_seed(SEED)       # every rank holds the same weights
    w = torch.randn(DOUT, DIN, generator=wgen)
    return x, w, g


# --------------------------------------------------------------------------------------------
# CPU leg: the checker (a port of the reference path) on the host cores
# --------------------------------------------------------------------------------------------
def cpu_layer_rate(target_seconds=10.0):
    """terms/s of oracle forward + backward on a batch slice sized for about target_seconds."""
    import numpy as np
    import oracle
    x, w, g = seeded_inputs(0)
    x, w, g = x.numpy(), w.numpy(), g.numpy()
    # All host cores this process may use.  A launcher (torch.distributed.run) exports
    # OMP_NUM_THREADS=1 to its workers and the OpenMP runtime has read that long before this point,
    # so the thread count is set through the runtime's own call.
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    try:
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(cores))
    except OSError:
        cores = int(os.environ.get("OMP_NUM_THREADS", cores))

    def run(nb):
        t0 = time.perf_counter()
        y, pos = oracle.inf_dist_forward(x[:nb], w, 1)
        oracle.inf_dist_backward(g[:nb], pos, DIN, 1)
        return time.perf_counter() - t0

    run(2)                                            # load the library, warm the caches
    probe = run(8)
    nb = int(max(8, min(B, 8 * target_seconds / max(probe, 1e-6))))
    reps, dt = 0, 0.0
    while dt < target_seconds and reps < 1000:        # repeat the slice until the time budget is used
        dt += run(nb)
        reps += 1
    return (reps * nb * DIN * DOUT / dt, cores,
            f"{reps} x forward+backward of {nb} of {B} batch rows, {dt:.2f} s in total")


def cpu_torch_branch_rate(target_seconds=6.0):
    """terms/s of the reference's pure-PyTorch distance branch, restated with the same torch ops
    (model/norm_dist.py:52-57: broadcast difference [B, G, CO/G, CI/G, HW], inf-norm normaliser under
    no_grad, norm of the normalised difference times the normaliser; backward through autograd), on a
    batch chunk of 4 rows at a time so that the temporary stays below 100 MB."""
    import torch
    x, w, g = seeded_inputs(0)
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)))
    p = float("inf")

    def run(rows):
        t0 = time.perf_counter()
        for r0 in range(0, rows, 4):
            xi = x[r0:r0 + 4].clone().requires_grad_(True); wi = w.clone().requires_grad_(True)
            y = xi.view(xi.size(0), 1, 1, -1, xi.size(2)) - wi.view(1, -1, wi.size(-1), 1)
            with torch.no_grad():
                normalize = torch.norm(y, dim=3, p=float("inf"), keepdim=True)
            y = torch.norm(y / normalize, dim=3, p=p, keepdim=True) * normalize
            y.view(y.size(0), -1, y.size(-1)).backward(g[r0:r0 + 4])
        return time.perf_counter() - t0

    run(4)
    rows, dt = 0, 0.0
    while dt < target_seconds and rows < B:
        dt += run(8)
        rows += 8
    return rows * DIN * DOUT / dt, torch.get_num_threads(), f"forward+backward of {rows} of {B} batch rows in chunks of 4, {dt:.2f} s"


def cpu_train_rate(rows=8):
    """samples/s of one CIFAR-shape training step (forward with the eps box, hinge loss, backward, AdamW with
    the l_inf row decay) on the host cores, the distance layers through the CPU checker, on `rows` samples."""
    import numpy as np
    import torch
    import oracle

    class DistF(torch.autograd.Function):          # the checker as an autograd function (p = inf)
        @staticmethod
        def forward(ctx, x, w):
            y, pos = oracle.inf_dist_forward(x.detach().numpy()[:, :, None], w.detach().numpy(), 1)
            ctx.pos, ctx.ci = pos, x.size(1)
            return torch.from_numpy(y[:, :, 0])

        @staticmethod
        def backward(ctx, g):
            gx, gw = oracle.inf_dist_backward(np.ascontiguousarray(g.numpy())[:, :, None], ctx.pos, ctx.ci, 1)
            return torch.from_numpy(gx[:, :, 0]), torch.from_numpy(gw)

    gen = torch.Generator().manual_seed(SEED)
    dims = [3072, 5120, 5120, 5120, 5120, 10]
    ws = [torch.randn(b, a, generator=gen).requires_grad_(True) for a, b in zip(dims, dims[1:])]
    bias = torch.zeros(10, requires_grad=True)
    params = ws + [bias]
    m = [torch.zeros_like(q) for q in params]; v = [torch.zeros_like(q) for q in params]
    x = torch.rand(rows, 3072, generator=gen); t = torch.randint(0, 10, (rows,), generator=gen)
    lr, wd, b1, b2, eps_adam, box = 0.02, 5e-3, 0.9, 0.99, 1e-10, 8 / 255

    def step(k):
        h = x
        for i, w in enumerate(ws):
            h = DistF.apply(h, w)
            h = h - h.mean(dim=0) if i < 4 else -(h + bias)
        lower, upper = h - box, h + box
        worst = (upper - lower.gather(1, t.view(-1, 1))).scatter(1, t.view(-1, 1), 0.0).clamp(min=0)
        loss = 0.75 * worst.max(dim=1)[0].mean() + 0.25 * worst.mean()
        for q in params:
            q.grad = None
        loss.backward()
        with torch.no_grad():
            for q, mq, vq in zip(params, m, v):
                if q.dim() == 2:                 # l_inf row decay: the entry of largest magnitude of every row
                    idx = q.abs().argmax(dim=1, keepdim=True)
                    q.scatter_add_(1, idx, -lr * wd * q.gather(1, idx))
                else:
                    q.mul_(1 - lr * wd)
                mq.mul_(b1).add_(q.grad, alpha=1 - b1); vq.mul_(b2).addcmul_(q.grad, q.grad, value=1 - b2)
                q.addcdiv_(mq, (vq.sqrt() / (1 - b2 ** k) ** 0.5).add_(eps_adam), value=-lr / (1 - b1 ** k))

    step(1)
    t0 = time.perf_counter()
    step(2)
    dt = time.perf_counter() - t0
    return rows / dt, f"one step (forward, loss, backward, AdamW) on {rows} of 512 samples, {dt:.2f} s"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.metric == "train":
        try:
            cores = len(os.sched_getaffinity(0))
        except AttributeError:
            cores = os.cpu_count() or 1
        try:
            import ctypes
            ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(cores))
        except OSError:
            pass
        rates, sample = [], None
        for i in range(min(args.warmup, 1) + min(args.steps, 5)):
            r, sample = cpu_train_rate()
            if i >= min(args.warmup, 1):
                rates.append(r)
        value = statistics.median(rates)
        line = {
            "impl": "reference", "metric": "CIFAR-shape L_inf-dist net train samples/s", "value": value, "unit": "samples/s",
            "n_gpus": args.gpus, "steps": len(rates), "warmup": min(args.warmup, 1), "ms_per_step": 512 / value * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": TRAIN_WORKLOAD, "note": "the training step on the host cores: distance layers through the CPU "
                       "restatement (oracle/linf_oracle.c, OpenMP), everything else torch CPU ops; a bounded batch slice, scaled per sample"},
            "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line), flush=True)
        return
    times = []
    rate = cores = sample = None
    for i in range(args.warmup + args.steps):
        r, cores, sample = cpu_layer_rate(target_seconds=2.0)
        if i >= args.warmup:
            times.append(r)
    value = statistics.median(times)
    nb_terms = B * DIN * DOUT
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": nb_terms / value * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement (oracle/linf_oracle.c, OpenMP) of the reference "
                   "path timed on the host cores; each step is a bounded batch slice, scaled per term"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# GPU leg
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(len(r) >= 6 and r[2 + k] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def _timed_us(torch, fn, flush, n=10, warm=3):
    """Median device time of fn() in microseconds (CUDA events on the current stream, L2 flushed between runs)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(n):
        flush.zero_()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def extra_legs(torch, lib, dev, flush, lane_peak, hbm_peak):
    """Configs 2 and 3, the reference's own kernels on config 1, the certification pass: rank 0's GPU only."""
    import ctypes
    from linfdist_b200 import _lib
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator().manual_seed(SEED + 1)
    out = {}

    # ---- config 2: L_p layer, B = 512, Din = Dout = 5120, x, w, g ~ N(0,1) -------------------------
    Bq, CI, CO = 512, 5120, 5120
    x = torch.randn(Bq, CI, 1, generator=gen).to(dev); w = torch.randn(CO, CI, generator=gen).to(dev)
    g = torch.randn(Bq, CO, 1, generator=gen).to(dev)
    y = torch.empty(Bq, CO, 1, device=dev); gx = torch.empty_like(x); gw = torch.empty_like(w)
    terms = Bq * CI * CO
    lp = {"workload": "L_p layer fp32 G=1: B=512, Din=5120, Dout=5120 (BASELINE configs[1])", "unit": "terms/s",
          "bound": "fp32-issue (integer p: the powers are multiplies on the FP32 pipe; no MUFU on this path)",
          "ops_per_term": "forward: subtract, scale by 1/M, log2(p) squarings, add; each gradient: subtract, scale by 1/y, "
                          "log2(p-2)+1 multiplies for s*|s|^(p-2), multiply by g, add"}
    import math
    for p in (8.0, 16.0, 64.0, 11.3):
        a = (x.data_ptr(), w.data_ptr(), Bq, CO, CI, 1, 1)
        t_f = _timed_us(torch, lambda: _lib.check(lib.linf_norm_dist_forward(*a, y.data_ptr(), p, stream), "lp forward"), flush, n=5, warm=2)
        b = (g.data_ptr(), x.data_ptr(), w.data_ptr(), y.data_ptr(), Bq, CO, CI, 1, 1)
        t_gx = _timed_us(torch, lambda: _lib.check(lib.linf_norm_dist_backward_input(*b, gx.data_ptr(), p, stream), "lp gx"), flush, n=5, warm=2)
        t_gw = _timed_us(torch, lambda: _lib.check(lib.linf_norm_dist_backward_weight(*b, gw.data_ptr(), p, stream), "lp gw"), flush, n=5, warm=2)
        entry = {"us_forward": t_f, "us_grad_input": t_gx, "us_grad_weight": t_gw,
                 "fwd_terms_per_s": terms / (t_f * 1e-6), "fwd_bwd_terms_per_s": terms / ((t_f + t_gx + t_gw) * 1e-6)}
        if p == int(p):
            sq = int(math.log2(p))
            ops_f, ops_b = 3 + sq, 4 + sq          # see ops_per_term; the forward also runs the max pass (2 ops per term)
            entry["frac_fp32_issue_forward"] = (ops_f + 2) * terms / (t_f * 1e-6) / lane_peak
            entry["frac_fp32_issue_backward"] = 2 * ops_b * terms / ((t_gx + t_gw) * 1e-6) / lane_peak
            lp[f"p{int(p)}"] = entry
        else:
            # a p met while annealing: one log2 / exp2 pair per term and pass on the special-function unit
            # (16 lanes per SM and clock), so 2 MUFU operations per term bound each pass
            mufu_peak = lane_peak / 8.0
            entry["bound"] = "mufu"
            entry["frac_mufu_forward"] = 2.0 * terms / (t_f * 1e-6) / mufu_peak
            entry["frac_mufu_backward"] = 2.0 * 2.0 * terms / ((t_gx + t_gw) * 1e-6) / mufu_peak
            lp[f"p{p:g}"] = entry
    out["lp"] = lp

    # ---- the inf-dist layer at the shape that dominates training (5120 -> 5120, B = 512; w, g of config 2) -----------
    # inputs as in the headline workload: x uniform in [0, 1), w ~ N(0,1); the backward is also timed on the arg-max
    # positions of x ~ N(0,1), where a few hundred input coordinates attract most positions of a sample
    pos = torch.empty(Bq, CO, 1, device=dev, dtype=torch.int32)
    need = lib.linf_inf_dist_forward_workspace_bytes(Bq, CO, CI, 1, 1)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
    x_u = torch.rand(Bq, CI, 1, generator=gen).to(dev)
    wide = {"workload": "inf-dist layer fwd+bwd fp32 G=1: B=512, Din=5120, Dout=5120 (the hidden layers of configs 4 and 5)",
            "unit": "terms/s", "note": "2 algorithmic fp32 operations per term, as in `roofline`; the backward adds none"}
    for tag, xin in (("uniform_x", x_u), ("normal_x", x)):
        def wide_fwd():
            a = (xin.data_ptr(), w.data_ptr(), Bq, CO, CI, 1, 1, y.data_ptr(), pos.data_ptr())
            rc = (lib.linf_inf_dist_forward_ws(*a, ws.data_ptr(), need, stream) if need else lib.linf_inf_dist_forward(*a, stream))
            _lib.check(rc, "wide forward")

        t_f = _timed_us(torch, wide_fwd, flush, n=7, warm=2)
        t_b = _timed_us(torch, lambda: _lib.check(lib.linf_inf_dist_backward(
            g.data_ptr(), pos.data_ptr(), Bq, CO, CI, 1, 1, gx.data_ptr(), gw.data_ptr(), stream), "wide backward"), flush, n=7, warm=2)
        wide[tag] = {"us_forward": t_f, "us_backward": t_b, "value": terms / ((t_f + t_b) * 1e-6),
                     "frac_fp32_issue_forward": 2.0 * terms / (t_f * 1e-6) / lane_peak,
                     "frac_fp32_issue_fwd_bwd": 2.0 * terms / ((t_f + t_b) * 1e-6) / lane_peak}
    out["layer_wide"] = wide
    del x_u
    del x, w, g, y, gx, gw, pos, ws

    # ---- config 3: interval bounds, B = 512, Din = 3072, Dout = 5120, groups 1 and 4 ----------------
    Bq, CI, CO = 512, 3072, 5120
    x = torch.rand(Bq, CI, 1, generator=gen)
    lo = (x - 8 / 255).clamp(0, 1).to(dev); up = (x + 8 / 255).clamp(0, 1).to(dev)
    bound = {"workload": "fused lower/upper bounds fp32: B=512, Din=3072, Dout=5120, eps 8/255 clamped to [0,1] (BASELINE configs[2])",
             "unit": "terms/s", "bound": "fp32-issue",
             "algorithmic": "6 fp32 non-FMA ops per term (2 subtracts, max(|tL|,|tU|), max into U, min(|tL|,|tU|), max into L)"}
    for G in (1, 4):
        w = torch.randn(CO, CI // G, generator=gen).to(dev)
        yl = torch.empty(Bq, CO, 1, device=dev); yu = torch.empty_like(yl)
        t = _timed_us(torch, lambda: _lib.check(lib.linf_inf_dist_bound_forward(
            lo.data_ptr(), up.data_ptr(), w.data_ptr(), Bq, CO, CI, G, 1, yl.data_ptr(), yu.data_ptr(), stream), "bound"), flush)
        tg = Bq * CO * (CI // G)
        bound[f"G{G}"] = {"us": t, "terms_per_s": tg / (t * 1e-6), "frac_fp32_issue": 6.0 * tg / (t * 1e-6) / lane_peak}
    out["bound"] = bound
    del lo, up, w, yl, yu

    # ---- the reference's own CUDA kernels on the headline workload ---------------------------------
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libref_norm_dist.so")
    if os.path.exists(ref_path):
        ref = ctypes.CDLL(ref_path)                      # test infrastructure, loaded for this leg only
        x_h, w_h, g_h = seeded_inputs(0)
        x, w, g = x_h.to(dev), w_h.to(dev), g_h.to(dev)
        y = torch.empty(B, DOUT, 1, device=dev); pos = torch.empty(B, DOUT, 1, device=dev, dtype=torch.int32)
        gx = torch.empty_like(x); gw = torch.empty_like(w)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        # the reference launches on the legacy default stream, which torch's current stream is here

        def ref_fwd():
            ref.ref_inf_dist_forward(P(x), P(w), B, DOUT, DIN, 1, 1, P(y), P(pos))

        def ref_bwd():
            gx.zero_(); gw.zero_()                       # model/norm_dist.py:34, 37: the caller zero-fills
            ref.ref_inf_dist_backward_input(P(g), P(pos), B, DOUT, DIN, 1, 1, P(gx))
            ref.ref_inf_dist_backward_weight(P(g), P(pos), B, DOUT, DIN, 1, 1, P(gw))

        t_f = _timed_us(torch, ref_fwd, flush); t_b = _timed_us(torch, ref_bwd, flush)
        out["gpu_baseline"] = {"what": "the reference's own kernels (model/inf_dist_cuda.cu) compiled for sm_100a, same inputs and timing",
                               "workload": WORKLOAD, "us_forward": t_f, "us_backward": t_b,
                               "value": B * DIN * DOUT / ((t_f + t_b) * 1e-6), "unit": UNIT}
        del x, w, g, y, pos, gx, gw
    else:
        out["gpu_baseline"] = {"unavailable": "oracle/_ref/libref_norm_dist.so was not prebuilt"}

    # ---- certification pass and one PGD step on the CIFAR-shape net ---------------------------------
    import linfdist_b200 as L
    from linfdist_b200.train_step import build_cifar_net
    net = build_cifar_net(dev)
    imgs = torch.rand(512, 3, 32, 32, generator=gen).to(dev); labels = torch.randint(0, 10, (512,), generator=gen).to(dev)
    one, zero = torch.ones((), device=dev), torch.zeros((), device=dev)
    t_c = _timed_us(torch, lambda: L.certify(net, imgs, labels, 8 / 255, one, zero), flush, n=5, warm=2)
    t_cv = _timed_us(torch, lambda: L.certify(net, imgs, labels, 8 / 255, one, zero, values=True), flush, n=5, warm=2)
    terms_net = 512 * (3072 * 5120 + 3 * 5120 * 5120 + 5120 * 10)
    atk = L.AttackPGD(net, 8 / 255, 2 / 255, 1, one, zero, random_start=False)
    net.eval()
    t_p = _timed_us(torch, lambda: atk.find(imgs, labels), flush, n=5, warm=2)
    out["certify"] = {"workload": "CIFAR-shape net 3072-5120x4-10, B=512, eps 8/255: lower/upper through five layers with the "
                                  "eval-mode mean shift / bias / sign flip inside the bound kernel, then margins (main.py:166-194 semantics)",
                      "us": t_c, "samples_per_s": 512 / (t_c * 1e-6), "bound_terms_per_s": terms_net / (t_c * 1e-6),
                      "frac_fp32_issue": 6.0 * terms_net / (t_c * 1e-6) / lane_peak,
                      "us_with_values": t_cv, "note": "us_with_values also runs the value forward of every layer, as the reference's loop does; "
                                                      "the margins are the same",
                      "pgd_step_us": t_p, "pgd_note": "one step of AttackPGD: forward, cross entropy, backward to the input only"}
    del net, imgs, labels
    import gc
    gc.collect(); torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    import linfdist_b200 as L
    from linfdist_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # collectives on a high-priority stream: their few CTAs are placed ahead of the queued CTAs
        # of the optimiser / scatter kernels instead of waiting for those grids to drain
        opts = dist.ProcessGroupNCCL.Options()
        opts.is_high_priority_stream = True
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    lib = _lib.load()
    L.set_backward_mode(args.backward)

    x_h, w_h, g_h = seeded_inputs(rank)
    x, w, g = x_h.to(dev), w_h.to(dev), g_h.to(dev)
    terms = B * DIN * DOUT
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)     # > 126 MB of L2
    stream = torch.cuda.current_stream().cuda_stream

    y = torch.empty(B, DOUT, 1, device=dev); pos = torch.empty(B, DOUT, 1, device=dev, dtype=torch.int32)
    gx = torch.empty_like(x); gw = torch.empty_like(w)
    need = lib.linf_inf_dist_forward_workspace_bytes(B, DOUT, DIN, 1, 1)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)

    def fwd():
        if need:
            rc = lib.linf_inf_dist_forward_ws(x.data_ptr(), w.data_ptr(), B, DOUT, DIN, 1, 1, y.data_ptr(),
                                              pos.data_ptr(), ws.data_ptr(), ws.numel(), stream)
        else:
            rc = lib.linf_inf_dist_forward(x.data_ptr(), w.data_ptr(), B, DOUT, DIN, 1, 1, y.data_ptr(),
                                           pos.data_ptr(), stream)
        _lib.check(rc, "forward")

    def bwd():
        if args.backward == "ordered":
            _lib.check(lib.linf_inf_dist_backward(g.data_ptr(), pos.data_ptr(), B, DOUT, DIN, 1, 1,
                                                  gx.data_ptr(), gw.data_ptr(), stream), "backward")
        else:
            gx.zero_(); gw.zero_()
            _lib.check(lib.linf_inf_dist_backward_atomic(g.data_ptr(), pos.data_ptr(), B, DOUT, DIN, 1, 1,
                                                         gx.data_ptr(), gw.data_ptr(), stream), "backward_atomic")


    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident measurement ---------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        fwd(); bwd()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    launches0 = lib.linf_launch_count()
    for s in range(args.steps):
        flush.zero_()
        ev[s][0].record(); fwd(); ev[s][1].record(); bwd(); ev[s][2].record()
    launches = lib.linf_launch_count() - launches0      # kernels of the library launched in the timed region (this rank)
    barrier()
    t_fwd = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps          # ms
    t_bwd = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    ms_step = max_over_ranks(t_fwd + t_bwd)
    t_fwd_max = max_over_ranks(t_fwd)
    value = world * terms / (ms_step * 1e-3)

    # ---- end to end through the Python API, host buffers ----------------------------------
    x_pin, g_pin = x_h.pin_memory(), g_h.pin_memory()
    wp = w.clone().requires_grad_(True)

    copy_stream = torch.cuda.Stream()
    res_pin = torch.zeros(64, dtype=torch.float32).pin_memory()
    e2e_count = [0]

    def issue_copy():
        """This step's host -> device copies, on their own stream so that they can run under the
        previous step's kernels (every step still copies its own inputs from pinned memory)."""
        with torch.cuda.stream(copy_stream):
            xd = x_pin.to(dev, non_blocking=True)
            gd = g_pin.to(dev, non_blocking=True)
            ev = torch.cuda.Event(); ev.record(copy_stream)
        return xd, gd, ev

    def e2e_step(cur, more):
        xd, gd, ev = cur
        nxt = issue_copy() if more else None
        main = torch.cuda.current_stream()
        main.wait_event(ev)
        xd.record_stream(main); gd.record_stream(main)
        xd.requires_grad_(True)
        out = L.norm_dist(xd, wp, 1, float("inf"))
        loss = torch.dot(out.view(-1), gd.view(-1))
        wp.grad = None
        loss.backward()
        # device -> host read of the step's result: an asynchronous 4-byte copy into pinned memory,
        # in stream order behind the backward kernels; the host looks at the values after the loop
        # (a training loop that logs its loss without stalling the GPU every step)
        res_pin[e2e_count[0] % res_pin.numel()].copy_(loss.detach(), non_blocking=True)
        e2e_count[0] += 1
        return nxt

    cur = issue_copy()
    for i in range(3):
        cur = e2e_step(cur, True)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e2e_steps = max(args.steps // 2, 5)
    cur = issue_copy()
    e0.record()
    for i in range(e2e_steps):
        cur = e2e_step(cur, i + 1 < e2e_steps)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)

    # The same loop with only the batch x crossing PCIe (the upstream gradient stays on the device, as
    # it does inside a network): reported beside the strict figure, which is bound by the host -> device
    # copy of grad_output (10.5 of its 12.1 MB per step).
    def issue_copy_x():
        with torch.cuda.stream(copy_stream):
            xd = x_pin.to(dev, non_blocking=True)
            ev = torch.cuda.Event(); ev.record(copy_stream)
        return xd, g, ev

    issue_copy = issue_copy_x
    cur = issue_copy()
    for i in range(3):
        cur = e2e_step(cur, True)
    barrier()
    b0 = torch.cuda.Event(enable_timing=True); b1 = torch.cuda.Event(enable_timing=True)
    cur = issue_copy()
    b0.record()
    for i in range(e2e_steps):
        cur = e2e_step(cur, i + 1 < e2e_steps)
    b1.record()
    barrier()
    e2e_x_ms = max_over_ranks(b0.elapsed_time(b1) / e2e_steps)

    # ---- training steps (CIFAR-shape at p = inf and p = 8, TinyImageNet-shape; data parallel) -------
    train = train_p8 = train_tiny = None
    if not args.no_train:
        from linfdist_b200.train_step import bench_train_step

        def leg(**kw):
            try:
                return bench_train_step(dev, world, rank, steps=args.train_steps, warmup=args.train_warmup, **kw)
            except Exception as exc:                                       # never lose the layer line
                return {"error": repr(exc)}

        train = leg()
        train_p8 = leg(p=8.0)
        train_tiny = leg(config="tiny")

    peaks = {}
    pk_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk_path):
        peaks = json.load(open(pk_path))
    sm_max = float(peaks.get("sm_max_mhz", 1965.0))
    props = torch.cuda.get_device_properties(dev)
    lane_peak = props.multi_processor_count * 128 * sm_max * 1e6           # fp32 lane-ops per second
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    extra = {}
    if rank == 0 and not args.no_extra:
        try:
            extra = extra_legs(torch, lib, dev, flush, lane_peak, hbm_peak)
        except Exception as exc:                                           # never lose the layer line
            extra = {"extra_error": repr(exc)}

    clocks = sampler.stop() if sampler else None      # sampled across the layer, e2e, training and extra legs
    if rank == 0:
        fwd_ops = 2.0 * terms / (t_fwd_max * 1e-3)                         # 1 subtract + 1 max per term
        bwd_bytes = B * DOUT * 8 + (B * DIN + DOUT * DIN) * 4
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "backward": args.backward, "parallelism": f"batch-sharded x{world}",
                       "l2": "256 MB buffer written between timed steps", "ms_forward": t_fwd, "ms_backward": t_bwd},
            "clocks": clocks,
            "e2e": {"value": world * terms / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": x_h.numel() * 4 + g_h.numel() * 4, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms,
                    "batch_only": {"value": world * terms / (e2e_x_ms * 1e-3), "ms_per_step": e2e_x_ms,
                                   "h2d_bytes_per_step": x_h.numel() * 4,
                                   "note": "x from pinned host memory every step, grad_output resident"}},
            "gpu_launches": int(launches),
            "roofline": {
                "bound": "fp32-issue", "kernel": "inf_forward_tiled_kernel",
                "achieved": fwd_ops / 1e12, "peak": lane_peak / 1e12, "unit": "T lane-op/s",
                "frac": fwd_ops / lane_peak,
                "peak_source": f"{props.multi_processor_count} SMs x 128 fp32 lanes x {sm_max:.0f} MHz "
                               "(sm_max_mhz of MEASURED_PEAKS.json; a max is not a multiply-add, so no tensor peak applies)",
                "algorithmic": "2 fp32 non-FMA ops per term (1 subtract, 1 max-of-abs) x B*Din*Dout terms per launch",
                "traffic": 17.8e6, "traffic_note": "dram read+write of one forward launch from the ncu capture "
                           "summarised in profiles/ (compulsory: 17.7 MB in, 21 MB out; the outputs are still in L2 "
                           "when the launch ends)",
                "backward_hbm": {"bound": "hbm", "achieved": bwd_bytes / (t_bwd * 1e-3) / 1e9, "peak": hbm_peak,
                                 "unit": "GB/s", "frac": bwd_bytes / (t_bwd * 1e-3) / 1e9 / hbm_peak},
            },
            "train": train,
            "train_p8": train_p8,
            "train_tiny": train_tiny,
        }
        line.update(extra)
        if args.metric == "train" and train and "value" in train:
            # the training step as the headline: its timed region copies every batch from pinned host
            # memory and ends with the loss read back, so the end-to-end figure is the same measurement
            line["layer"] = {"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms_step}
            line.update({"metric": train["metric"], "value": train["value"], "unit": train["unit"],
                         "ms_per_step": train["ms_per_step"], "steps": train["steps"], "warmup": args.train_warmup})
            line["config"] = dict(line["config"], workload=TRAIN_WORKLOAD, exchange=train.get("exchange"))
            line["e2e"] = {"value": train["value"], "unit": train["unit"], "h2d_bytes_per_step": 512 * 3 * 32 * 32 * 4 + 512 * 8,
                           "d2h_bytes_per_step": 4, "ms_per_step": train["ms_per_step"]}
            line["gpu_launches"] = train.get("gpu_launches", 0)
        if not args.no_cpu:
            rate, cores, sample = cpu_layer_rate()
            line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
            try:
                t_rate, t_threads, t_sample = cpu_torch_branch_rate()
                line["cpu_baseline"]["torch_branch"] = {
                    "value": t_rate, "unit": UNIT, "threads": t_threads, "sample": t_sample,
                    "what": "the reference's pure-PyTorch distance branch (model/norm_dist.py:52-57) restated with the same torch ops"}
            except Exception as exc:
                line["cpu_baseline"]["torch_branch"] = {"error": repr(exc)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
