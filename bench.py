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
FP32 non-FMA issue peak, `cpu_baseline` times the CPU checker (oracle/) on the host cores, and
`train` / `train_tiny` report the CIFAR-shape and TinyImageNet-shape training steps (BASELINE
configs[3] and [4]; data parallel over the same GPUs).

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
    ap.add_argument("--train-steps", type=int, default=8)
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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
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

    launches_per_step = 1 + (2 if args.backward == "ordered" else 1)

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
    for s in range(args.steps):
        flush.zero_()
        ev[s][0].record(); fwd(); ev[s][1].record(); bwd(); ev[s][2].record()
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

    # ---- training step (CIFAR-shape net, DDP) ----------------------------------------------
    train = train_tiny = None
    if not args.no_train:
        try:
            from linfdist_b200.train_step import bench_train_step
            train = bench_train_step(dev, world, rank, steps=args.train_steps, warmup=5)
        except Exception as exc:                                           # never lose the layer line
            train = {"error": repr(exc)}
        try:
            train_tiny = bench_train_step(dev, world, rank, steps=args.train_steps, warmup=5, config="tiny")
        except Exception as exc:
            train_tiny = {"error": repr(exc)}

    clocks = sampler.stop() if sampler else None      # sampled across the layer, e2e and training legs
    if rank == 0:
        peaks = {}
        pk_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(pk_path):
            peaks = json.load(open(pk_path))
        sm_max = float(peaks.get("sm_max_mhz", 1965.0))
        props = torch.cuda.get_device_properties(dev)
        lane_peak = props.multi_processor_count * 128 * sm_max * 1e6       # fp32 lane-ops per second
        fwd_ops = 2.0 * terms / (t_fwd_max * 1e-3)                         # 1 subtract + 1 max per term
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
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
            "gpu_launches": launches_per_step * args.steps,
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
            "train_tiny": train_tiny,
        }
        if not args.no_cpu:
            rate, cores, sample = cpu_layer_rate()
            line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
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
