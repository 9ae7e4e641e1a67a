"""Worker of tests/test_gpu_multi.py (one process per GPU, launched with torch.distributed.run): trains a small
L_inf-dist net for a few steps with the plain all-reduce exchange, with the row-sharded exchange (NCCL reduce-scatter /
all-gather around a sharded optimiser) and with the sparse exchange (lists of non-zeros read from peer memory), from
the same start and data, and checks that (1) all leave the same parameters up to summation order -- the sparse
exchange on two ranks the very bits of the all-reduce, (2) the replicas of every run are bit-identical, (3) the sparse
lists were really used, (4) a wait on a late peer's flag ends at its time limit with an error word, not with a hang."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

import linfdist_b200 as L
from linfdist_b200.train_step import DataParallelStep, MarginLoss, ShardedNcclStep, SparseRowsStep, build_cifar_net, hinge


def run(kind, dev, rank, steps=3):
    net = build_cifar_net(dev, depth=3, width=1)
    opt = L.AdamW(net, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
    model = {"sharded": ShardedNcclStep, "nccl": DataParallelStep, "sparse": SparseRowsStep}[kind](net, opt)
    loss_fn = MarginLoss(hinge(0.75), 1.0)
    gen = torch.Generator().manual_seed(100 + rank)
    for _ in range(steps):
        x = torch.rand(64, 3, 32, 32, generator=gen).to(dev)
        t = torch.randint(0, 10, (64,), generator=gen).to(dev)
        out, worst = model(x, targets=t)
        loss = loss_fn(out, worst, t)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        model.finish_step()
    model.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    model.close()
    used = len(model.big) if kind == "sharded" else len(model.lists) if kind == "sparse" else 0
    return [q.detach().clone() for q in net.parameters()], used


def late_peer_check(dev, rank):
    """A peer that is late: rank 0 waits 300 ms for a flag in rank 1's memory that rank 1 raises only after two seconds.
    The wait must end at its limit with the error word set and the context usable; once the flag is up the same
    wait succeeds.  Nobody dies, nothing hangs: the bounded wait is all that is tested."""
    import time
    import torch.distributed._symmetric_memory as symm_mem
    from linfdist_b200 import _lib
    lib = _lib.load()
    world = dist.get_world_size()
    flag = symm_mem.empty(2, dtype=torch.int32, device=dev)
    hdl = symm_mem.rendezvous(flag, dist.group.WORLD.group_name)
    flag.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    peers = [hdl.get_buffer(q, (2,), torch.int32) for q in range(world)]
    ptrs = torch.tensor([t.data_ptr() for t in peers], dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    if rank == 1:
        time.sleep(2.0)
    assert lib.linf_flag_publish(flag.data_ptr(), 7, stream) == 0
    if rank == 0:
        t0 = time.time()
        assert lib.linf_flags_wait(ptrs.data_ptr(), world, 7, 300, err.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        waited = time.time() - t0
        assert int(err.item()) == 1 and 0.25 <= waited < 1.5, (int(err.item()), waited)
        assert float((torch.ones(8, device=dev) * 2).sum().item()) == 16.0          # the context is usable
        err.zero_()
    dist.barrier()                                                                   # rank 1 has published by now
    torch.cuda.synchronize()
    assert lib.linf_flags_wait(ptrs.data_ptr(), world, 7, 2000, err.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    dist.barrier()


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    b, _ = run("nccl", dev, rank)
    a, n_big = run("sharded", dev, rank)
    assert n_big >= 2, "the large weight matrices must take the sharded path"
    for qa, qb in zip(a, b):
        torch.testing.assert_close(qa, qb, rtol=1e-5, atol=1e-6)
    c, n_lists = run("sparse", dev, rank)
    assert n_lists >= 3, "the distance layers' weights must take the sparse path"
    for qc, qb in zip(c, b):
        if dist.get_world_size() == 2:             # halves add exactly: the average of the all-reduce, bit for bit
            assert torch.equal(qc, qb)
        else:
            torch.testing.assert_close(qc, qb, rtol=1e-5, atol=1e-6)
    for params in (a, b, c):                       # replicas identical, bit for bit
        for q in params:
            ref = q.clone()
            dist.broadcast(ref, src=0)
            assert torch.equal(ref, q)
    late_peer_check(dev, rank)
    if rank == 0:
        print("MGPU_OK sharded and sparse exchange on %d ranks, %d sharded tensors, %d sparse lists" % (dist.get_world_size(), n_big, n_lists), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
