"""The four kernels of the sparse gradient exchange (csrc/sparse_exchange.cu) on ONE GPU: the lists of W made-up
ranks live in ordinary device buffers, which is all the merge kernel needs to know about a peer.  Checked against
the dense sum in rank order, bit for bit.  The bounded wait is made to run out with a flag that nothing sets."""
import numpy as np
import pytest
import torch

from helpers import stream

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


def _sparse_grad(rows, cols, per_row, seed):
    rng = np.random.default_rng(seed)
    g = np.zeros((rows, cols), dtype=np.float32)
    for r in range(rows):
        n = int(rng.integers(0, per_row + 1)) if r % 3 else 0          # many empty rows, as in training
        c = rng.choice(cols, size=min(n, cols), replace=False)
        g[r, c] = rng.standard_normal(len(c)).astype(np.float32)
    return g


@pytest.mark.parametrize("rows,cols,cap,world", [(64, 256, 16, 2), (300, 1000, 40, 4), (5120, 3072, 64, 8), (33, 130, 130, 3),
                                                 (17, 67, 8, 2)])
def test_compact_and_merge_equal_the_dense_sum_in_rank_order(cuda, lib, rows, cols, cap, world):
    dense = [_sparse_grad(rows, cols, min(cap, cols), 50 + q) for q in range(world)]
    scale = np.float32(1.0 / world)
    want = np.zeros((rows, cols), dtype=np.float32)
    for q in range(world):
        want = want + dense[q] * scale                                  # product and sum rounded separately, rank order
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    grads = [torch.from_numpy(d).cuda() for d in dense]
    cnts = [torch.full((rows,), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    ents = [torch.zeros(rows * cap * 2, dtype=torch.int32, device="cuda") for _ in range(world)]
    flags = torch.zeros(world, dtype=torch.int32, device="cuda")
    for q in range(world):
        assert lib.linf_grad_rows_compact(grads[q].data_ptr(), rows, cols, cap, cnts[q].data_ptr(), ents[q].data_ptr(),
                                          err.data_ptr(), stream()) == 0
        assert lib.linf_flag_publish(flags[q:].data_ptr(), 7, stream()) == 0
    torch.cuda.synchronize()
    for q in range(world):
        assert not grads[q].any(), "compaction leaves the dense gradient zero"
        assert np.array_equal(cnts[q].cpu().numpy(), (dense[q] != 0).sum(axis=1))
        e = ents[q].cpu().numpy().reshape(rows, cap, 2)
        for r in range(0, rows, max(1, rows // 50)):
            c = np.nonzero(dense[q][r])[0]                              # ascending columns
            assert np.array_equal(e[r, :len(c), 0], c)
            assert np.array_equal(e[r, :len(c), 1].view(np.float32), dense[q][r, c])
    fp, cp, ep = _ptrs([flags[q:] for q in range(world)]), _ptrs(cnts), _ptrs(ents)
    assert lib.linf_flags_wait(fp.data_ptr(), world, 7, 1000, err.data_ptr(), stream()) == 0
    for q in range(world):                                              # every "rank" merges into its own gradient
        assert lib.linf_grad_rows_merge(grads[q].data_ptr(), rows, cols, cap, cp.data_ptr(), ep.data_ptr(), world,
                                        float(scale), err.data_ptr(), stream()) == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    for q in range(world):
        got = grads[q].cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"rank {q}"


def test_a_flag_that_nobody_raises_ends_the_wait_with_an_error_word(cuda, lib):
    rows, cols, cap = 16, 64, 8
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    flags[0] = 5                                                        # this rank has published step 5; the peer never does
    fp = _ptrs([flags[0:], flags[1:]])
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.linf_flags_wait(fp.data_ptr(), 2, 5, 50, err.data_ptr(), stream()) == 0
    t1.record()
    torch.cuda.synchronize()
    assert int(err.item()) == 1
    assert 40.0 <= t0.elapsed_time(t1) <= 2000.0, "the wait ends at its time limit"
    # every later kernel of the exchange leaves its output alone
    g = torch.zeros(rows, cols, device="cuda")
    cnt = torch.ones(rows, dtype=torch.int32, device="cuda")
    ent = torch.zeros(rows * cap * 2, dtype=torch.int32, device="cuda")
    ent.view(rows, cap, 2)[:, 0, 1] = torch.tensor(1.0).view(torch.int32)
    assert lib.linf_grad_rows_merge(g.data_ptr(), rows, cols, cap, _ptrs([cnt]).data_ptr(), _ptrs([ent]).data_ptr(), 1, 1.0,
                                    err.data_ptr(), stream()) == 0
    torch.cuda.synchronize()
    assert not g.any()
    # a step number already passed counts as reached (the peer is a step ahead)
    err.zero_(); flags[1] = 9
    assert lib.linf_flags_wait(fp.data_ptr(), 2, 5, 50, err.data_ptr(), stream()) == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0


def test_more_nonzeros_than_the_capacity_is_reported(cuda, lib):
    g = torch.ones(4, 32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(4, dtype=torch.int32, device="cuda"); ent = torch.zeros(4 * 8 * 2, dtype=torch.int32, device="cuda")
    assert lib.linf_grad_rows_compact(g.data_ptr(), 4, 32, 8, cnt.data_ptr(), ent.data_ptr(), err.data_ptr(), stream()) == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 2 and cnt.tolist() == [32, 32, 32, 32]


def test_argument_checks(cuda, lib):
    assert lib.linf_grad_rows_compact(None, 4, 32, 8, None, None, None, None) == 1
    assert lib.linf_flag_publish(None, 1, None) == 1
    assert lib.linf_flags_wait(None, 2, 1, 50, None, None) == 1
    e = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.linf_flags_wait(e.data_ptr(), 0, 1, 50, e.data_ptr(), None) == 2
    assert lib.linf_flags_wait(e.data_ptr(), 2, 1, 0, e.data_ptr(), None) == 2
    assert lib.linf_grad_rows_merge(None, 4, 32, 8, None, None, 2, 0.5, None, None) == 1
