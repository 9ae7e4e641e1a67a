"""GPU: the forward entry point that allocates nothing (scratch in a fixed device array inside
the library, for callers whose device memory is planned up front and who therefore cannot hand in
a workspace) must give exactly what the workspace-taking entry point gives.  Kept in a file that
sorts last, so that a failure here cannot hide the result of any other test; it also has to pass
when run alone in a fresh process, which is why it sets up everything it needs itself."""
import numpy as np
import pytest
import torch

from helpers import assert_bits_equal, c_inf_forward, dev, make_inputs, stream

pytestmark = pytest.mark.gpu


def _noalloc_forward(lib, x, w, G):
    B, CI, HW = x.shape; CO = w.shape[0]
    y = torch.full((B, CO, HW), float("nan"), device=x.device)
    pos = torch.full((B, CO, HW), -7, device=x.device, dtype=torch.int32)
    rc = lib.linf_inf_dist_forward_noalloc(x.data_ptr(), w.data_ptr(), B, CO, CI, G, HW,
                                           y.data_ptr(), pos.data_ptr(), stream())
    assert rc == 0, lib.linf_error_string(rc)
    return y, pos


@pytest.mark.parametrize("shape", [(512, 784, 5120, 1, 1), (33, 100, 65, 1, 1), (130, 784, 200, 1, 1),
                                   (16, 64, 256, 1, 4), (7, 17, 10, 1, 1),
                                   # wide layers: the k-range is dealt out to every CTA slot of the GPU, so the
                                   # parked partial tiles reach (almost) the end of the library's fixed array
                                   (512, 5120, 2048, 1, 1), (128, 5120, 5120, 1, 1), (512, 5120, 5120, 1, 1), (512, 784, 2560, 1, 1)],
                         ids=lambda s: "B{}_CI{}_CO{}_HW{}_G{}".format(*s))
def test_noalloc_forward_matches_workspace_forward_twice(cuda, lib, shape):
    B, CI, CO, HW, G = shape
    x, w, _ = make_inputs(B, CI, CO, HW, G, seed=7000 + CO)
    xd, wd = dev(x), dev(w)
    y_ref, pos_ref = c_inf_forward(xd, wd, G, use_ws=True)
    torch.cuda.synchronize()
    if (B, CI, CO) in ((512, 5120, 2048), (128, 5120, 5120)):
        # these shapes must really exercise the scratch array, close to its full extent
        need = lib.linf_inf_dist_forward_workspace_bytes(B, CO, CI, G, HW)
        assert 0.8 * 30 * 1024 * 1024 <= need <= 30 * 1024 * 1024, need
    for call in range(2):                               # the second call meets the first call's leftovers
        y, pos = _noalloc_forward(lib, xd, wd, G)
        torch.cuda.synchronize()
        assert_bits_equal(y, y_ref, f"values, call {call}")
        assert_bits_equal(pos, pos_ref, f"arg-max, call {call}")
    # a different layer right after, through the same shared array
    x2, w2, _ = make_inputs(40, 128, 96, 1, 1, seed=7001)
    y2_ref, pos2_ref = c_inf_forward(dev(x2), dev(w2), 1, use_ws=True)
    y2, pos2 = _noalloc_forward(lib, dev(x2), dev(w2), 1)
    assert_bits_equal(y2, y2_ref, "values after a shape change")
    assert_bits_equal(pos2, pos2_ref, "arg-max after a shape change")


def test_noalloc_argument_checks(cuda, lib):
    x = torch.rand(4, 8, 1, device="cuda"); w = torch.randn(6, 8, device="cuda")
    y = torch.empty(4, 6, 1, device="cuda"); pos = torch.empty(4, 6, 1, device="cuda", dtype=torch.int32)
    assert lib.linf_inf_dist_forward_noalloc(None, w.data_ptr(), 4, 6, 8, 1, 1, y.data_ptr(), pos.data_ptr(), None) == 1
    assert lib.linf_inf_dist_forward_noalloc(x.data_ptr(), w.data_ptr(), 4, 6, 8, 3, 1, y.data_ptr(), pos.data_ptr(), None) == 3
