"""CPU: the shared library loads and exports every function include/linfdist.h declares, and
argument validation answers without touching a GPU."""
import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "linfdist.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(linf_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in linfdist.h but not exported"


def test_binding_covers_header(lib):
    from linfdist_b200 import _lib
    assert sorted(_lib.EXPORTED) == _declared()


def test_error_codes_without_gpu(lib):
    assert lib.linf_version() >= 100
    assert lib.linf_error_string(0) == b"ok"
    one = ctypes.c_void_p(256)
    # null pointer
    assert lib.linf_inf_dist_forward(None, one, 1, 1, 1, 1, 1, one, one, None) == 1
    # non-positive dimension
    assert lib.linf_inf_dist_forward(one, one, 0, 1, 1, 1, 1, one, one, None) == 2
    # channels not divisible by the group count
    assert lib.linf_inf_dist_bound_forward(one, one, one, 2, 6, 9, 2, 1, one, one, None) == 3
    assert lib.linf_inf_dist_backward_input(one, one, 2, 5, 8, 2, 1, one, None) == 3
    # p must be finite and > 1
    assert lib.linf_norm_dist_forward(one, one, 2, 4, 4, 1, 1, one, 1.0, None) == 4
    assert lib.linf_norm_dist_forward(one, one, 2, 4, 4, 1, 1, one, float("inf"), None) == 4
    assert lib.linf_norm_dist_backward_weight(one, one, one, one, 2, 4, 4, 1, 1, one, float("nan"), None) == 4
    assert lib.linf_inf_dist_backward_atomic(one, one, 2, 4, 4, 1, 1, None, None, None) == 1
    # tensors beyond int32 element counts are refused
    assert lib.linf_inf_dist_forward(one, one, 1 << 20, 1 << 12, 4, 1, 1, one, one, None) == 2
    assert b"unknown" in lib.linf_error_string(99)


def test_workspace_query(lib):
    # 256 tiles of 64 x 64 on 444 CTA slots, long rows: the k-tiles are dealt evenly to the CTAs, which needs scratch
    assert lib.linf_inf_dist_forward_workspace_bytes(512, 2048, 5120, 1, 1) > 0
    assert lib.linf_inf_dist_forward_workspace_bytes(128, 5120, 5120, 1, 1) > 0
    # 640 tiles of 64 x 64 on 444 slots: run as 856 tiles of 64 x 48 instead, no scratch
    assert lib.linf_inf_dist_forward_workspace_bytes(512, 5120, 5120, 1, 1) == 0
    assert lib.linf_inf_dist_forward_workspace_bytes(512, 5120, 784, 1, 1) == 0
    # conv-shaped and tiny problems take the generic path: no scratch
    assert lib.linf_inf_dist_forward_workspace_bytes(8, 16, 27, 1, 9) == 0
    assert lib.linf_inf_dist_forward_workspace_bytes(0, 16, 27, 1, 9) == 0
