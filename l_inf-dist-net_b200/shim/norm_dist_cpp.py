"""Stand-in for the reference's compiled extension `norm_dist_cpp` (model/norm_dist.cpp:92-100 of
zbh2047/L_inf-dist-net): the same seven functions on torch tensors, forwarded to liblinfdist.so.

Put this directory on sys.path ahead of the compiled extension and the reference's unmodified
model/norm_dist.py runs on this library.  Sizes are derived exactly as the reference binding derives
them (model/norm_dist.cpp:26, 37, 49, 59, 71, 80, 88); tensors must be contiguous CUDA tensors
(model/norm_dist.cpp:3-5); the launch goes on torch's current stream.

The library is looked for in LINF_LIB, else next to the package this file ships in.
"""
import ctypes
import os

import torch

_path = os.environ.get("LINF_LIB") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "liblinfdist.so")
if not os.path.exists(_path):
    raise ImportError(f"{_path} is missing: build liblinfdist.so first (there is no CPU fallback)")
_lib = ctypes.CDLL(_path)
_lib.linf_error_string.restype = ctypes.c_char_p


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _s():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ok(rc):
    if rc:
        raise RuntimeError(_lib.linf_error_string(rc).decode())


def _chk(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("tensor must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError("tensor must be contiguous")


def inf_dist_forward(input, weight, output, pos, G):
    _chk(input, weight, output, pos)
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        _ok(_lib.linf_inf_dist_forward(_p(input), _p(weight), B, CO, CI, G, HW, _p(output), _p(pos), _s()))


def inf_dist_bound_forward(input_lower, input_upper, weight, output_lower, output_upper, G):
    _chk(input_lower, input_upper, weight, output_lower, output_upper)
    B, CO, CI, HW = input_lower.size(0), output_lower.size(1), input_lower.size(1), input_lower.size(2)
    with torch.cuda.device(input_lower.device):
        _ok(_lib.linf_inf_dist_bound_forward(_p(input_lower), _p(input_upper), _p(weight), B, CO, CI, G, HW,
                                             _p(output_lower), _p(output_upper), _s()))


def inf_dist_backward_input(grad_output, pos, grad_input, G):
    _chk(grad_output, pos, grad_input)
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_input.size(1), grad_input.size(2)
    with torch.cuda.device(grad_output.device):
        _ok(_lib.linf_inf_dist_backward_input(_p(grad_output), _p(pos), B, CO, CI, G, HW, _p(grad_input), _s()))


def inf_dist_backward_weight(grad_output, pos, grad_weight, G):
    _chk(grad_output, pos, grad_weight)
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_weight.size(1) * G, grad_output.size(2)
    with torch.cuda.device(grad_output.device):
        _ok(_lib.linf_inf_dist_backward_weight(_p(grad_output), _p(pos), B, CO, CI, G, HW, _p(grad_weight), _s()))


def norm_dist_forward(input, weight, output, G, p):
    _chk(input, weight, output)
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        _ok(_lib.linf_norm_dist_forward(_p(input), _p(weight), B, CO, CI, G, HW, _p(output), ctypes.c_float(p), _s()))


def norm_dist_backward_input(grad_output, input, weight, output, grad_input, G, p):
    _chk(grad_output, input, weight, output, grad_input)
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        _ok(_lib.linf_norm_dist_backward_input(_p(grad_output), _p(input), _p(weight), _p(output),
                                               B, CO, CI, G, HW, _p(grad_input), ctypes.c_float(p), _s()))


def norm_dist_backward_weight(grad_output, input, weight, output, grad_weight, G, p):
    _chk(grad_output, input, weight, output, grad_weight)
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        _ok(_lib.linf_norm_dist_backward_weight(_p(grad_output), _p(input), _p(weight), _p(output),
                                                B, CO, CI, G, HW, _p(grad_weight), ctypes.c_float(p), _s()))
