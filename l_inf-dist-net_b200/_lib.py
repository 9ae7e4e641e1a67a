"""ctypes binding of liblinfdist.so (declared in include/linfdist.h) and its nvcc build."""
import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblinfdist.so")
CSRC = os.path.join(_HERE, "csrc")
SOURCES = ["adamw.cu", "api.cu", "epilogue.cu", "sparse_exchange.cu", "inf_forward.cu", "inf_bound.cu", "inf_backward.cu", "inf_backward_accum.cu", "inf_backward_direct.cu", "lp.cu", "lp_tiled.cu", "no_alloc.cu", "skinny.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC"]

_F = ctypes.c_void_p     # device pointers travel as integers
_INT = ctypes.c_int

# name -> argument types (return type is int unless listed in _RESTYPE)
_PROTOS = {
    "linf_version": [],
    "linf_launch_count": [],
    "linf_error_string": [_INT],
    "linf_tune_set": [_INT, _INT],
    "linf_inf_dist_forward": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _F],
    "linf_inf_dist_forward_workspace_bytes": [_INT, _INT, _INT, _INT, _INT],
    "linf_inf_dist_forward_ws": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _F, ctypes.c_size_t, _F],
    "linf_inf_dist_forward_noalloc": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _F],
    "linf_inf_dist_bound_forward": [_F, _F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _F],
    "linf_inf_dist_forward_post": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _INT, _F, _F, ctypes.c_size_t, _F],
    "linf_inf_dist_bound_forward_post": [_F, _F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _INT, _F, _F, _F],
    "linf_mean_shift": [_F, _INT, _INT, _F, ctypes.c_float, _F, _F, _F],
    "linf_grad_rows_compact": [_F, _INT, _INT, _INT, _F, _F, _F, _F],
    "linf_flag_publish": [_F, _INT, _F],
    "linf_flags_wait": [_F, _INT, _INT, _INT, _F, _F],
    "linf_grad_rows_merge": [_F, _INT, _INT, _INT, _F, _F, _INT, ctypes.c_float, _F, _F],
    "linf_inf_dist_backward_input": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F],
    "linf_inf_dist_backward_weight": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F],
    "linf_inf_dist_backward": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _F],
    "linf_inf_dist_backward_atomic": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, _F, _F],
    "linf_adamw_step": [_F, _F, _F, _F, _INT, _INT, ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                        ctypes.c_float, ctypes.c_float, _INT, _F],
    "linf_norm_dist_forward": [_F, _F, _INT, _INT, _INT, _INT, _INT, _F, ctypes.c_float, _F],
    "linf_norm_dist_backward_input": [_F, _F, _F, _F, _INT, _INT, _INT, _INT, _INT, _F, ctypes.c_float, _F],
    "linf_norm_dist_backward_weight": [_F, _F, _F, _F, _INT, _INT, _INT, _INT, _INT, _F, ctypes.c_float, _F],
}
_RESTYPE = {
    "linf_error_string": ctypes.c_char_p,
    "linf_launch_count": ctypes.c_ulonglong,
    "linf_inf_dist_forward_workspace_bytes": ctypes.c_size_t,
}
# the symbols include/linfdist.h declares
EXPORTED = list(_PROTOS)

_lib = None


def build(force=False, verbose=False):
    """Compiles csrc/*.cu for sm_100a into liblinfdist.so next to this file."""
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, "common.cuh"),
                   os.path.join(_HERE, "..", "include", "linfdist.h")]
    if not force and os.path.exists(LIB_PATH):
        t = os.path.getmtime(LIB_PATH)
        if all(os.path.getmtime(d) <= t for d in deps):
            return LIB_PATH
    cmd = ["nvcc"] + NVCC_FLAGS + ["-o", LIB_PATH] + srcs
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    global _lib
    _lib = None
    return LIB_PATH


def load():
    """Returns the loaded library; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` "
                "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _PROTOS.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPE.get(name, ctypes.c_int)
        _lib = lib
    return _lib


def check(rc, what):
    if rc != 0:
        msg = load().linf_error_string(rc).decode()
        raise RuntimeError(f"{what}: {msg} (code {rc})")
