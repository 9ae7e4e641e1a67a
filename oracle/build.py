"""Builds the checker libraries (test infrastructure, never used by the product).

  oracle/liblinf_oracle.so         gcc -fopenmp build of linf_oracle.c (the CPU restatement)
  oracle/_ref/libref_norm_dist.so  the reference's own two CUDA files, compiled where they lie
                                   together with ref_shim.cu -- only when the reference tree
                                   is present; the result travels to the GPU box as a binary

Run:  python oracle/build.py [--reference /path/to/L_inf-dist-net]
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REFERENCE = "/root/reference"


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(verbose=False):
    src = os.path.join(HERE, "linf_oracle.c")
    out = os.path.join(HERE, "liblinf_oracle.so")
    if _newer(out, [src]):
        cmd = ["gcc", "-O2", "-march=x86-64-v2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
               "-shared", "-fPIC", "-o", out, src, "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return out


def build_reference_kernels(reference=DEFAULT_REFERENCE, verbose=False):
    """Returns the path of the built library, or None when the reference tree is absent."""
    srcs = [os.path.join(reference, "model", f) for f in ("inf_dist_cuda.cu", "norm_dist_cuda.cu")]
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libref_norm_dist.so")
    if not all(os.path.exists(s) for s in srcs):
        return out if os.path.exists(out) else None
    shim = os.path.join(HERE, "ref_shim.cu")
    if _newer(out, srcs + [shim]):
        os.makedirs(out_dir, exist_ok=True)
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--shared",
               "-Xcompiler", "-fPIC", "-o", out, shim] + srcs
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    a = ap.parse_args()
    print(build_oracle(verbose=True))
    print(build_reference_kernels(a.reference, verbose=True))
    sys.exit(0)
