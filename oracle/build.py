"""Builds the checker libraries (test infrastructure, never used by the product).

  oracle/liblinf_oracle.so         gcc -fopenmp build of linf_oracle.c (the CPU restatement)
  oracle/_ref/libref_norm_dist.so  the reference's own two CUDA files, compiled where they lie
                                   together with ref_shim.cu -- only when the reference tree
                                   is present; the result travels to the GPU box as a binary
  baseline/_ref/model/norm_dist.py the reference's Python operator file, copied unmodified for the drop-in test

Run:  python oracle/build.py --reference /path/to/L_inf-dist-net      (or LINF_REFERENCE=/path/...)
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# where the reference checkout lies: --reference on the command line, else this environment variable
DEFAULT_REFERENCE = os.environ.get("LINF_REFERENCE", "")


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
    srcs = [os.path.join(reference or "/nonexistent", "model", f) for f in ("inf_dist_cuda.cu", "norm_dist_cuda.cu")]
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


def stage_reference_python(reference=DEFAULT_REFERENCE, verbose=False):
    """Copies the reference's model/norm_dist.py, unmodified, into baseline/_ref/model/ (a folder that
    is kept out of the repository's history): the drop-in test runs that very file on top of the
    norm_dist_cpp stand-in.  Returns the folder to put on sys.path, or None without a reference tree."""
    import shutil
    src = os.path.join(reference, "model", "norm_dist.py") if reference else ""
    root = os.path.join(os.path.dirname(HERE), "baseline", "_ref")
    dst = os.path.join(root, "model", "norm_dist.py")
    if not src or not os.path.exists(src):
        return root if os.path.exists(dst) else None
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    if _newer(dst, [src]):
        shutil.copyfile(src, dst)
        if verbose:
            print("staged", src, "->", dst)
    return root


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE, required=not DEFAULT_REFERENCE,
                    help="checkout of zbh2047/L_inf-dist-net (or set LINF_REFERENCE)")
    a = ap.parse_args()
    print(build_oracle(verbose=True))
    print(build_reference_kernels(a.reference, verbose=True))
    print(stage_reference_python(a.reference, verbose=True))
    sys.exit(0)
