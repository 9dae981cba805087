"""Compile the reference's own CUDA extension, in place, for sm_100a.

TEST INFRASTRUCTURE ONLY.  Nothing in the product imports this file or its output.

The two pybind11 modules of the reference (``lpmm/cpp_extension/fused_adamw*.{cc,cu}`` and
``lpmm/cpp_extension/quantization*.{cc,cu}``, built upstream by ``setup.py:21-30``) are compiled
from the sources where they lie in the read-only reference checkout.  Only the resulting shared
objects are written, into ``oracle/_ref/`` (git-ignored).  No reference source is copied.

``copy_python`` additionally places the reference's Python layer (``lpmm/*.py``, ``lpmm/optim``,
``lpmm/configs``; no native sources) under ``oracle/_ref/lpmm_py/`` -- the same thing an install of the
reference into a git-ignored directory would do -- so that ``bench.py --impl reference`` can time the
reference's own CPU path on a machine that has no reference checkout.  ``oracle/_ref`` is git-ignored:
nothing of it enters the repository's history.

The GPU parity tests load these modules, when present, as the authoritative result of the
reference kernels on the same inputs.  The flags mirror what the reference's ``setup.py`` gives
``CUDAExtension`` (no optimisation or fast-math flags of its own: nvcc defaults, i.e.
``-fmad=true``, IEEE division and square root), plus the sm_100a ``-gencode``.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--only fused_adamw|quantization|python]

The reference checkout is looked for at ``--reference``, else ``$LPMM_REFERENCE_ROOT``, else a directory
named ``reference`` beside this repository.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

MODULES = {
    "fused_adamw": ["fused_adamw.cc", "fused_adamw_kernel.cu"],
    "quantization": ["quantization.cc", "quantization_kernel.cu"],
}


PY_OUT = os.path.join(OUT, "lpmm_py")


def reference_root(explicit=None):
    """Where the reference checkout is: the argument, ``$LPMM_REFERENCE_ROOT``, or ``../reference`` seen from
    the repository root.  Returns None when there is none."""
    for cand in (explicit, os.environ.get("LPMM_REFERENCE_ROOT"),
                 os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "lpmm", "cpp_extension")):
            return cand
    return None


def copy_python(root: str) -> str:
    """The reference's Python layer (no native sources) into ``oracle/_ref/lpmm_py/lpmm``."""
    src = os.path.join(root, "lpmm")
    dst = os.path.join(PY_OUT, "lpmm")
    os.makedirs(dst, exist_ok=True)
    for name in os.listdir(src):
        if name.endswith(".py"):
            shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
    for sub, suffix in (("optim", ".py"), ("configs", ".yml")):
        os.makedirs(os.path.join(dst, sub), exist_ok=True)
        for name in os.listdir(os.path.join(src, sub)):
            if name.endswith(suffix):
                shutil.copyfile(os.path.join(src, sub, name), os.path.join(dst, sub, name))
    return PY_OUT


def have_python() -> bool:
    return os.path.exists(os.path.join(PY_OUT, "lpmm", "optim", "adamw.py"))


def build(reference_root: str, only=None, verbose=True) -> None:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils import cpp_extension

    src_dir = os.path.join(reference_root, "lpmm", "cpp_extension")
    if not os.path.isdir(src_dir):
        raise FileNotFoundError(f"reference sources not found under {src_dir}")
    if only in (None, "python"):
        copy_python(reference_root)
    for name, files in MODULES.items():
        if only and name != only:
            continue
        out_dir = os.path.join(OUT, name)
        os.makedirs(out_dir, exist_ok=True)
        cpp_extension.load(
            name=name,
            sources=[os.path.join(src_dir, f) for f in files],
            extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a"],
            build_directory=out_dir,
            verbose=verbose,
            is_python_module=True,
        )


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--only", default=None, choices=list(MODULES) + ["python"])
    a = ap.parse_args()
    root = reference_root(a.reference)
    if root is None:
        sys.exit("no reference checkout found (give --reference or set LPMM_REFERENCE_ROOT)")
    build(root, a.only)
    print("built into", OUT)
    sys.exit(0)
