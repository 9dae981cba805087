"""Compile the reference's own CUDA extension, in place, for sm_100a.

TEST INFRASTRUCTURE ONLY.  Nothing in the product imports this file or its output.

The two pybind11 modules of the reference (``lpmm/cpp_extension/fused_adamw*.{cc,cu}`` and
``lpmm/cpp_extension/quantization*.{cc,cu}``, built upstream by ``setup.py:21-30``) are compiled
from the sources where they lie in the read-only reference checkout.  Only the resulting shared
objects are written, into ``oracle/_ref/`` (git-ignored).  No reference source is copied.

The GPU parity tests load these modules, when present, as the authoritative result of the
reference kernels on the same inputs.  The flags mirror what the reference's ``setup.py`` gives
``CUDAExtension`` (no optimisation or fast-math flags of its own: nvcc defaults, i.e.
``-fmad=true``, IEEE division and square root), plus the sm_100a ``-gencode``.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--only fused_adamw|quantization]
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

MODULES = {
    "fused_adamw": ["fused_adamw.cc", "fused_adamw_kernel.cu"],
    "quantization": ["quantization.cc", "quantization_kernel.cu"],
}


def build(reference_root: str, only=None, verbose=True) -> None:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils import cpp_extension

    src_dir = os.path.join(reference_root, "lpmm", "cpp_extension")
    if not os.path.isdir(src_dir):
        raise FileNotFoundError(f"reference sources not found under {src_dir}")
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
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--only", default=None, choices=list(MODULES))
    a = ap.parse_args()
    build(a.reference, a.only)
    print("built into", OUT)
    sys.exit(0)
