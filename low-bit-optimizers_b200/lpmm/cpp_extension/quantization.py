"""``lpmm.cpp_extension.quantization`` (reference: lpmm/cpp_extension/quantization.cc:54-84).
The absmax-linear pair of the reference is exported there but never called by its Python code and
is not provided."""
from .._kernels import pack_nonlinear, unpack_nonlinear  # noqa: F401

__all__ = ["pack_nonlinear", "unpack_nonlinear"]
