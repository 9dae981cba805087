"""``lpmm.cpp_extension.fused_adamw`` (reference: lpmm/cpp_extension/fused_adamw.cc:15-84)."""
from .._kernels import adamw4bit_single_tensor, adamw_single_tensor  # noqa: F401

__all__ = ["adamw_single_tensor", "adamw4bit_single_tensor"]
