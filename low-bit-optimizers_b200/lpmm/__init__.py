"""lpmm -- 4-bit optimizers whose step runs in hand-written sm_100a CUDA.

Same import surface as the reference package (``lpmm/__init__.py:1`` imports ``optim``):
``lpmm.optim.AdamW``, ``lpmm.optim.SGD``, ``lpmm.functional``, ``lpmm.config``.
"""
from . import optim  # noqa: F401

__all__ = ["optim"]
