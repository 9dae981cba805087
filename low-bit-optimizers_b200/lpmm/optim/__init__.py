from .adamw import AdamW  # noqa: F401
from .sgd import SGD  # noqa: F401
from ..zero import ZeroAdamW  # noqa: F401  (ZeRO-1 sharded form of AdamW(fused=True); no counterpart in the reference)

__all__ = ["AdamW", "SGD", "ZeroAdamW"]
