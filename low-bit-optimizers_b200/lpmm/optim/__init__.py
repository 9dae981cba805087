from .adamw import AdamW  # noqa: F401
from .sgd import SGD  # noqa: F401

__all__ = ["AdamW", "SGD"]
