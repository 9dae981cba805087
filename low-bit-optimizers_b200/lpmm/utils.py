"""Rank helpers used by the config and optimizer code (reference: lpmm/utils.py:48-58)."""
import torch


def get_rank():
    return torch.distributed.get_rank() if torch.distributed.is_available() and torch.distributed.is_initialized() else 0


def get_world_size():
    return (torch.distributed.get_world_size()
            if torch.distributed.is_available() and torch.distributed.is_initialized() else 1)


def print0(*args, **kwargs):
    if get_rank() == 0:
        print(*args, **kwargs)
