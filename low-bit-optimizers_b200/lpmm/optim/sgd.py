"""4-bit momentum SGD (reference: lpmm/optim/sgd.py).

The momentum buffer of tensors above the threshold is stored as 4-bit codes with the first-moment
config (``QUANT.M``: signed 'nonlinear' map, group-128 scales) in the layout of
``vectorwise_quant``; each tensor is updated by one fused launch that reproduces the reference's
sequence of torch operations (sgd.py:152-187).
"""
from typing import Optional

import torch

from .. import _kernels
from .optimizer import LowBitOptimizer

__all__ = ["SGD"]


class SGD(LowBitOptimizer):
    def __init__(self, params, lr, momentum=0, dampening=0, weight_decay=0, nesterov=False, qconfig=None, *,
                 maximize: bool = False, fused: Optional[bool] = False):
        if lr < 0.0:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if momentum < 0.0:
            raise ValueError("Invalid momentum value: {}".format(momentum))
        if weight_decay < 0.0:
            raise ValueError("Invalid weight_decay value: {}".format(weight_decay))
        if fused is True:
            raise ValueError("Not support fused SGD currently.")
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay, dampening=dampening, nesterov=nesterov,
                        maximize=maximize)
        super().__init__(params, defaults, qconfig)

    def get_subqconfig(self, optimizer_state_name):
        if optimizer_state_name == "momentum_buffer":
            return self.qconfig.QUANT.M
        raise ValueError(f"unknown optimizer state {optimizer_state_name!r}")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        md = self.get_qmetadata_by_state_name("momentum_buffer")
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("SGD does not support sparse gradients")
                state = self.state[p]
                if len(state) == 0:
                    state["momentum_buffer"] = torch.zeros((), dtype=torch.float, device=p.device)
                    self.init_qstate(p, "momentum_buffer")
                _kernels.sgd4bit_step(p, p.grad, state, self._q_enabled(p, "momentum_buffer"), md,
                                      weight_decay=group["weight_decay"], momentum=group["momentum"], lr=group["lr"],
                                      dampening=group["dampening"], nesterov=group["nesterov"],
                                      maximize=group["maximize"])
        return loss
