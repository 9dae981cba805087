"""4-bit momentum SGD (reference: lpmm/optim/sgd.py).

The momentum buffer of tensors above the threshold is stored as 4-bit codes with the first-moment
config (``QUANT.M``: signed 'nonlinear' map, group-128 scales) in the layout of
``vectorwise_quant``; each tensor is updated by one launch that reproduces the reference's sequence
of torch operations (sgd.py:152-187).

Once the buffers exist, every parameter group is stepped by one multi-tensor launch with the same
arithmetic and the same state layout as the per-tensor launch (results and ``state_dict`` are
identical bit for bit); a tensor's first step, which creates its buffer, and configurations the
multi-tensor kernel does not cover (wider codes, larger groups, no momentum) use the per-tensor
launch.  ``fused=True``, which the reference rejects (sgd.py:31-32), is accepted and means the same;
``fused=False`` with ``LPMM_SGD_PER_TENSOR=1`` in the environment forces the per-tensor launches.
"""
import os
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
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay, dampening=dampening, nesterov=nesterov,
                        maximize=maximize)
        super().__init__(params, defaults, qconfig)
        # not a param_group entry: the state_dict stays the reference's
        self._fused = bool(fused) or os.environ.get("LPMM_SGD_PER_TENSOR", "0") != "1"
        self._lists = {}  # (group index, device) -> (pointer key, TensorList) of the multi-tensor launch

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
        multi_ok = (md["b"] == 4 and md["gp_sz"] == 128 and md["scale_type"] == "group"
                    and md["round_type"] == "real-nearest")
        if md["round_type"] == "real-sr":
            return self._step_stochastic(md, loss)
        for gi, group in enumerate(self.param_groups):
            fused = self._fused and group["momentum"] != 0 and multi_ok
            batch = {}  # device -> entries of the multi-tensor launch
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("SGD does not support sparse gradients")
                state = self.state[p]
                if len(state) == 0:
                    state["momentum_buffer"] = torch.zeros((), dtype=torch.float, device=p.device)
                    self.init_qstate(p, "momentum_buffer")
                buf = state["momentum_buffer"]
                if fused and buf.numel() > 1 and p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() \
                        and p.grad.dtype == torch.float32 and p.grad.is_contiguous():
                    quant = self._q_enabled(p, "momentum_buffer")
                    max1 = state["momentum_buffer_qstate"]["overhead"].get("max1") if quant else None
                    if (quant and buf.dtype == torch.int8 and max1 is not None) or (not quant and buf.dtype == torch.float32):
                        batch.setdefault(p.device, []).append((p, p.grad, buf, buf, max1, None))
                        continue
                _kernels.sgd4bit_step(p, p.grad, state, self._q_enabled(p, "momentum_buffer"), md,
                                      weight_decay=group["weight_decay"], momentum=group["momentum"], lr=group["lr"],
                                      dampening=group["dampening"], nesterov=group["nesterov"],
                                      maximize=group["maximize"])
            for device, entries in batch.items():
                key = tuple((e[0].data_ptr(), e[1].data_ptr(), e[2].data_ptr()) for e in entries)
                cached = self._lists.get((gi, device))
                if cached is None or cached[0] != key:
                    cached = (key, _kernels.TensorList(entries))
                    self._lists[(gi, device)] = cached
                qmap = self.state[entries[0][0]]["momentum_buffer_qstate"]["qmap"]
                with torch.cuda.device(device):
                    _kernels.sgd4bit_multi_tensor(cached[1], qmap, weight_decay=group["weight_decay"],
                                                  momentum=group["momentum"], lr=group["lr"],
                                                  dampening=group["dampening"], nesterov=group["nesterov"],
                                                  maximize=group["maximize"])
        return loss

    def _step_stochastic(self, md, loss):
        """'real-sr' momentum buffers: dequantise, fp32 step, quantise with the reference's random stream
        (sgd.py:152-187), parameter by parameter."""
        from ..functional import vectorwise_dequant, vectorwise_quant
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
                quant = self._q_enabled(p, "momentum_buffer")
                buf, first = None, False
                if group["momentum"] != 0:
                    t, qs = state["momentum_buffer"], state["momentum_buffer_qstate"]
                    first = t.numel() <= 1
                    if first:
                        buf = torch.empty_like(p, memory_format=torch.preserve_format)
                    elif quant:
                        buf = vectorwise_dequant(t, qmap=qs["qmap"], shape=p.shape, **md, **qs["overhead"]).contiguous()
                    else:
                        buf = t
                _kernels.sgd_fp32_buffer_step(p, p.grad, buf, first, weight_decay=group["weight_decay"],
                                              momentum=group["momentum"], lr=group["lr"], dampening=group["dampening"],
                                              nesterov=group["nesterov"], maximize=group["maximize"])
                if group["momentum"] != 0:
                    qs = state["momentum_buffer_qstate"]
                    if quant:
                        qx, gen = vectorwise_quant(buf, qmap=qs["qmap"], shape=p.shape, mimic_rng=True, **md)
                        state["momentum_buffer"] = qx
                        qs["overhead"].update(gen)
                    else:
                        state["momentum_buffer"] = buf
        return loss
