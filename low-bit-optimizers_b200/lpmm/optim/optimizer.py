"""Base class of the low-bit optimizers (reference: lpmm/optim/optimizer.py).

Holds the quantization config, the per-parameter quantization state (enable flag, per-step
metadata dict called ``overhead``, the quantization map) and a checkpoint format identical to the
reference's: torch's optimizer ``state_dict`` plus a top-level ``'qconfig'`` entry, with packed
int8 code tensors never cast to the parameter dtype on load.
"""
import copy
from collections import defaultdict
from collections.abc import Iterable
from itertools import chain

import torch

from ..config import get_config
from ..functional import create_general_qmap, init_lpmm_generator
from ..utils import get_rank


def quantize_enabled(p, config_enable, threshold):
    """A state of parameter ``p`` is quantized iff its config enables it and the tensor has more
    than ``threshold`` elements (reference optimizer.py:156-163; exactly ``threshold`` stays fp32)."""
    if not config_enable:
        return False
    return not (threshold is not None and p.numel() <= threshold)


class LowBitOptimizer(torch.optim.Optimizer):
    def __init__(self, params, defaults, config):
        super().__init__(params, defaults)
        # All ranks agree on one seed for stochastic rounding (reference optimizer.py:19-22).
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            dev = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
            seed = torch.randint(1 << 31, size=[], device=dev)
            torch.distributed.broadcast(seed, src=0)
            init_lpmm_generator(get_rank() if dev.type == "cuda" else "cpu", seed.item())
        self.qconfig = get_config(config)
        self.override_q_enable = {}
        self.qmaps = {}

    # ---- per-parameter quantization state ------------------------------------------------------
    def override_quantize_enable(self, module, param_name, enable):
        """Force (or forbid) quantization of one parameter's states; only before its first step."""
        p = getattr(module, param_name)
        assert p is not None
        assert isinstance(p, (torch.Tensor, torch.nn.Parameter))
        if len(self.state[p]) != 0:
            raise ValueError("overriding enabling of quantized parameters is prohibited after state initialization.")
        self.override_q_enable[id(p)] = enable

    def get_subqconfig(self, optimizer_state_name):
        raise NotImplementedError("The get_subconfig method needs overriding")

    def get_qmetadata_by_state_name(self, optimizer_state_name):
        sub = self.get_subqconfig(optimizer_state_name)
        return dict(b=sub.BITS, scale_type=sub.SCALE_TYPE.DEFAULT, quant_type=sub.QUANT_TYPE.DEFAULT,
                    round_type=sub.ROUND_TYPE, gp_sz=sub.GROUP_SIZE, signed=sub.SIGNED)

    def init_qstate(self, p, state_name):
        sub = self.get_subqconfig(state_name)
        md = self.get_qmetadata_by_state_name(state_name)
        key = (md["quant_type"], md["b"], md["signed"])
        if key not in self.qmaps:
            self.qmaps[key] = create_general_qmap(*key)
        self.qmaps[key] = self.qmaps[key].to(p.device)  # one shared tensor per map, on the params' device
        self.state[p][f"{state_name}_qstate"] = {
            "enable": quantize_enabled(p, sub.ENABLE, sub.THRESHOLD),
            "overhead": dict(),
            "qmap": self.qmaps[key],
        }

    def _q_enabled(self, p, state_name):
        if id(p) in self.override_q_enable:
            return self.override_q_enable[id(p)]
        return self.state[p][f"{state_name}_qstate"]["enable"]

    # ---- checkpointing ------------------------------------------------------------------------
    def state_dict(self):
        sd = super().state_dict()
        sd["qconfig"] = self.qconfig
        return sd

    def load_state_dict(self, state_dict):
        """Restore a checkpoint made by ``state_dict`` (of this class or of the reference's).
        Floating tensors follow the parameter's dtype and device, except ``step`` and the int8
        code tensors, which keep their dtype (reference optimizer.py:73-136)."""
        self.qconfig = state_dict["qconfig"]
        state_dict = copy.deepcopy(state_dict)
        groups, saved_groups = self.param_groups, state_dict["param_groups"]
        if len(groups) != len(saved_groups):
            raise ValueError("loaded state dict has a different number of parameter groups")
        if any(len(g["params"]) != len(s["params"]) for g, s in zip(groups, saved_groups)):
            raise ValueError("loaded state dict contains a parameter group that doesn't match the size of "
                             "optimizer's group")
        id_map = dict(zip(chain.from_iterable(g["params"] for g in saved_groups),
                          chain.from_iterable(g["params"] for g in groups)))

        def adopt(param, value, key=None):
            if isinstance(value, torch.Tensor):
                if key == "step":
                    return value
                # scales and moments next to 16-bit parameters (fused step for bf16 / fp16) stay fp32
                if (param.is_floating_point() and value.dtype != torch.int8 and value.is_floating_point()
                        and param.dtype not in (torch.bfloat16, torch.float16)):
                    value = value.to(param.dtype)
                return value.to(param.device)
            if isinstance(value, dict):
                return {k: adopt(param, v, key=k) for k, v in value.items()}
            if isinstance(value, torch.Size) or isinstance(value, (str, bytes)):
                return value
            if isinstance(value, Iterable):
                return type(value)(adopt(param, v) for v in value)
            return value

        state = defaultdict(dict)
        for k, v in state_dict["state"].items():
            if k in id_map:
                state[id_map[k]] = adopt(id_map[k], v)
            else:
                state[k] = v
        new_groups = []
        for g, s in zip(groups, saved_groups):
            s["params"] = g["params"]
            new_groups.append(s)
        self.__setstate__({"state": state, "param_groups": new_groups})
        # maps are shared per (type, bits, signed): re-share them after the copy
        self.qmaps = {}

    @torch.no_grad()
    def step(self, closure=None):
        raise NotImplementedError("The step method needs overriding")
