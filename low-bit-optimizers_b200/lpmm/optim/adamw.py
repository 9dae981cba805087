"""4-bit AdamW (reference: lpmm/optim/adamw.py).

Constructor, lazily created state, state names and layouts are those of the reference:

* ``fused=True``  -- ``exp_avg`` / ``exp_avg_sq`` are ``int8[(numel + 1) // 2]`` packed codes with
  ``float32[(numel + 127) // 128]`` scales in ``state['exp_avg_qstate']['overhead']['max1']``
  (adamw.py:508-523).  The whole parameter list of a group is updated by ONE multi-tensor launch
  instead of the reference's per-tensor loop (adamw.py:463-561).
* ``fused=False`` -- codes in the padded 2048-row layout of ``vectorwise_quant`` with the
  generated metadata (``max1`` or ``max_dims``, ``dim``, ``scaled_shape``, ``dtype``, ``stride``)
  in ``overhead`` (adamw.py:425-434); each tensor is updated by one fused launch that reproduces
  the reference's sequence of torch operations (adamw.py:369-422).
* ``fused=True, fused_rank1=True`` (an extension; the reference's fused step cannot hold rank-1 scales and
  falls back to group scales with a warning, adamw.py:503-506) -- with a rank-1 second-moment
  configuration the states have the ``fused=False`` layout (per-axis maxima in ``max_dims``) and are
  stepped with the fused kernel's arithmetic (``lpmm_b200_adamw4bit_fused_arith_step_many``).
* ``exact_params=False`` (an extension) -- the tolerance mode: moments, scales and packed codes stay
  bit-identical to the reference's, the parameters follow it to within 1e-6 relative (approximate square root
  and reciprocal in the parameter update only), for fewer instructions.  It applies to the fused step and to the
  list-wide kernels of the non-fused step (plain, rank-1 and factored tensors stepped together).
* tensors with at most ``THRESHOLD`` (4096) elements, or overridden, keep fp32 moments.
* ``factor_second_moment=True`` keeps fp32 row/column accumulators for every >=2-D tensor
  (adamw.py:124-126, 579-627).
"""
from typing import Optional

import torch

from .. import _kernels
from .optimizer import LowBitOptimizer

__all__ = ["AdamW"]


class AdamW(LowBitOptimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, use_first_moment=True,
                 factor_second_moment=False, qconfig=None, *, fused: Optional[bool] = False, fused_rank1: bool = False,
                 exact_params: bool = True):
        if not 0.0 <= lr:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if not 0.0 <= eps:
            raise ValueError("Invalid epsilon value: {}".format(eps))
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError("Invalid beta parameter at index 0: {}".format(betas[0]))
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError("Invalid beta parameter at index 1: {}".format(betas[1]))
        if not 0.0 <= weight_decay:
            raise ValueError("Invalid weight_decay value: {}".format(weight_decay))
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=fused,
                        use_first_moment=use_first_moment, factor_second_moment=factor_second_moment)
        super().__init__(params, defaults, qconfig)
        self._fused_rank1 = bool(fused_rank1)
        self._exact_params = bool(exact_params)
        self._lists = {}  # cached descriptor arrays of the multi-tensor step, per param group
        self._spare = {}  # per-parameter buffers that are not optimizer state (alternate rank-1 maxima)
        self._plans = {}  # fused groups: everything needed to repeat the last launch
        self._batches = {}  # non-fused groups: the descriptors of all tensors, stepped by one library call

    def __setstate__(self, state):
        super().__setstate__(state)
        self.__dict__.setdefault("_fused_rank1", False)
        self.__dict__.setdefault("_exact_params", True)
        self._lists = {}
        self._spare = {}
        self._plans = {}
        self._batches = {}
        for group in self.param_groups:
            group.setdefault("fused", None)
        values = list(self.state.values())
        if values and not torch.is_tensor(values[0]["step"]):
            for s in values:
                s["step"] = torch.tensor(float(s["step"]))

    def get_subqconfig(self, optimizer_state_name):
        if optimizer_state_name == "exp_avg":
            return self.qconfig.QUANT.M
        if optimizer_state_name == "exp_avg_sq":
            return self.qconfig.QUANT.SQM
        raise ValueError(f"unknown optimizer state {optimizer_state_name!r}")

    @staticmethod
    def _get_options(param_group, param_shape):
        return len(param_shape) >= 2 and param_group["factor_second_moment"], param_group["use_first_moment"]

    def _init_state(self, group, p):
        """Lazy state of one parameter (reference adamw.py:116-129): a CPU step counter, 0-dim
        placeholders for the moments (their first use allocates the real storage) and the qstates."""
        state = self.state[p]
        factored, _ = self._get_options(group, p.shape)
        state["step"] = torch.tensor(0.0)
        state["exp_avg"] = torch.zeros((), dtype=torch.float, device=p.device)
        self.init_qstate(p, "exp_avg")
        if factored:
            state["exp_avg_sq_row"] = torch.zeros(p.shape[:-1], device=p.device)
            state["exp_avg_sq_col"] = torch.zeros(p.shape[:-2] + p.shape[-1:], device=p.device)
        else:
            state["exp_avg_sq"] = torch.zeros((), dtype=torch.float, device=p.device)
        self.init_qstate(p, "exp_avg_sq")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            self._step_group(gi, group)
        return loss

    def _params_to_step(self, group):
        params = []
        for p in group["params"]:
            if p.grad is None:
                continue
            if p.grad.is_sparse:
                raise RuntimeError("AdamW does not support sparse gradients")
            if len(self.state[p]) == 0:
                self._init_state(group, p)
            params.append(p)
        return params

    def _step_group(self, gi, group):
        params = self._params_to_step(group)
        if not params:
            return
        if group["fused"] and self._fused_rank1_applies(group):
            self._step_single(gi, group, params, fused_arith=True)
        elif group["fused"]:
            self._step_fused(gi, group, params)
        else:
            self._step_single(gi, group, params)

    @torch.no_grad()
    def step_from_host(self, host_grads, chunk_bytes=256 << 20):
        """One step whose gradients arrive from host memory (an extension; the reference has no such call).

        ``host_grads``: one CPU tensor (pinned, for the copies to be asynchronous) per parameter of the optimizer, in
        the order of ``param_groups``; ``None`` leaves that parameter out of the step.  Each is copied into the
        parameter's ``.grad`` (allocated here if missing) on a copy stream.  A ``fused=True`` group that has been stepped
        before is updated while the copies are still running: every ``chunk_bytes`` of gradients that have landed are
        followed by a launch over just those tensors' groups (``group_begin`` / ``group_end`` of the list step), so the
        step ends one chunk's update after the last byte arrives instead of a whole list's.  Other groups wait for
        their copies and take the ordinary step.  Results are those of copying everything and calling ``step()``."""
        all_params = [p for group in self.param_groups for p in group["params"]]
        host = list(host_grads)
        if len(host) != len(all_params):
            raise ValueError(f"expected {len(all_params)} host gradients (None for a parameter to skip), got {len(host)}")
        k = 0
        for gi, group in enumerate(self.param_groups):
            pairs = []
            for p in group["params"]:
                h = host[k]
                k += 1
                if h is None:
                    p.grad = None
                    continue
                if h.numel() != p.numel() or h.dtype != p.dtype:
                    raise RuntimeError("a host gradient must have its parameter's size and dtype")
                if p.grad is None:
                    p.grad = torch.empty_like(p, memory_format=torch.contiguous_format)
                pairs.append((p, h))
            if not pairs:
                continue
            if not pairs[0][0].is_cuda:  # nothing to overlap
                for p, h in pairs:
                    p.grad.copy_(h.view_as(p.grad))
                self._step_group(gi, group)
                continue
            device = pairs[0][0].device
            main = torch.cuda.current_stream(device)
            copies = self.__dict__.setdefault("_copy_streams", {})
            cs = copies.get(device)
            if cs is None:
                cs = copies[device] = torch.cuda.Stream(device=device)
            cs.wait_stream(main)  # work already enqueued may still read the gradient buffers
            params = self._params_to_step(group)
            plan = None
            if group["fused"] and not self._fused_rank1_applies(group):
                plan = self._plan_ready(gi, params)
            if plan is None:
                with torch.cuda.stream(cs):
                    for p, h in pairs:
                        p.grad.copy_(h.view_as(p.grad), non_blocking=True)
                main.wait_stream(cs)
                self._step_group(gi, group)
                continue
            if "gstart" not in plan:  # first group of every tensor in the list-wide group numbering
                gs, acc = [], 0
                for p in plan["params"]:
                    gs.append(acc)
                    acc += (p.numel() + 127) // 128
                plan["gstart"] = gs + [acc]
            torch._foreach_add_(plan["steps"], 1.0)
            plan["step"] += 1.0
            gstart, done, pending = plan["gstart"], 0, 0
            for i, (p, h) in enumerate(pairs):  # pairs and plan["params"] are the same parameters in the same order
                with torch.cuda.stream(cs):
                    p.grad.copy_(h.view_as(p.grad), non_blocking=True)
                pending += p.numel() * p.element_size()
                if pending >= chunk_bytes or i + 1 == len(pairs):
                    ev = torch.cuda.Event()
                    ev.record(cs)
                    main.wait_event(ev)
                    self._plan_launch(group, plan, gstart[done], gstart[i + 1])
                    done, pending = i + 1, 0

    def _fused_rank1_applies(self, group):
        """fused_rank1=True and a configuration the fused kernel cannot hold as such: a rank-1 second moment
        (4-bit codes, nearest rounding, no factored second moment)."""
        if not self._fused_rank1 or group["factor_second_moment"]:
            return False
        md_m = self.get_qmetadata_by_state_name("exp_avg")
        md_v = self.get_qmetadata_by_state_name("exp_avg_sq")
        if md_v["scale_type"] != "rank1" or md_m["scale_type"] != "group":
            return False
        if md_m["b"] != 4 or md_v["b"] != 4:
            raise NotImplementedError("the fused step stores 4-bit codes; use fused=False for "
                                      f"{md_m['b']}/{md_v['b']}-bit states")
        if md_m["round_type"] == "real-sr" or md_v["round_type"] == "real-sr":
            raise NotImplementedError("the fused step rounds to nearest; use fused=False for stochastic rounding")
        return True

    # ---- fused=True ---------------------------------------------------------------------------
    def _step_fused(self, gi, group, params):
        if self._step_fused_planned(gi, group, params):
            return
        beta1, beta2 = group["betas"]
        md_m = self.get_qmetadata_by_state_name("exp_avg")
        md_v = self.get_qmetadata_by_state_name("exp_avg_sq")
        by_step = {}
        warned = False
        for p in params:
            state = self.state[p]
            factored, _ = self._get_options(group, p.shape)
            state["step"] += 1
            if factored:  # the fused kernel does not cover factored tensors (reference adamw.py:472-495)
                self._factored_update(group, p, state)
                continue
            en_m, en_v = self._q_enabled(p, "exp_avg"), self._q_enabled(p, "exp_avg_sq")
            if en_m != en_v:
                raise ValueError("For same tensor, exp_avg and exp_avg_sq should be both quantized or unquantized "
                                 f"simultaneously, but get ({en_m} {en_v})")
            if en_m:
                if md_m["b"] != 4 or md_v["b"] != 4:
                    # the reference's fused kernel reads the first 16 entries of a wider map as a 4-bit map
                    # (fused_adamw_kernel.cu:27-60); that is not reproduced
                    raise NotImplementedError("the fused step stores 4-bit codes; use fused=False for "
                                              f"{md_m['b']}/{md_v['b']}-bit states")
                if not warned and (md_m["scale_type"] != "group" or md_v["scale_type"] != "group"):
                    print("Warning: fused_adamw4bit only support block-wise scaling, but get scale types "
                          f"({md_m['scale_type']}, {md_v['scale_type']}).")
                    warned = True
                n = p.numel()
                if state["exp_avg"].numel() <= 1:
                    state["exp_avg"].data = torch.zeros(((n + 1) // 2,), dtype=torch.int8, device=p.device)
                if state["exp_avg_sq"].numel() <= 1:
                    state["exp_avg_sq"].data = torch.zeros(((n + 1) // 2,), dtype=torch.int8, device=p.device)
                oh_m, oh_v = state["exp_avg_qstate"]["overhead"], state["exp_avg_sq_qstate"]["overhead"]
                if "max1" not in oh_m:
                    oh_m["max1"] = torch.zeros(((n + 127) // 128,), dtype=torch.float32, device=p.device)
                if "max1" not in oh_v:
                    oh_v["max1"] = torch.zeros(((n + 127) // 128,), dtype=torch.float32, device=p.device)
                entry = (p, p.grad, state["exp_avg"], state["exp_avg_sq"], oh_m["max1"], oh_v["max1"])
            else:
                if state["exp_avg"].numel() <= 1:  # fp32 moments also next to 16-bit parameters
                    state["exp_avg"].data = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
                if state["exp_avg_sq"].numel() <= 1:
                    state["exp_avg_sq"].data = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
                entry = (p, p.grad, state["exp_avg"], state["exp_avg_sq"], None, None)
            for t, nm in zip(entry[:4], ("p", "g", "exp_avg", "exp_avg_sq")):
                if not t.is_contiguous():
                    raise RuntimeError(f"{nm} must be contiguous!")
                if not t.is_cuda:
                    raise RuntimeError(f"{nm} must be a CUDA tensor!")
            if p.dtype not in (torch.float32, torch.bfloat16, torch.float16) or p.grad.dtype != p.dtype:
                raise RuntimeError("The type of p / g is not kFloat32 (or both kBFloat16 / kHalf)!")
            if entry[2].dtype not in (torch.int8, torch.float32) or entry[3].dtype != entry[2].dtype:
                raise RuntimeError("exp_avg / exp_avg_sq must be packed int8 codes or float32!")
            key = (float(state["step"].item()), p.device, p.dtype)
            by_step.setdefault(key, []).append((entry, state))
        for (step, device, dtype), items in by_step.items():
            entries = [e for e, _ in items]
            qm = items[0][1]["exp_avg_qstate"]["qmap"]
            qv = items[0][1]["exp_avg_sq_qstate"]["qmap"]
            tl = self._tensor_list((gi, (step, dtype) if len(by_step) > 1 else None, device), entries)
            with torch.cuda.device(device):
                _kernels.adamw4bit_multi_tensor(tl, qm, qv, beta1, beta2, group["lr"], group["weight_decay"],
                                                group["eps"], step, dtype=dtype, exact_params=self._exact_params)
            if len(by_step) == 1 and len(items) == len(params):
                # every tensor of the group took this one launch: remember it, so that the following steps
                # only bump the counters, refresh changed gradient pointers and launch
                self._plans[gi] = dict(
                    params=list(params), tl=tl, step=step, device=device, qm=qm, qv=qv, dtype=dtype,
                    states=[st for _, st in items], steps=[st["step"] for _, st in items],
                    m=[e[2] for e in entries], v=[e[3] for e in entries],
                    ptrs=[(e[0].data_ptr(), e[2].data_ptr(), e[3].data_ptr()) for e in entries],
                    gptrs=[e[1].data_ptr() for e in entries])

    def _step_fused_planned(self, gi, group, params):
        """Fast path of a fused group whose tensors, states and step counters are unchanged since the
        last step.  Returns False (after dropping the plan) whenever anything differs."""
        plan = self._plan_ready(gi, params)
        if plan is None:
            return False
        torch._foreach_add_(plan["steps"], 1.0)
        plan["step"] += 1.0
        self._plan_launch(group, plan)
        return True

    def _plan_ready(self, gi, params):
        """The plan of group ``gi`` if it still describes ``params`` (gradient pointers refreshed), else None (the
        plan is dropped)."""
        plan = self._plans.get(gi)
        if plan is None:
            return None
        pp = plan["params"]
        if len(pp) != len(params):
            del self._plans[gi]
            return None
        tl, gptrs = plan["tl"], plan["gptrs"]
        for i, p in enumerate(params):
            st = plan["states"][i]
            m, v = plan["m"][i], plan["v"][i]
            if (p is not pp[i] or st.get("exp_avg") is not m or st.get("exp_avg_sq") is not v
                    or st.get("step") is not plan["steps"][i]
                    or (p.data_ptr(), m.data_ptr(), v.data_ptr()) != plan["ptrs"][i]):
                del self._plans[gi]
                return None
            g = p.grad
            gp = g.data_ptr()
            if gp != gptrs[i]:
                if g.dtype != plan["dtype"] or not g.is_cuda or not g.is_contiguous() or g.numel() != p.numel():
                    del self._plans[gi]
                    return None
                tl.array[i].g = gp
                gptrs[i] = gp
        return plan

    def _plan_launch(self, group, plan, group_begin=0, group_end=-1):
        beta1, beta2 = group["betas"]
        with torch.cuda.device(plan["device"]):
            _kernels.adamw4bit_multi_tensor(plan["tl"], plan["qm"], plan["qv"], beta1, beta2, group["lr"],
                                            group["weight_decay"], group["eps"], plan["step"], group_begin, group_end,
                                            dtype=plan["dtype"], exact_params=self._exact_params)

    def _tensor_list(self, key, entries):
        """Descriptor array of a parameter list, rebuilt only when a pointer changed."""
        sig = tuple(t.data_ptr() if t is not None else 0 for e in entries for t in e)
        cached = self._lists.get(key)
        if cached is None or cached[0] != sig:
            cached = (sig, _kernels.TensorList(entries))
            self._lists[key] = cached
        return cached[1]

    # ---- fused=False --------------------------------------------------------------------------
    def _step_single(self, gi, group, params, fused_arith=False):
        md_m = self.get_qmetadata_by_state_name("exp_avg")
        md_v = self.get_qmetadata_by_state_name("exp_avg_sq")
        if md_m["round_type"] == "real-sr" or md_v["round_type"] == "real-sr":
            return self._step_single_stochastic(group, params, md_m, md_v)
        if self._step_single_batched(gi, group, params, fused_arith):
            return
        self._step_single_each(group, params, fused_arith)
        self._prepare_batch(gi, params)

    def _step_single_stochastic(self, group, params, md_m, md_v):
        """Configurations with stochastic rounding ('real-sr'): the reference's own sequence per parameter
        (adamw.py:332-436, 579-627) -- dequantise, one fp32 step, quantise -- so that every quantisation
        call takes its random stream from torch's CUDA generator in the reference's order (first moment,
        then second moment, parameter by parameter; nearest-rounded states advance the generator too)."""
        for p in params:
            state = self.state[p]
            state["step"] += 1
            self._stochastic_update(group, p, state, md_m, md_v)

    def _stochastic_update(self, group, p, state, md_m, md_v):
        from ..functional import vectorwise_dequant, vectorwise_quant
        beta1, beta2 = group["betas"]
        factored, _ = self._get_options(group, p.shape)
        moments = {}
        for name, md in (("exp_avg", md_m), ("exp_avg_sq", md_v)):
            if name == "exp_avg_sq" and factored:
                continue
            t, qs = state[name], state[f"{name}_qstate"]
            if t.numel() <= 1:
                moments[name] = torch.zeros_like(p, memory_format=torch.preserve_format)
            elif self._q_enabled(p, name):
                moments[name] = vectorwise_dequant(t, qmap=qs["qmap"], shape=p.shape, **md, **qs["overhead"]).contiguous()
            else:
                moments[name] = t
        _kernels.adamw_fp32_moments_step(
            p, p.grad, moments["exp_avg"], moments.get("exp_avg_sq"), state.get("exp_avg_sq_row"),
            state.get("exp_avg_sq_col"), beta1=beta1, beta2=beta2, lr=group["lr"],
            weight_decay=group["weight_decay"], eps=group["eps"], step=state["step"].item())
        for name, md in (("exp_avg", md_m), ("exp_avg_sq", md_v)):
            if name not in moments:
                continue
            qs = state[f"{name}_qstate"]
            if self._q_enabled(p, name):
                qx, gen = vectorwise_quant(moments[name], qmap=qs["qmap"], shape=p.shape, mimic_rng=True, **md)
                state[name] = qx
                qs["overhead"].update(gen)
            else:
                state[name] = moments[name]

    def _prepare_batch(self, gi, params):
        """After a per-tensor step: if every tensor now has a cached descriptor, on the current device and
        with the same two maps, keep them as one array for ``lpmm_b200_adamw4bit_unfused_step_many``."""
        import ctypes
        if not torch.cuda.is_available():
            return
        cur = torch.cuda.current_device()
        spares, plans, states, maps = [], [], [], set()
        for p in params:
            sp = self._spare.get(id(p))
            plan = sp.get("plan") if sp else None
            st = self.state[p]
            if plan is None or not p.is_cuda or p.device.index != cur or not plan.matches(p, st):
                return
            maps.add((st["exp_avg_qstate"]["qmap"].data_ptr(), st["exp_avg_sq_qstate"]["qmap"].data_ptr()))
            spares.append(sp)
            plans.append(plan)
            states.append(st)
        if len(maps) != 1:
            return
        n = len(params)
        ptrs = (ctypes.c_void_p * n)()
        addrs = []
        for i, plan in enumerate(plans):
            a = tuple(ctypes.addressof(d) for d in plan.descs)
            addrs.append(a)
            ptrs[i] = a[plan.which if len(a) > 1 else 0]
        self._batches[gi] = dict(params=list(params), plans=plans, states=states, spares=spares, ptrs=ptrs, addrs=addrs,
                                 steps=(ctypes.c_double * n)(), device=cur, qm=states[0]["exp_avg_qstate"]["qmap"],
                                 qv=states[0]["exp_avg_sq_qstate"]["qmap"],
                                 rank1_index=[i for i, pl in enumerate(plans) if pl.axis_sets is not None],
                                 scratch=_kernels.unfused_step_many_scratch_bytes(ptrs, n))

    def _step_single_batched(self, gi, group, params, fused_arith=False):
        """All tensors of a non-fused group through one library call.  Returns False (after dropping the
        cached batch) whenever a tensor, a state or a storage is not the one the batch was built for."""
        b = self._batches.get(gi)
        if b is None:
            return False
        plans, states = b["plans"], b["states"]
        ok = len(params) == len(plans) and torch.cuda.current_device() == b["device"]
        if ok:
            bp = b["params"]
            for i, p in enumerate(params):
                if p is not bp[i] or not plans[i].matches(p, states[i]) or not plans[i].set_grad(p.grad):
                    ok = False
                    break
        if not ok:
            del self._batches[gi]
            return False
        steps, ptrs, addrs = b["steps"], b["ptrs"], b["addrs"]
        step_tensors = b.get("step_tensors")
        if step_tensors is None or any(st["step"] is not t for st, t in zip(states, step_tensors)):
            step_tensors = b["step_tensors"] = [st["step"] for st in states]
        torch._foreach_add_(step_tensors, 1.0)  # one call instead of one CPU tensor op per parameter
        steps[:] = torch.stack(step_tensors).tolist()
        beta1, beta2 = group["betas"]
        _kernels.adamw4bit_unfused_step_many(ptrs, len(plans), b["qm"], b["qv"], steps, b["scratch"], params[0].device,
                                             beta1=beta1, beta2=beta2, lr=group["lr"],
                                             weight_decay=group["weight_decay"], eps=group["eps"], fused_arith=fused_arith,
                                             exact_params=self._exact_params)
        for i in b["rank1_index"]:  # rank-1: the freshly written maxima become the state's
            plan = plans[i]
            plan.which ^= 1
            plan.oh_v["max_dims"] = plan.axis_sets[plan.which]
            b["spares"][i]["max_dims"] = plan.axis_sets[plan.which ^ 1]
            ptrs[i] = addrs[i][plan.which]
        return True

    def _step_single_each(self, group, params, fused_arith=False):
        beta1, beta2 = group["betas"]
        md_m = self.get_qmetadata_by_state_name("exp_avg")
        md_v = self.get_qmetadata_by_state_name("exp_avg_sq")
        # torch's current device and stream, looked up once for all tensors that live on that device
        cur = torch.cuda.current_device() if torch.cuda.is_available() else -1
        handle = torch.cuda.current_stream().cuda_stream if cur >= 0 else None
        lr, wd, eps = group["lr"], group["weight_decay"], group["eps"]
        for p in params:
            state = self.state[p]
            factored, _ = self._get_options(group, p.shape)
            state["step"] += 1
            if factored:
                self._factored_update(group, p, state)
                continue
            _kernels.adamw4bit_unfused_step(
                p, p.grad, state, self._q_enabled(p, "exp_avg"), self._q_enabled(p, "exp_avg_sq"), md_m, md_v,
                self._spare.setdefault(id(p), {}),
                beta1=beta1, beta2=beta2, lr=lr, weight_decay=wd, eps=eps, step=state["step"].item(),
                stream=handle if (p.is_cuda and p.device.index == cur) else None, fused_arith=fused_arith)

    def _factored_update(self, group, p, state):
        md_m = self.get_qmetadata_by_state_name("exp_avg")
        if md_m["round_type"] == "real-sr":
            return self._stochastic_update(group, p, state, md_m, self.get_qmetadata_by_state_name("exp_avg_sq"))
        beta1, beta2 = group["betas"]
        _kernels.adamw4bit_factored_step(
            p, p.grad, state, self._q_enabled(p, "exp_avg"), self.get_qmetadata_by_state_name("exp_avg"),
            beta1=beta1, beta2=beta2, lr=group["lr"], weight_decay=group["weight_decay"], eps=group["eps"],
            step=state["step"].item(), spare=self._spare.setdefault(id(p), {}))
