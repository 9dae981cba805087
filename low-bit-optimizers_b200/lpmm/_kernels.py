"""Tensor-level wrappers of the C-ABI entry points: argument checks in the style of the
reference's bindings (CUDA, contiguous, dtype; ``lpmm/cpp_extension/common.h:1-28``), pointer
extraction, launch on torch's current stream of the tensors' device."""
import ctypes

import torch

from . import _native as N

_vp = ctypes.c_void_p


def _ptr(t):
    return _vp(t.data_ptr()) if t is not None else _vp(None)


def _stream():
    return _vp(torch.cuda.current_stream().cuda_stream)


def _check_cuda_float(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor!")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous!")
    if t.dtype != torch.float32:
        raise RuntimeError(f"The type of {name} is not kFloat32!")


def _check_cuda_int8(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor!")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous!")
    if t.dtype != torch.int8:
        raise RuntimeError(f"The type of {name} is not correct!")


# ----------------------------------------------------------------------------------------------
# fused AdamW
# ----------------------------------------------------------------------------------------------
def adamw4bit_single_tensor(p, g, exp_avg, exp_avg_sq, exp_avg_scale, exp_avg_sq_scale, exp_avg_qmap, exp_avg_sq_qmap,
                            beta1, beta2, lr, weight_decay, eps, step):
    for t, n in ((p, "p"), (g, "g"), (exp_avg_scale, "exp_avg_scale"), (exp_avg_sq_scale, "exp_avg_sq_scale"),
                 (exp_avg_qmap, "exp_avg_qmap"), (exp_avg_sq_qmap, "exp_avg_sq_qmap")):
        _check_cuda_float(t, n)
    _check_cuda_int8(exp_avg, "exp_avg")
    _check_cuda_int8(exp_avg_sq, "exp_avg_sq")
    n = p.numel()
    nbytes, ngroups = (n + 1) // 2, (n + 127) // 128
    if exp_avg.numel() != nbytes or exp_avg_sq.numel() != nbytes:
        raise RuntimeError("number of elements in exp_avg / exp_avg_sq must be (p.numel() + 1) // 2")
    if g.numel() != n:
        raise RuntimeError("number of elements in g and p tensors should be equal")
    if exp_avg_scale.numel() != ngroups or exp_avg_sq_scale.numel() != ngroups:
        raise RuntimeError("one scale per 128 elements expected")
    if exp_avg_qmap.numel() != 16 or exp_avg_sq_qmap.numel() != 16:
        raise RuntimeError("4-bit quantization maps must have 16 entries")
    with torch.cuda.device(p.device):
        N.check(N.lib.lpmm_b200_adamw4bit_single_tensor(
            _ptr(p), _ptr(g), _ptr(exp_avg), _ptr(exp_avg_sq), _ptr(exp_avg_scale), _ptr(exp_avg_sq_scale),
            _ptr(exp_avg_qmap), _ptr(exp_avg_sq_qmap), beta1, beta2, lr, weight_decay, eps, step, n, _stream()))


def adamw_single_tensor(p, g, exp_avg, exp_avg_sq, beta1, beta2, lr, weight_decay, eps, step):
    for t, n in ((p, "p"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq"), (g, "g")):
        _check_cuda_float(t, n)
    n = p.numel()
    if exp_avg.numel() != n:
        raise RuntimeError("number of elements in exp_avg and p tensors should be equal")
    if exp_avg_sq.numel() != n:
        raise RuntimeError("number of elements in exp_avg_sq and p tensors should be equal")
    if g.numel() != n:
        raise RuntimeError("number of elements in g and p tensors should be equal")
    with torch.cuda.device(p.device):
        N.check(N.lib.lpmm_b200_adamw_single_tensor(_ptr(p), _ptr(g), _ptr(exp_avg), _ptr(exp_avg_sq), beta1, beta2, lr,
                                                    weight_decay, eps, step, n, _stream()))


class TensorList:
    """A host-side ``lpmm_b200_tensor`` array for the multi-tensor step.  Entries are
    (p, g, m, v, m_scale, v_scale) with scales ``None`` for fp32-state tensors."""

    def __init__(self, entries):
        self.n = len(entries)
        self.array = (N.Tensor * max(self.n, 1))()
        self._keep = entries  # keep the tensors alive while the descriptors exist
        for i, (p, g, m, v, sm, sv) in enumerate(entries):
            kind = N.KIND_Q4 if sm is not None else N.KIND_FP32
            self.array[i] = N.Tensor(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                     sm.data_ptr() if sm is not None else None,
                                     sv.data_ptr() if sv is not None else None, p.numel(), kind, 0)
        self.total_groups = int(N.lib.lpmm_b200_count_groups(self.array, self.n)) if self.n else 0

    def set_grads(self, grads):
        for i, g in enumerate(grads):
            self.array[i].g = g.data_ptr()


_DTYPE16 = {torch.bfloat16: N.DTYPE_BF16, torch.float16: N.DTYPE_FP16}


def adamw4bit_multi_tensor(tl, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, step, group_begin=0, group_end=-1,
                           dtype=torch.float32, exact_params=True):
    """``dtype``: element type of every parameter and gradient of the list (fp32, or bf16 / fp16 for
    ``lpmm_b200_adamw4bit_multi_tensor_16bit``).  ``exact_params=False``: the parameter update may differ from
    the reference's in the last bits (``LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE``); moments, scales and codes
    are the same either way."""
    if tl.n == 0:
        return
    h = N.Hyper(beta1, beta2, lr, weight_decay, eps, step)
    flags = 0 if exact_params else N.FLAG_PARAMS_WITHIN_TOLERANCE
    if dtype != torch.float32:
        N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_flags(tl.array, tl.n, _DTYPE16[dtype], _ptr(qmap_m),
                                                                   _ptr(qmap_v), h, group_begin, group_end, flags,
                                                                   _stream()))
        return
    N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(tl.array, tl.n, _ptr(qmap_m), _ptr(qmap_v), h, group_begin,
                                                         group_end, flags, _stream()))


def sgd4bit_multi_tensor(tl, qmap, *, weight_decay, momentum, lr, dampening, nesterov, maximize, group_begin=0,
                         group_end=-1):
    """Momentum SGD of a ``TensorList`` (entries ``(p, g, buffer, buffer, max1 or None, None)``) in one
    launch; buffers must be initialised."""
    if tl.n == 0:
        return
    N.check(N.lib.lpmm_b200_sgd4bit_multi_tensor(tl.array, tl.n, _ptr(qmap), weight_decay, momentum, lr, dampening,
                                                 int(bool(nesterov)), int(bool(maximize)), group_begin, group_end,
                                                 _stream()))


# ----------------------------------------------------------------------------------------------
# standalone quantize / dequantize
# ----------------------------------------------------------------------------------------------
SUPPORTED_BITS = (4, 5, 6, 7, 8)
SUPPORTED_GROUPS = (128, 256, 512, 1024, 2048, 4096)


def packed_len(n_scaled, bits=4):
    """Bytes of the packed-code tensor for ``n_scaled`` normalised values: rows of 2048 codes, two
    codes per byte for 4 bits and one per byte for 5 to 8, plus one trailing byte."""
    rows = (n_scaled + 2047) // 2048
    return rows * (1024 if bits == 4 else 2048) + 1


def _check_layout(bits, gp_sz=128):
    if bits not in SUPPORTED_BITS:
        raise NotImplementedError(f"code widths {SUPPORTED_BITS} are built in this implementation, not {bits}")
    if gp_sz not in SUPPORTED_GROUPS:
        raise NotImplementedError(f"group sizes {SUPPORTED_GROUPS} are built in this implementation, not {gp_sz}")


def _check_qmap(qmap, bits):
    if qmap.numel() != (1 << bits):
        raise RuntimeError(f"a {bits}-bit quantization map must have {1 << bits} entries, got {qmap.numel()}")


def _i64_array(values):
    return (ctypes.c_int64 * max(len(values), 1))(*values)


def _ptr_array(tensors):
    return (_vp * max(len(tensors), 1))(*[t.data_ptr() for t in tensors])


def philox_inputs(device, bits):
    """What the reference's pack kernels take from torch's default CUDA generator on every call,
    stochastic or not (``gen->philox_engine_inputs(group_size * work_per_thread)`` with group_size 2048,
    quantization_kernel.cu:479-487, 556-564): returns ``(seed, offset)`` and advances the generator's
    offset by 16384 (4-bit codes) or 8192 (wider codes)."""
    gen = torch.cuda.default_generators[device.index if device.index is not None else torch.cuda.current_device()]
    offset = gen.get_offset()
    gen.set_offset(offset + (16384 if bits == 4 else 8192))
    return gen.initial_seed(), offset


def pack_nonlinear(data, qmap, bits, stochastic):
    """``quantization.pack_nonlinear`` (reference quantization.cc:54-63).  ``stochastic=True`` draws from
    torch's default CUDA generator exactly as the reference does (same codes for the same generator
    state); ``stochastic=False`` leaves the generator alone (the reference advances it there too)."""
    if bits > 8:
        raise RuntimeError("bits <= 8")
    _check_cuda_float(data, "data")
    _check_cuda_float(qmap, "qmap")
    if data.dim() != 2 or qmap.dim() != 1:
        raise RuntimeError("The dimension of data / qmap is not correct!")
    _check_layout(bits)
    _check_qmap(qmap, bits)
    if data.shape[1] % (8 if bits == 4 else 4) != 0:
        raise RuntimeError("group_size % work_per_thread == 0")
    n = data.numel()
    out = torch.empty((n // 2 if bits == 4 else n) + 1, dtype=torch.int8, device=data.device)
    with torch.cuda.device(data.device):
        if stochastic:
            if n % 8 != 0:
                raise NotImplementedError("the stochastic pack needs a multiple of 8 values")
            seed, offset = philox_inputs(data.device, bits)
            N.check(N.lib.lpmm_b200_pack_nonlinear_sr(_ptr(data), n, _ptr(qmap), bits, _ptr(out), seed, offset, _stream()))
        else:
            N.check(N.lib.lpmm_b200_pack_nonlinear(_ptr(data), n, _ptr(qmap), bits, _ptr(out), _stream()))
    return out


def unpack_nonlinear(data, qmap, bits, num_groups, group_size):
    """``quantization.unpack_nonlinear`` (reference quantization.cc:65-76)."""
    if bits > 8:
        raise RuntimeError("bits <= 8")
    _check_cuda_int8(data, "data")
    _check_cuda_float(qmap, "qmap")
    if data.dim() != 1 or qmap.dim() != 1:
        raise RuntimeError("The dimension of data / qmap is not correct!")
    _check_layout(bits)
    _check_qmap(qmap, bits)
    n = int(num_groups) * int(group_size)
    if data.numel() < (n // 2 if bits == 4 else n):
        raise RuntimeError("packed tensor is too short for num_groups * group_size codes")
    out = torch.empty((int(num_groups), int(group_size)), dtype=qmap.dtype, device=data.device)
    with torch.cuda.device(data.device):
        N.check(N.lib.lpmm_b200_unpack_nonlinear(_ptr(data), _ptr(qmap), bits, n, _ptr(out), _stream()))
    return out


def _qmap_on(qmap, device):
    return qmap if qmap.device == device else qmap.to(device)


def _groups(n, gp_sz):
    return (n + gp_sz - 1) // gp_sz


def quant_group(x, qmap, gp_sz, bits=4, sr=None):
    """``sr``: ``(seed, offset)`` from ``philox_inputs`` for stochastic rounding, None for nearest."""
    _check_layout(bits, gp_sz)
    _check_qmap(qmap, bits)
    _check_cuda_float(x, "x")
    n = x.numel()
    groups = _groups(n, gp_sz)
    codes = torch.empty(packed_len(groups * gp_sz, bits), dtype=torch.int8, device=x.device)
    max1 = torch.empty((groups, 1), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        if sr is not None:
            N.check(N.lib.lpmm_b200_quant_group_sr(_ptr(x), n, _ptr(_qmap_on(qmap, x.device)), bits, gp_sz, _ptr(codes),
                                                   _ptr(max1), sr[0], sr[1], _stream()))
        else:
            N.check(N.lib.lpmm_b200_quant_group(_ptr(x), n, _ptr(_qmap_on(qmap, x.device)), bits, gp_sz, _ptr(codes),
                                                _ptr(max1), _stream()))
    return codes, max1


def dequant_group(codes, qmap, max1, numel, gp_sz, bits=4):
    _check_layout(bits, gp_sz)
    _check_qmap(qmap, bits)
    _check_cuda_int8(codes, "qx")
    out = torch.empty(numel, dtype=torch.float32, device=codes.device)
    with torch.cuda.device(codes.device):
        N.check(N.lib.lpmm_b200_dequant_group(_ptr(codes), _ptr(_qmap_on(qmap, codes.device)), bits, gp_sz, _ptr(max1),
                                              numel, _ptr(out), _stream()))
    return out


def dequant_plain(codes, qmap, n, bits=4):
    _check_layout(bits)
    _check_qmap(qmap, bits)
    _check_cuda_int8(codes, "qx")
    n2 = (n + 1) // 2 * 2
    out = torch.empty(n2, dtype=torch.float32, device=codes.device)
    with torch.cuda.device(codes.device):
        N.check(N.lib.lpmm_b200_unpack_nonlinear(_ptr(codes), _ptr(_qmap_on(qmap, codes.device)), bits, n2, _ptr(out),
                                                 _stream()))
    return out[:n]


def _axis_vectors(shape, device):
    nd = len(shape)
    return [torch.empty([shape[i] if j == i else 1 for j in range(nd)], dtype=torch.float32, device=device)
            for i in range(nd)]


def axis_absmax(x):
    _check_cuda_float(x, "x")
    if x.dim() < 1 or x.dim() > 8:
        raise NotImplementedError("1 to 8 dimensions")
    vecs = _axis_vectors(tuple(x.shape), x.device)
    with torch.cuda.device(x.device):
        N.check(N.lib.lpmm_b200_axis_absmax(_ptr(x), _i64_array(list(x.shape)), x.dim(), _ptr_array(vecs), _stream()))
    return vecs


def quant_rank1(x, qmap, bits=4, sr=None):
    _check_layout(bits)
    _check_qmap(qmap, bits)
    _check_cuda_float(x, "x")
    if x.dim() < 2 or x.dim() > 8:
        raise NotImplementedError("2 to 8 dimensions")
    vecs = _axis_vectors(tuple(x.shape), x.device)
    codes = torch.empty(packed_len(x.numel(), bits), dtype=torch.int8, device=x.device)
    with torch.cuda.device(x.device):
        if sr is not None:
            N.check(N.lib.lpmm_b200_quant_rank1_sr(_ptr(x), _i64_array(list(x.shape)), x.dim(),
                                                   _ptr(_qmap_on(qmap, x.device)), bits, _ptr_array(vecs), _ptr(codes),
                                                   sr[0], sr[1], _stream()))
        else:
            N.check(N.lib.lpmm_b200_quant_rank1(_ptr(x), _i64_array(list(x.shape)), x.dim(),
                                                _ptr(_qmap_on(qmap, x.device)), bits, _ptr_array(vecs), _ptr(codes),
                                                _stream()))
    return codes, vecs


def dequant_rank1(codes, qmap, max_dims, shape, bits=4):
    _check_layout(bits)
    _check_qmap(qmap, bits)
    _check_cuda_int8(codes, "qx")
    out = torch.empty(tuple(shape), dtype=torch.float32, device=codes.device)
    with torch.cuda.device(codes.device):
        N.check(N.lib.lpmm_b200_dequant_rank1(_ptr(codes), _ptr(_qmap_on(qmap, codes.device)), bits,
                                              _ptr_array(list(max_dims)), _i64_array(list(shape)), len(shape), _ptr(out),
                                              _stream()))
    return out


# ----------------------------------------------------------------------------------------------
# non-fused optimizer steps (one tensor per call)
# ----------------------------------------------------------------------------------------------
_scratch = {}


def _scratch_for(device, nbytes):
    buf = _scratch.get(device)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[device] = buf
    return buf


def _check_param_grad(p, g):
    _check_cuda_float(p, "p")
    _check_cuda_float(g, "g")
    if g.numel() != p.numel():
        raise RuntimeError("number of elements in g and p tensors should be equal")


def _check_group_md(md, what):
    if md["round_type"] != "real-nearest":
        raise NotImplementedError(f"{what}: only round_type 'real-nearest' is built in this implementation")
    _check_layout(md["b"], md["gp_sz"])


def _ensure_group_state(state, name, p, quantized, bits=4, gp_sz=128):
    """Allocate the storage of a group-scaled / fp32 state on first use; returns (tensor, max1, first)."""
    t = state[name]
    first = t.numel() <= 1  # the reference's test for "not initialised yet" (adamw.py:394)
    oh = state[f"{name}_qstate"]["overhead"]
    if quantized:
        n = p.numel()
        groups = _groups(n, gp_sz)
        if not first and t.dtype != torch.int8:
            # an initialised moment that is not packed although quantization is now enabled (a checkpoint saved
            # with this state in fp32, a changed threshold): quantise what is there, never pair fresh storage
            # with first = False
            if t.numel() != n or not t.is_floating_point():
                raise RuntimeError(f"{name}: an initialised state of {t.numel()} {t.dtype} elements cannot become the "
                                   f"quantized state of a parameter of {n} elements")
            codes, max1 = quant_group(t.detach().to(torch.float32).contiguous().view(-1),
                                      state[f"{name}_qstate"]["qmap"], gp_sz, bits)
            t.data = codes
            oh["max1"] = max1
        elif first:
            t.data = torch.empty(packed_len(groups * gp_sz, bits), dtype=torch.int8, device=p.device)
        if not isinstance(oh.get("max1"), torch.Tensor) or oh["max1"].numel() != groups:
            if not first:
                raise RuntimeError(f"{name}: packed codes without their {groups} group scales (overhead['max1'])")
            oh["max1"] = torch.empty((groups, 1), dtype=torch.float32, device=p.device)
        oh["dtype"], oh["stride"] = p.dtype, p.stride()
        oh["scaled_shape"] = torch.Size([groups, gp_sz])
        return t, oh["max1"], first
    if first:
        t.data = torch.zeros_like(p, memory_format=torch.preserve_format)
    return t, None, first


class _StepPlan:
    """The ``lpmm_b200_step_tensor`` of one parameter, kept between steps: as long as the parameter, its
    state tensors and their storage are the ones the plan was built for, a step only refreshes the
    gradient pointer and launches.  Rank-1 tensors alternate between two descriptors (the per-axis
    maxima the codes were written with / the ones being computed swap roles every step)."""
    __slots__ = ("p_ptr", "m", "v", "m_ptr", "v_ptr", "g_ptr", "numel", "descs", "which", "axis_sets", "oh_v",
                 "scratch", "extra")

    def matches(self, p, state):
        m, v = state["exp_avg"], state.get("exp_avg_sq")
        if p.data_ptr() != self.p_ptr or m is not self.m or v is not self.v or m.data_ptr() != self.m_ptr:
            return False
        if v is not None and v.data_ptr() != self.v_ptr:
            return False
        if self.axis_sets is not None and self.oh_v.get("max_dims") is not self.axis_sets[self.which]:
            return False
        for k, t, ptr in self.extra:
            if state.get(k) is not t or t.data_ptr() != ptr:
                return False
        return True

    def set_grad(self, g):
        gp = g.data_ptr()
        if gp != self.g_ptr:
            if g.dtype != torch.float32 or not g.is_cuda or not g.is_contiguous() or g.numel() != self.numel:
                return False
            for d in self.descs:
                d.g = gp
            self.g_ptr = gp
        return True


def _make_plan(t, p, g, state, axis_sets=None, oh_v=None):
    plan = _StepPlan()
    plan.p_ptr, plan.g_ptr, plan.numel = p.data_ptr(), g.data_ptr(), p.numel()
    plan.m, plan.v = state["exp_avg"], state.get("exp_avg_sq")
    plan.m_ptr = plan.m.data_ptr()
    plan.v_ptr = plan.v.data_ptr() if plan.v is not None else None
    plan.axis_sets, plan.oh_v, plan.which, plan.scratch, plan.extra = axis_sets, oh_v, 0, None, ()
    t.first = 0
    if axis_sets is None:
        plan.descs = [t]
    else:
        # descriptor k reads the maxima in axis_sets[k] and writes axis_sets[1 - k]
        t2 = N.StepTensor()
        ctypes.memmove(ctypes.byref(t2), ctypes.byref(t), ctypes.sizeof(t))
        for i in range(len(axis_sets[0])):
            t.v_max_dims_old[i], t.v_max_dims_new[i] = axis_sets[0][i].data_ptr(), axis_sets[1][i].data_ptr()
            t2.v_max_dims_old[i], t2.v_max_dims_new[i] = axis_sets[1][i].data_ptr(), axis_sets[0][i].data_ptr()
        plan.descs = [t, t2]
    return plan


def _step_one(desc, qm, qv, beta1, beta2, lr, weight_decay, eps, step, stream, fused_arith):
    if fused_arith:
        N.check(N.lib.lpmm_b200_adamw4bit_fused_arith_step(ctypes.byref(desc), _ptr(qm), _ptr(qv), beta1, beta2, lr,
                                                           weight_decay, eps, step, stream))
    else:
        N.check(N.lib.lpmm_b200_adamw4bit_unfused_step(ctypes.byref(desc), _ptr(qm), _ptr(qv), beta1, beta2, lr,
                                                       weight_decay, eps, step, None, 0, stream))


def adamw4bit_unfused_step(p, g, state, m_quant, v_quant, md_m, md_v, spare, *, beta1, beta2, lr, weight_decay, eps,
                           step, stream=None, fused_arith=False):
    """``spare`` is a dict owned by the optimizer (not part of its state) that keeps the second set
    of per-axis maxima a rank-1 tensor alternates with, and the descriptor cached between steps.
    ``stream``: raw handle of torch's current stream when the caller has already looked it up and
    ``p``'s device is the current device (saves both look-ups per tensor).
    ``fused_arith``: the arithmetic of the reference's fused kernel on these states
    (``lpmm_b200_adamw4bit_fused_arith_step``) instead of that of its torch operations."""
    plan = spare.get("plan")
    if plan is not None:
        if plan.matches(p, state) and plan.set_grad(g):
            qm = state["exp_avg_qstate"]["qmap"]
            qv = state["exp_avg_sq_qstate"]["qmap"]
            if stream is not None:
                _step_one(plan.descs[plan.which], qm, qv, beta1, beta2, lr, weight_decay, eps, step, _vp(stream), fused_arith)
            else:
                with torch.cuda.device(p.device):
                    _step_one(plan.descs[plan.which], qm, qv, beta1, beta2, lr, weight_decay, eps, step, _stream(),
                              fused_arith)
            if plan.axis_sets is not None:  # the freshly written maxima become the state's, the old set the spare
                plan.which ^= 1
                plan.oh_v["max_dims"], spare["max_dims"] = plan.axis_sets[plan.which], plan.axis_sets[plan.which ^ 1]
            return
        del spare["plan"]
    _check_param_grad(p, g)
    if m_quant:
        _check_group_md(md_m, "first moment")
        if md_m["scale_type"] != "group":
            raise NotImplementedError("first moment: only scale_type 'group' is built in this implementation")
    if v_quant:
        _check_group_md(md_v, "second moment")
        if md_v["scale_type"] not in ("group", "rank1"):
            raise NotImplementedError("second moment: only scale_type 'group' / 'rank1' is built in this implementation")
    if m_quant and v_quant and (md_m["b"] == 4) != (md_v["b"] == 4):
        raise NotImplementedError("4-bit and wider codes cannot be mixed within one tensor in this implementation")
    t = N.StepTensor()
    t.p, t.g, t.numel, t.ndim = p.data_ptr(), g.data_ptr(), p.numel(), max(p.dim(), 1)
    for i, d in enumerate(p.shape):
        t.shape[i] = d
    if m_quant:
        t.m_bits, t.m_group = md_m["b"], md_m["gp_sz"]
    if v_quant:
        t.v_bits, t.v_group = md_v["b"], md_v["gp_sz"]
    m, m_max1, first_m = _ensure_group_state(state, "exp_avg", p, m_quant, md_m["b"], md_m["gp_sz"])
    t.m_mode = N.STATE_GROUP4 if m_quant else N.STATE_FP32
    t.m, t.m_max1 = m.data_ptr(), (m_max1.data_ptr() if m_max1 is not None else None)
    rank1 = v_quant and md_v["scale_type"] == "rank1" and p.dim() >= 2
    oh_v = state["exp_avg_sq_qstate"]["overhead"]
    axis_sets = None
    if rank1:
        v = state["exp_avg_sq"]
        first_v = v.numel() <= 1
        if first_v:
            v.data = torch.empty(packed_len(p.numel(), md_v["b"]), dtype=torch.int8, device=p.device)
            oh_v["max_dims"] = _axis_vectors(tuple(p.shape), p.device)
        elif v.dtype != torch.int8:
            # an initialised fp32 second moment met by a step that wants it packed (see _ensure_group_state)
            if v.numel() != p.numel() or not v.is_floating_point():
                raise RuntimeError("exp_avg_sq: an initialised state of another size cannot become the quantized state")
            codes, vecs = quant_rank1(v.detach().to(torch.float32).contiguous().view(p.shape),
                                      state["exp_avg_sq_qstate"]["qmap"], md_v["b"])
            v.data = codes
            oh_v["max_dims"] = vecs
        if "max_dims" not in spare or spare["max_dims"][0].device != p.device:
            spare["max_dims"] = _axis_vectors(tuple(p.shape), p.device)
        old, new = oh_v["max_dims"], spare["max_dims"]
        for i in range(p.dim()):
            t.v_max_dims_old[i] = old[i].data_ptr()
            t.v_max_dims_new[i] = new[i].data_ptr()
        t.v_mode, t.v = N.STATE_RANK1_4, v.data_ptr()
        new, old = list(new), list(old)
        oh_v["max_dims"], spare["max_dims"] = new, old
        oh_v.update(dim=p.dim(), max1=None, scaled_shape=p.shape, dtype=p.dtype, stride=p.stride())
        axis_sets = [new, old]  # after this step the state's maxima are `new`
    else:
        v, v_max1, first_v = _ensure_group_state(state, "exp_avg_sq", p, v_quant, md_v["b"], md_v["gp_sz"])
        if v_quant and md_v["scale_type"] == "rank1":
            oh_v["dim"] = p.dim()
        t.v_mode = N.STATE_GROUP4 if v_quant else N.STATE_FP32
        t.v, t.v_max1 = v.data_ptr(), (v_max1.data_ptr() if v_max1 is not None else None)
    if first_m != first_v:
        raise RuntimeError("exp_avg and exp_avg_sq must be initialised together")
    t.first = int(first_m)
    qm = state["exp_avg_qstate"]["qmap"]
    qv = state["exp_avg_sq_qstate"]["qmap"]
    with torch.cuda.device(p.device):
        _step_one(t, qm, qv, beta1, beta2, lr, weight_decay, eps, step, _stream(), fused_arith)
    spare["plan"] = _make_plan(t, p, g, state, axis_sets, oh_v if rank1 else None)


def unfused_step_many_scratch_bytes(ptrs, n):
    need = int(N.lib.lpmm_b200_unfused_step_many_scratch_bytes(ptrs, n))
    if need < 0:
        N.check(need)
    return need


def adamw4bit_unfused_step_many(ptrs, n, qm, qv, steps, scratch_need, device, *, beta1, beta2, lr, weight_decay, eps,
                                fused_arith=False, exact_params=True):
    """``ptrs``: ctypes array of n addresses of ``lpmm_b200_step_tensor`` descriptors (kept alive and up
    to date by the caller), ``steps``: ctypes array of n doubles, ``scratch_need``: what
    ``unfused_step_many_scratch_bytes`` returned for them.  The caller guarantees that ``device`` is the
    current device.  ``exact_params=False``: the tolerance mode of the list-wide kernels (states unchanged,
    parameters within 1e-6 relative)."""
    scratch = _scratch_for(device, scratch_need)
    fn = (N.lib.lpmm_b200_adamw4bit_fused_arith_step_many_flags if fused_arith
          else N.lib.lpmm_b200_adamw4bit_unfused_step_many_flags)
    N.check(fn(ptrs, n, _ptr(qm), _ptr(qv), beta1, beta2, lr, weight_decay, eps, steps, _ptr(scratch),
               scratch.numel() if scratch is not None else 0, _stream(),
               0 if exact_params else N.FLAG_PARAMS_WITHIN_TOLERANCE))


def adamw_fp32_moments_step(p, g, m, v, row, col, *, beta1, beta2, lr, weight_decay, eps, step):
    """One non-fused step on fp32 moments given as plain tensors (``v`` None: factored, ``row`` / ``col``
    are the accumulators).  Used where the moments are quantized outside the step (stochastic rounding)."""
    _check_param_grad(p, g)
    _check_cuda_float(m, "exp_avg")
    t = N.StepTensor()
    t.p, t.g, t.numel, t.ndim, t.first = p.data_ptr(), g.data_ptr(), p.numel(), max(p.dim(), 1), 0
    for i, d in enumerate(p.shape):
        t.shape[i] = d
    t.m_mode, t.m = N.STATE_FP32, m.data_ptr()
    scratch = None
    if v is not None:
        _check_cuda_float(v, "exp_avg_sq")
        t.v_mode, t.v = N.STATE_FP32, v.data_ptr()
    else:
        _check_cuda_float(row, "exp_avg_sq_row")
        _check_cuda_float(col, "exp_avg_sq_col")
        t.v_mode, t.row, t.col = N.STATE_FACTORED, row.data_ptr(), col.data_ptr()
        need = int(N.lib.lpmm_b200_factored_scratch_bytes(_i64_array(list(p.shape)), p.dim()))
        scratch = _scratch_for(p.device, need)
    with torch.cuda.device(p.device):
        N.check(N.lib.lpmm_b200_adamw4bit_unfused_step(ctypes.byref(t), None, None, beta1, beta2, lr, weight_decay, eps,
                                                       step, _ptr(scratch), scratch.numel() if scratch is not None else 0,
                                                       _stream()))


def sgd_fp32_buffer_step(p, g, buf, first, *, weight_decay, momentum, lr, dampening, nesterov, maximize):
    """Momentum SGD on an fp32 buffer given as a plain tensor (``first``: it receives the decayed gradient)."""
    _check_param_grad(p, g)
    with torch.cuda.device(p.device):
        N.check(N.lib.lpmm_b200_sgd_lowbit_step(_ptr(p), _ptr(g), p.numel(), _ptr(buf), None, N.STATE_FP32, 4, 128,
                                                int(first), None, weight_decay, momentum, lr, dampening,
                                                int(bool(nesterov)), int(bool(maximize)), _stream()))


def adamw4bit_factored_step(p, g, state, m_quant, md_m, *, beta1, beta2, lr, weight_decay, eps, step, spare=None):
    plan = spare.get("plan") if spare is not None else None
    if plan is not None:
        if plan.matches(p, state) and plan.set_grad(g):
            scratch = _scratch_for(p.device, plan.scratch)
            with torch.cuda.device(p.device):
                N.check(N.lib.lpmm_b200_adamw4bit_unfused_step(ctypes.byref(plan.descs[0]),
                                                               _ptr(state["exp_avg_qstate"]["qmap"]), None, beta1, beta2,
                                                               lr, weight_decay, eps, step, _ptr(scratch),
                                                               scratch.numel(), _stream()))
            return
        del spare["plan"]
    _check_param_grad(p, g)
    if m_quant:
        _check_group_md(md_m, "first moment")
        if md_m["scale_type"] != "group":
            raise NotImplementedError("first moment: only scale_type 'group' is built in this implementation")
    t = N.StepTensor()
    t.p, t.g, t.numel, t.ndim = p.data_ptr(), g.data_ptr(), p.numel(), p.dim()
    for i, d in enumerate(p.shape):
        t.shape[i] = d
    if m_quant:
        t.m_bits, t.m_group = md_m["b"], md_m["gp_sz"]
    m, m_max1, first = _ensure_group_state(state, "exp_avg", p, m_quant, md_m["b"], md_m["gp_sz"])
    t.m_mode = N.STATE_GROUP4 if m_quant else N.STATE_FP32
    t.m, t.m_max1 = m.data_ptr(), (m_max1.data_ptr() if m_max1 is not None else None)
    t.v_mode = N.STATE_FACTORED
    row, col = state["exp_avg_sq_row"], state["exp_avg_sq_col"]
    _check_cuda_float(row, "exp_avg_sq_row")
    _check_cuda_float(col, "exp_avg_sq_col")
    t.row, t.col, t.first = row.data_ptr(), col.data_ptr(), int(first)
    shape = _i64_array(list(p.shape))
    need = int(N.lib.lpmm_b200_factored_scratch_bytes(shape, p.dim()))
    scratch = _scratch_for(p.device, need)
    qm = state["exp_avg_qstate"]["qmap"]
    with torch.cuda.device(p.device):
        N.check(N.lib.lpmm_b200_adamw4bit_unfused_step(ctypes.byref(t), _ptr(qm), None, beta1, beta2, lr, weight_decay,
                                                       eps, step, _ptr(scratch), scratch.numel(), _stream()))
    if spare is not None:
        plan = _make_plan(t, p, g, state)
        plan.scratch = need
        # the accumulators are part of what the descriptor points at
        plan.extra = (("exp_avg_sq_row", row, row.data_ptr()), ("exp_avg_sq_col", col, col.data_ptr()))
        spare["plan"] = plan


def sgd4bit_step(p, g, state, quant, md, *, weight_decay, momentum, lr, dampening, nesterov, maximize):
    _check_param_grad(p, g)
    bits, gp_sz = 4, 128
    if quant:
        _check_group_md(md, "momentum buffer")
        if md["scale_type"] != "group":
            raise NotImplementedError("momentum buffer: only scale_type 'group' is built in this implementation")
        bits, gp_sz = md["b"], md["gp_sz"]
    buf = buf_max1 = None
    first = False
    if momentum != 0:
        b = state["momentum_buffer"]
        first = b.numel() <= 1
        oh = state["momentum_buffer_qstate"]["overhead"]
        if quant:
            groups = _groups(p.numel(), gp_sz)
            if first:
                b.data = torch.empty(packed_len(groups * gp_sz, bits), dtype=torch.int8, device=p.device)
                oh["max1"] = torch.empty((groups, 1), dtype=torch.float32, device=p.device)
            oh.update(dtype=p.dtype, stride=p.stride(), scaled_shape=torch.Size([groups, gp_sz]))
            buf_max1 = oh["max1"]
        elif first:
            b.data = torch.empty_like(p, memory_format=torch.preserve_format)
        buf = b
    qmap = state["momentum_buffer_qstate"]["qmap"]
    with torch.cuda.device(p.device):
        N.check(N.lib.lpmm_b200_sgd_lowbit_step(_ptr(p), _ptr(g), p.numel(), _ptr(buf), _ptr(buf_max1),
                                                N.STATE_GROUP4 if quant else N.STATE_FP32, bits, gp_sz, int(first),
                                                _ptr(qmap), weight_decay, momentum, lr, dampening,
                                                int(bool(nesterov)), int(bool(maximize)), _stream()))
