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


def adamw4bit_multi_tensor(tl, qmap_m, qmap_v, beta1, beta2, lr, weight_decay, eps, step, group_begin=0, group_end=-1):
    if tl.n == 0:
        return
    h = N.Hyper(beta1, beta2, lr, weight_decay, eps, step)
    N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor(tl.array, tl.n, _ptr(qmap_m), _ptr(qmap_v), h, group_begin, group_end,
                                                   _stream()))
