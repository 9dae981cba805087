"""``lpmm.optim.AdamW(fused=True, fused_rank1=True)`` with the default configuration (4-bit group-128 first
moment, 4-bit rank-1 second moment) on a B200: the fused kernel's arithmetic on the states of the
non-fused step (``lpmm_b200_adamw4bit_fused_arith_step`` / ``_step_many``).

The reference has no such step (its fused=True falls back to group scales, lpmm/optim/adamw.py:503-506),
so the oracle is a composition of its parts, each pinned on its own: the reference's dequantisation and
quantisation (``oracle/torch_ref.py``) around the element-wise update of its fused kernels
(``oracle/lpmm_oracle.c``), with the device's bias corrections.  Codes, scales, per-axis maxima and
parameters must be bit-identical.  Tensors whose second moment keeps group scales (vectors) must also
agree with the fused multi-tensor kernel itself."""
import ctypes

import pytest
import torch

from gpu_helpers import bits_equal, device, nibbles, student_t
from golden_cases import THRESHOLD
from test_gpu_unfused import _check_adamw, _dev, _make_opt

pytestmark = pytest.mark.gpu


def _device_bias_corrections(beta1, beta2, step):
    from lpmm import _native as N
    out = torch.zeros(2, device=device())
    N.check(N.lib.lpmm_b200_bias_corrections(beta1, beta2, float(step), ctypes.c_void_p(out.data_ptr()),
                                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    return tuple(float(x) for x in out.cpu().numpy())


def _run_pair(shapes, grads_of_step, steps, kw, qmaps, seed):
    from oracle import torch_ref as T
    qm, qv = _dev(qmaps["m"]), _dev(qmaps["v"])
    torch.manual_seed(seed)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    params = [torch.nn.Parameter(p.clone()) for p in p0s]
    opt = _make_opt("AdamW", params, dict(qconfig="default.yml", fused=True, fused_rank1=True, **kw))
    o_params = [p.clone() for p in p0s]
    o_states = [dict() for _ in p0s]
    b1, b2 = kw["betas"]
    for s in range(1, steps + 1):
        grads = grads_of_step(s)
        for p, g in zip(params, grads):
            p.grad = g.clone()
        opt.step()
        c = _device_bias_corrections(b1, b2, s)
        for i, (op, g) in enumerate(zip(o_params, grads)):
            quant = op.numel() > THRESHOLD
            T.adamw_step(op, g, o_states[i], qm, qv, m_quant=quant, v_quant=quant, v_scale_type="rank1", beta1=b1,
                         beta2=b2, lr=kw["lr"], weight_decay=kw["weight_decay"], eps=kw["eps"], step=float(s),
                         arithmetic="fused", c=c)
    torch.cuda.synchronize()
    return opt, params, o_states, o_params


@pytest.mark.parametrize("hyper", [dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01),
                                   dict(lr=3e-4, betas=(0.8, 0.95), eps=1e-6, weight_decay=0.0),
                                   dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-30, weight_decay=0.1)])
def test_fused_rank1_optimizer_against_composed_oracle(qmaps, hyper):
    """Matrices that are stepped together from the second step on (rows multiples of 8: wide, very narrow,
    shorter than a 128-element unit), shapes that stay on per-tensor launches (odd row length, 4-D),
    vectors (group scales) and small tensors (fp32 moments); 20 % exact zeros; eps = 1e-30 takes the IEEE
    sqrt / division branch."""
    shapes = [(1000, 768), (768, 3072), (130, 4104), (4097, 8), (333, 1024), (1024,), (3, 3, 64, 64), (70, 61),
              (5000, 16), (4100,), (2, 5, 7, 96)]
    opt, params, o_states, o_params = _run_pair(
        shapes, lambda s: [student_t(sh, s * 100003 + i, zero_fraction=0.2) for i, sh in enumerate(shapes)], 6, hyper,
        qmaps, 51)
    _check_adamw(opt, params, o_states, o_params, "rank1")


def test_fused_rank1_vectors_agree_with_the_fused_kernel(qmaps):
    """A vector keeps group scales under a rank-1 configuration (lpmm/functional.py:190-193), so with the
    fused arithmetic it must match the fused multi-tensor kernel itself: parameters and scales bit for
    bit, codes equal (the two state layouts differ only in padding)."""
    shapes = [(8192,), (5000,), (128 * 300 + 77,), (1000,)]
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(61)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    pa = [torch.nn.Parameter(p.clone()) for p in p0s]
    pb = [torch.nn.Parameter(p.clone()) for p in p0s]
    oa = _make_opt("AdamW", pa, dict(qconfig="default.yml", fused=True, fused_rank1=True, **kw))
    ob = _make_opt("AdamW", pb, dict(qconfig=None, fused=True, **kw))
    for s in range(1, 6):
        grads = [student_t(sh, s * 977 + i, zero_fraction=0.1) for i, sh in enumerate(shapes)]
        for a, b, g in zip(pa, pb, grads):
            a.grad = g.clone()
            b.grad = g.clone()
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    for a, b in zip(pa, pb):
        assert bits_equal(a.detach(), b.detach())
        sa, sb = oa.state[a], ob.state[b]
        n = a.numel()
        if n <= THRESHOLD:
            assert bits_equal(sa["exp_avg"], sb["exp_avg"]) and bits_equal(sa["exp_avg_sq"], sb["exp_avg_sq"])
            continue
        for name in ("exp_avg", "exp_avg_sq"):
            assert torch.equal(nibbles(sa[name], n), nibbles(sb[name], n)), name
            assert bits_equal(sa[f"{name}_qstate"]["overhead"]["max1"].reshape(-1),
                              sb[f"{name}_qstate"]["overhead"]["max1"].reshape(-1)), name


def test_fused_rank1_state_continues_under_the_non_fused_step(qmaps):
    """The states are those of fused=False: a state_dict written by the fused rank-1 step loads into a
    non-fused optimizer, which continues from it exactly as the oracle does."""
    from oracle import torch_ref as T
    shapes = [(256, 384), (3, 4, 40, 24), (6000,)]
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    grads_of = lambda s: [student_t(sh, s * 31 + i) for i, sh in enumerate(shapes)]
    opt, params, o_states, o_params = _run_pair(shapes, grads_of, 3, kw, qmaps, 71)
    sd = opt.state_dict()
    p2 = [torch.nn.Parameter(p.detach().clone()) for p in params]
    opt2 = _make_opt("AdamW", p2, dict(qconfig="default.yml", fused=False, **kw))
    opt2.load_state_dict(sd)
    for g in opt2.param_groups:
        g["fused"] = False
    qm, qv = _dev(qmaps["m"]), _dev(qmaps["v"])
    for s in range(4, 6):
        grads = grads_of(s)
        for p, g in zip(p2, grads):
            p.grad = g.clone()
        opt2.step()
        for i, (op, g) in enumerate(zip(o_params, grads)):
            T.adamw_step(op, g, o_states[i], qm, qv, m_quant=True, v_quant=True, v_scale_type="rank1", beta1=0.9,
                         beta2=0.999, lr=kw["lr"], weight_decay=kw["weight_decay"], eps=kw["eps"], step=float(s))
    torch.cuda.synchronize()
    _check_adamw(opt2, p2, o_states, o_params, "rank1")
