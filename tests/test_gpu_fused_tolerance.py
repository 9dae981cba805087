"""The tolerance mode of the fused step (``LPMM_B200_FLAG_PARAMS_WITHIN_TOLERANCE``,
``lpmm.optim.AdamW(fused=True, exact_params=False)``) on a B200, through the C ABI, against the reference's own
compiled kernel.

What must hold: packed codes and group scales of both moments bit-identical to the reference (they never depend
on the parameter), parameters within 1e-6 of the largest parameter magnitude after 100 free-running steps
(``max|p - p_ref| / max|p_ref| <= 1e-6``, the tolerance of the headline configuration)."""
import ctypes

import numpy as np
import pytest
import torch

from gpu_helpers import HYPER, bits_equal, device, device_qmaps, fused_state, load_reference_extension, stream, student_t, vp

pytestmark = pytest.mark.gpu

PARAM_TOL = 1e-6


def _lib():
    from lpmm import _native as N
    return N


def _tensor(N, p, g, st):
    return N.Tensor(p.data_ptr(), g.data_ptr(), st[0].data_ptr(), st[1].data_ptr(), st[2].data_ptr(), st[3].data_ptr(),
                    p.numel(), N.KIND_Q4, 0)


def tol_step(N, p, g, st, qm, qv, step, h=HYPER, flags=None):
    arr = (N.Tensor * 1)(_tensor(N, p, g, st))
    hy = N.Hyper(h["beta1"], h["beta2"], h["lr"], h["weight_decay"], h["eps"], float(step))
    N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(arr, 1, vp(qm), vp(qv), hy, 0, -1,
                                                         N.FLAG_PARAMS_WITHIN_TOLERANCE if flags is None else flags,
                                                         stream()))


def ref_step(ref, p, g, st, qm, qv, step, h=HYPER):
    ref.adamw4bit_single_tensor(p, g, st[0], st[1], st[2], st[3], qm, qv, h["beta1"], h["beta2"], h["lr"],
                                h["weight_decay"], h["eps"], float(step))


def _states_identical(st_a, st_b, what):
    assert torch.equal(st_a[0], st_b[0]), f"{what}: first-moment codes differ"
    assert torch.equal(st_a[1], st_b[1]), f"{what}: second-moment codes differ"
    assert bits_equal(st_a[2], st_b[2]), f"{what}: first-moment scales differ"
    assert bits_equal(st_a[3], st_b[3]), f"{what}: second-moment scales differ"


def _free_run(qmaps, shape, steps, seed_mul):
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    n = int(np.prod(shape))
    torch.manual_seed(0)
    p_ref = (torch.randn(shape, device=device()) * 0.02).view(-1)
    p_my = p_ref.clone()
    st_ref, st_my = fused_state(n), fused_state(n)
    for s in range(1, steps + 1):
        g = student_t(shape, s * seed_mul).view(-1)
        tol_step(N, p_my, g, st_my, qm, qv, s)
        ref_step(ref, p_ref, g, st_ref, qm, qv, s)
        del g
    torch.cuda.synchronize()
    _states_identical(st_my, st_ref, f"after {steps} steps")
    err = float((p_my - p_ref).abs().max()) / float(p_ref.abs().max())
    differing = float((p_my != p_ref).float().mean())
    print(f"tolerance mode, {shape}, {steps} steps: max|dp|/max|p| = {err:.3e}, parameters that differ: {differing:.3f}")
    assert err <= PARAM_TOL
    return err


def test_hundred_free_running_steps_codes_identical_params_within_tolerance(qmaps):
    _free_run(qmaps, (1024, 1536), 100, 100003)


def test_embedding_of_the_7b_list_hundred_steps(qmaps):
    """The 32000 x 4096 embedding at full size, 100 free-running steps."""
    _free_run(qmaps, (32000, 4096), 100, 100003 + 7)


def test_tolerance_mode_on_hard_inputs_keeps_states_identical(qmaps):
    """Zero groups, tiny and huge gradients, mixed scales: states identical, parameters close."""
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    n = 128 * 256

    def grads(kind, s):
        if kind == "tiny":
            return student_t((n,), 20 + s, scale=1e-31)
        if kind == "huge":
            return student_t((n,), 30 + s, scale=1e19)
        g = student_t((n,), 40 + s)
        sc = torch.ones(n // 128, device=device())
        sc[::3] = 1e-25
        sc[1::7] = 1e18
        sc[5::11] = 0
        return (g.view(-1, 128) * sc[:, None]).reshape(-1).contiguous()

    for kind in ("tiny", "huge", "mixed"):
        torch.manual_seed(3)
        p_ref = torch.randn(n, device=device()) * 0.02
        p_my = p_ref.clone()
        st_ref, st_my = fused_state(n), fused_state(n)
        for s in range(1, 6):
            g = grads(kind, s)
            tol_step(N, p_my, g, st_my, qm, qv, s)
            ref_step(ref, p_ref, g, st_ref, qm, qv, s)
        torch.cuda.synchronize()
        _states_identical(st_my, st_ref, kind)
        assert torch.isfinite(p_my).all()
        err = float((p_my - p_ref).abs().max()) / float(p_ref.abs().max())
        assert err <= PARAM_TOL, f"{kind}: {err}"


def test_hyper_parameters_outside_the_folded_constants_take_the_exact_update(qmaps):
    """lr = 0 (no finite 1 / lr) and eps = 0 (outside the short sequences): the flag is accepted and the result is the
    exact one, bit for bit."""
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    n = 128 * 100
    for hov in (dict(lr=0.0), dict(eps=0.0)):
        h = dict(HYPER, **hov)
        torch.manual_seed(4)
        p_ref = torch.randn(n, device=device()) * 0.02
        p_my = p_ref.clone()
        st_ref, st_my = fused_state(n), fused_state(n)
        for s in range(1, 4):
            g = student_t((n,), 60 + s)
            tol_step(N, p_my, g, st_my, qm, qv, s, h)
            ref_step(ref, p_ref, g, st_ref, qm, qv, s, h)
        torch.cuda.synchronize()
        _states_identical(st_my, st_ref, str(hov))
        assert bits_equal(p_my, p_ref)


def test_flags_zero_is_the_exact_step_and_unknown_flags_are_refused(qmaps):
    ref = load_reference_extension("fused_adamw")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    n = 128 * 64
    torch.manual_seed(6)
    p = torch.randn(n, device=device()) * 0.02
    g = student_t((n,), 77)
    st = fused_state(n)
    arr = (N.Tensor * 1)(_tensor(N, p, g, st))
    hy = N.Hyper(0.9, 0.999, 1e-3, 0.01, 1e-8, 1.0)
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(arr, 1, vp(qm), vp(qv), hy, 0, -1, 2, stream()) == -3
    assert N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_flags(arr, 1, N.DTYPE_BF16, vp(qm), vp(qv), hy, 0, -1, 8,
                                                              stream()) == -3
    if ref is not None:
        p_ref, st_ref = p.clone(), fused_state(n)
        tol_step(N, p, g, st, qm, qv, 1, flags=0)
        ref_step(ref, p_ref, g, st_ref, qm, qv, 1)
        torch.cuda.synchronize()
        _states_identical(st, st_ref, "flags = 0")
        assert bits_equal(p, p_ref)


def test_optimizer_exact_params_false_keeps_state_dict_identical(qmaps):
    """Through ``lpmm.optim.AdamW``: 20 steps of a small list with ``exact_params=False`` and with the default;
    optimizer states identical, parameters within tolerance."""
    import lpmm
    shapes = [(300, 256), (4096,), (128 * 41 + 6,), (64, 1000)]
    torch.manual_seed(9)
    init = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    pa = [torch.nn.Parameter(x.clone()) for x in init]
    pb = [torch.nn.Parameter(x.clone()) for x in init]
    oa = lpmm.optim.AdamW(pa, fused=True, exact_params=False)
    ob = lpmm.optim.AdamW(pb, fused=True)
    for s in range(20):
        for i, (a, b) in enumerate(zip(pa, pb)):
            a.grad = student_t(shapes[i], 1000 + 10 * s + i)
            b.grad = a.grad.clone()
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    for a, b in zip(pa, pb):
        sa, sb = oa.state[a], ob.state[b]
        if a.numel() > 4096:
            assert torch.equal(sa["exp_avg"], sb["exp_avg"]) and torch.equal(sa["exp_avg_sq"], sb["exp_avg_sq"])
            assert bits_equal(sa["exp_avg_qstate"]["overhead"]["max1"], sb["exp_avg_qstate"]["overhead"]["max1"])
            assert bits_equal(sa["exp_avg_sq_qstate"]["overhead"]["max1"], sb["exp_avg_sq_qstate"]["overhead"]["max1"])
        else:
            assert bits_equal(sa["exp_avg"], sb["exp_avg"]) and bits_equal(sa["exp_avg_sq"], sb["exp_avg_sq"])
        assert float((a.detach() - b.detach()).abs().max()) / float(b.detach().abs().max()) <= PARAM_TOL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_16bit_parameters_tolerance_mode_against_exact_mode(qmaps, dtype):
    """16-bit parameters are rounded to 8 (bf16) or 11 (fp16) significant bits on store, so the approximate update is
    invisible except where the exact fp32 result lies within ~1e-9 of a rounding boundary of the 16-bit format:
    states identical, and the parameters that differ do so by at most one unit in the last place of the 16-bit format
    (plus 2e-9 absolute where the step nearly cancels the parameter) and are few (the observed fraction is printed;
    the bound here is 1e-4 per step)."""
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    n = 128 * 8192
    torch.manual_seed(12)
    p0 = (torch.randn(n, device=device()) * 0.02).to(dtype)
    pa, pb = p0.clone(), p0.clone()
    sa, sb = fused_state(n), fused_state(n)
    dt = N.DTYPE_BF16 if dtype == torch.bfloat16 else N.DTYPE_FP16
    steps, differing = 10, 0
    for s in range(1, steps + 1):
        g = student_t((n,), 2000 + s, scale=1e-3 if dtype == torch.bfloat16 else 3e-5).to(dtype)
        hy = N.Hyper(0.9, 0.999, 1e-3, 0.01, 1e-8, float(s))
        pb.copy_(pa)  # teacher-forced parameters: count single-step differences
        for p, st, flags in ((pa, sa, N.FLAG_PARAMS_WITHIN_TOLERANCE), (pb, sb, 0)):
            arr = (N.Tensor * 1)(_tensor(N, p, g, st))
            N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_flags(arr, 1, dt, vp(qm), vp(qv), hy, 0, -1, flags, stream()))
        torch.cuda.synchronize()
        _states_identical(sa, sb, f"{dtype} step {s}")
        fa, fb = pa.float(), pb.float()
        ulp = torch.maximum(fa.abs(), fb.abs()) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)
        if dtype == torch.float16:
            ulp = ulp.clamp_min(2.0 ** -24)  # the spacing of fp16 subnormals
        assert bool(((fa - fb).abs() <= ulp + 2e-9).all())
        differing += int((pa.view(torch.int16) != pb.view(torch.int16)).sum())
    rate = differing / (n * steps)
    print(f"{dtype}: tolerance mode changes {rate:.2e} of the stored 16-bit parameters per step (by one ulp)")
    assert rate <= 1e-4
