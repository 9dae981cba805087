"""Fused 4-bit AdamW kernel through the C ABI, on a B200, against (a) the reference's own compiled
kernels when ``oracle/_ref`` is present and (b) the C oracle.  Integer outputs (codes) and the
fp32 scales and parameters are all required to be bit-identical."""
import ctypes

import numpy as np
import pytest
import torch

from gpu_helpers import (HYPER, bits_equal, device, device_qmaps, fused_state, load_reference_extension, stream,
                         student_t, vp)

pytestmark = pytest.mark.gpu


def _lib():
    from lpmm import _native as N
    return N


def mine_step(N, p, g, st, qm, qv, step, h=HYPER):
    N.check(N.lib.lpmm_b200_adamw4bit_single_tensor(vp(p), vp(g), vp(st[0]), vp(st[1]), vp(st[2]), vp(st[3]), vp(qm),
                                                    vp(qv), h["beta1"], h["beta2"], h["lr"], h["weight_decay"],
                                                    h["eps"], float(step), p.numel(), stream()))


def ref_step(ref, p, g, st, qm, qv, step, h=HYPER):
    ref.adamw4bit_single_tensor(p, g, st[0], st[1], st[2], st[3], qm, qv, h["beta1"], h["beta2"], h["lr"],
                                h["weight_decay"], h["eps"], float(step))


def assert_same(p_a, st_a, p_b, st_b, what):
    assert torch.equal(st_a[0], st_b[0]), f"{what}: first-moment codes differ"
    assert torch.equal(st_a[1], st_b[1]), f"{what}: second-moment codes differ"
    assert bits_equal(st_a[2], st_b[2]), f"{what}: first-moment scales differ"
    assert bits_equal(st_a[3], st_b[3]), f"{what}: second-moment scales differ"
    assert bits_equal(p_a, p_b), f"{what}: parameters differ"


def _grad_cases():
    def zero_groups(n):
        def f(s):
            g = student_t((n,), 10 + s)
            g[: 128 * 5] = 0
            if s % 2:
                g[128 * 7: 128 * 9] = 0
            return g
        return f

    def mixed(n):
        def f(s):
            g = student_t((n,), 40 + s)
            sc = torch.ones(n // 128, device=device())
            sc[::3] = 1e-25
            sc[1::7] = 1e18
            sc[5::11] = 0
            return (g.view(-1, 128) * sc[:, None]).reshape(-1).contiguous()
        return f

    return [
        ("matrix_4096x4096", 4096 * 4096, 5, lambda s: student_t((4096, 4096), s).view(-1), {}),
        ("ragged_even", 128 * 37 + 70, 5, lambda s: student_t((128 * 37 + 70,), s), {}),
        ("tiny_6", 6, 3, lambda s: student_t((6,), s), {}),
        ("zero_groups", 128 * 64, 6, zero_groups(128 * 64), {}),
        ("tiny_grads", 128 * 64, 4, lambda s: student_t((128 * 64,), 20 + s, scale=1e-31), {}),
        ("huge_grads", 128 * 64, 4, lambda s: student_t((128 * 64,), 30 + s, scale=1e19), {}),
        ("mixed_scales", 128 * 256, 5, mixed(128 * 256), {}),
        ("eps_tiny", 128 * 100, 4, lambda s: student_t((128 * 100,), 50 + s), dict(eps=1e-20)),
        ("eps_zero", 128 * 100, 3, lambda s: student_t((128 * 100,), 60 + s), dict(eps=0.0)),
        ("other_betas", 128 * 100, 4, lambda s: student_t((128 * 100,), 70 + s),
         dict(beta1=0.5, beta2=0.9, weight_decay=0.0, lr=3e-2)),
    ]


@pytest.mark.parametrize("case", _grad_cases(), ids=lambda c: c[0])
def test_fused_matches_reference_kernels(qmaps, case):
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built (needs the reference checkout at build time)")
    N = _lib()
    name, n, steps, gfn, hov = case
    h = dict(HYPER, **hov)
    qm, qv, _ = device_qmaps(qmaps)
    torch.manual_seed(n % 1000)
    p_ref = torch.randn(n, device=device()) * 0.02
    p_my = p_ref.clone()
    st_ref, st_my = fused_state(n), fused_state(n)
    for s in range(1, steps + 1):
        g = gfn(s)
        mine_step(N, p_my, g, st_my, qm, qv, s, h)
        torch.cuda.synchronize()
        ref_step(ref, p_ref, g, st_ref, qm, qv, s, h)
        torch.cuda.synchronize()
        assert_same(p_my, st_my, p_ref, st_ref, f"{name} step {s}")


@pytest.mark.parametrize("eps", [1e-8, 1e-13])
def test_second_moments_below_the_domain_of_the_short_square_root(qmaps, eps):
    """Gradients of 1e-22 ... 1e-15 with no history: the second moments lie in (0, 2^-102), where the short square-root
    sequence is not the IEEE one (last bit in [2^-126, 2^-102); far off for denormals, which are below 2^-63 either
    way).  With eps = 1e-8 the short sequences are selected: a denormal's root vanishes against eps by construction of
    the host's selection, and a last-bit difference of the root can move the denominator only when the sum lands
    within 2^-19 of a rounding boundary -- so codes and scales are identical and at most a handful of the 2^20
    parameters may differ, by one unit in the last place.  With eps = 1e-13 the host selects the IEEE instantiation and
    everything is identical."""
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    n = 1 << 20
    h = dict(HYPER, eps=eps)
    torch.manual_seed(5)
    p_ref = torch.randn(n, device=device()) * 0.02
    p_my = p_ref.clone()
    st_ref, st_my = fused_state(n), fused_state(n)
    worst = 0
    for s in range(1, 4):
        gen = torch.Generator(device=device())
        gen.manual_seed(900 + s)
        mag = torch.pow(10.0, -22.0 + 7.0 * torch.rand(n, generator=gen, device=device()))
        sign = torch.where(torch.rand(n, generator=gen, device=device()) < 0.5, -1.0, 1.0)
        g = (mag * sign).contiguous()
        mine_step(N, p_my, g, st_my, qm, qv, s, h)
        ref_step(ref, p_ref, g, st_ref, qm, qv, s, h)
        torch.cuda.synchronize()
        for k in range(4):
            assert torch.equal(st_my[k].view(torch.uint8).view(-1), st_ref[k].view(torch.uint8).view(-1)), f"step {s}: state {k}"
        diff = (p_my.view(torch.int32) - p_ref.view(torch.int32)).abs()
        assert int(diff.max()) <= 1, f"step {s}: a parameter differs by more than one unit in the last place"
        worst = max(worst, int((diff != 0).sum()))
        p_my.copy_(p_ref)  # keep the two runs on the same trajectory
    assert worst <= (8 if eps == 1e-8 else 0), f"{worst} parameters differ"


def test_fused_nonlinear_second_moment_map(qmaps):
    """A second-moment map other than the linear one takes the table path instead of the closed form."""
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, _, qv2 = device_qmaps(qmaps)
    n = 128 * 100
    torch.manual_seed(1)
    p_ref = torch.randn(n, device=device()) * 0.02
    p_my = p_ref.clone()
    st_ref, st_my = fused_state(n), fused_state(n)
    for s in range(1, 5):
        g = student_t((n,), 80 + s)
        mine_step(N, p_my, g, st_my, qm, qv2, s)
        ref_step(ref, p_ref, g, st_ref, qm, qv2, s)
        torch.cuda.synchronize()
        assert_same(p_my, st_my, p_ref, st_ref, f"step {s}")


def test_fused_unaligned_views_match_reference(qmaps):
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    n = 128 * 50
    base = torch.randn(n + 8, device=device()) * 0.02
    gb = torch.randn(n + 8, device=device()) * 1e-3
    p_my, g_my = base[1:n + 1], gb[3:n + 3]
    p_ref, g_ref = p_my.clone(), g_my.clone()
    st_ref, st_my = fused_state(n), fused_state(n)
    for s in range(1, 4):
        mine_step(N, p_my, g_my, st_my, qm, qv, s)
        ref_step(ref, p_ref, g_ref, st_ref, qm, qv, s)
        torch.cuda.synchronize()
    assert_same(p_my, st_my, p_ref, st_ref, "unaligned")


@pytest.mark.parametrize("n", [128 * 3 + 77, 1, 127, 128, 4097, 128 * 37 + 70])
def test_fused_matches_c_oracle(qmaps, n):
    """Odd and ragged sizes (which the reference's binding rejects) against the C oracle, fed the
    device's own bias corrections so that parameters can be compared bit for bit too."""
    from oracle import cpu as O
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    torch.manual_seed(5)
    p = torch.randn(n, device=device()) * 0.02
    st = fused_state(n)
    p_o = p.cpu().numpy().copy()
    st_o = [x.cpu().numpy().copy() for x in st]
    st_o[0], st_o[1] = st_o[0].view(np.uint8), st_o[1].view(np.uint8)
    cdev = torch.zeros(2, device=device())
    for s in range(1, 5):
        g = student_t((n,), 90 + s)
        N.check(N.lib.lpmm_b200_bias_corrections(HYPER["beta1"], HYPER["beta2"], float(s), vp(cdev), stream()))
        torch.cuda.synchronize()
        c = cdev.cpu().numpy()
        mine_step(N, p, g, st, qm, qv, s)
        O.adamw4bit(p_o, g.cpu().numpy(), *st_o, qmaps["m"], qmaps["v"], HYPER["beta1"], HYPER["beta2"], HYPER["lr"],
                    HYPER["weight_decay"], HYPER["eps"], float(s), c=(float(c[0]), float(c[1])))
        torch.cuda.synchronize()
        assert np.array_equal(st[0].cpu().numpy().view(np.uint8), st_o[0])
        assert np.array_equal(st[1].cpu().numpy().view(np.uint8), st_o[1])
        assert np.array_equal(st[2].cpu().numpy().view(np.int32), st_o[2].view(np.int32))
        assert np.array_equal(st[3].cpu().numpy().view(np.int32), st_o[3].view(np.int32))
        assert np.array_equal(p.cpu().numpy().view(np.int32), p_o.view(np.int32))


def test_fused_fp32_state_kernel_matches_reference(qmaps):
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    for n in (4096, 127, 1000):
        torch.manual_seed(n)
        p_ref = torch.randn(n, device=device()) * 0.02
        p_my = p_ref.clone()
        m_r, v_r, m_m, v_m = (torch.zeros(n, device=device()) for _ in range(4))
        for s in range(1, 5):
            g = student_t((n,), 300 + s)
            N.check(N.lib.lpmm_b200_adamw_single_tensor(vp(p_my), vp(g), vp(m_m), vp(v_m), HYPER["beta1"], HYPER["beta2"],
                                                        HYPER["lr"], HYPER["weight_decay"], HYPER["eps"], float(s), n,
                                                        stream()))
            ref.adamw_single_tensor(p_ref, g, m_r, v_r, HYPER["beta1"], HYPER["beta2"], HYPER["lr"],
                                    HYPER["weight_decay"], HYPER["eps"], float(s))
            torch.cuda.synchronize()
            assert bits_equal(m_m, m_r) and bits_equal(v_m, v_r) and bits_equal(p_my, p_ref)


def test_multi_tensor_equals_single_tensor_and_shards(qmaps):
    """One launch over a mixed list (4-bit, fp32-state, ragged) equals per-tensor launches, and
    updating the list as two group ranges (ZeRO-1 shards) equals updating it at once."""
    from lpmm import _kernels as K
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    shapes = [(300, 128), (4096,), (5000,), (77, 129), (128,), (64, 64, 3)]

    def build(seed):
        torch.manual_seed(seed)
        out = []
        for s in shapes:
            n = int(np.prod(s))
            p = torch.randn(s, device=device()) * 0.02
            if n > 4096:
                st = fused_state(n)
                out.append([p, None, st[0], st[1], st[2], st[3]])
            else:
                out.append([p, None, torch.zeros(s, device=device()), torch.zeros(s, device=device()), None, None])
        return out

    a, b, c = build(3), build(3), build(3)
    for s in range(1, 4):
        grads = [student_t(sh, 500 + 10 * s + i) for i, sh in enumerate(shapes)]
        for lst in (a, b, c):
            for e, g in zip(lst, grads):
                e[1] = g
        # a: one launch
        K.adamw4bit_multi_tensor(K.TensorList([tuple(e) for e in a]), qm, qv, HYPER["beta1"], HYPER["beta2"],
                                 HYPER["lr"], HYPER["weight_decay"], HYPER["eps"], float(s))
        # b: per tensor
        for e in b:
            if e[4] is not None:
                mine_step(N, e[0], e[1], e[2:6], qm, qv, s)
            else:
                K.adamw_single_tensor(e[0], e[1], e[2], e[3], HYPER["beta1"], HYPER["beta2"], HYPER["lr"],
                                      HYPER["weight_decay"], HYPER["eps"], float(s))
        # c: two shards
        tl = K.TensorList([tuple(e) for e in c])
        cut = tl.total_groups // 3
        for lo, hi in ((0, cut), (cut, tl.total_groups)):
            K.adamw4bit_multi_tensor(tl, qm, qv, HYPER["beta1"], HYPER["beta2"], HYPER["lr"], HYPER["weight_decay"],
                                     HYPER["eps"], float(s), lo, hi)
        torch.cuda.synchronize()
        for ea, eb, ec in zip(a, b, c):
            for i in (0, 2, 3, 4, 5):
                if ea[i] is None:
                    continue
                x, y, z = ea[i], eb[i], ec[i]
                if x.dtype == torch.float32:
                    assert bits_equal(x, y) and bits_equal(x, z)
                else:
                    assert torch.equal(x, y) and torch.equal(x, z)


def test_argument_errors_are_reported_not_launched():
    N = _lib()
    lib = N.lib
    assert lib.lpmm_b200_adamw4bit_single_tensor(None, None, None, None, None, None, None, None, 0.9, 0.999, 1e-3, 0.0,
                                                 1e-8, 1.0, 128, None) == -1
    assert lib.lpmm_b200_adamw_single_tensor(None, None, None, None, 0.9, 0.999, 1e-3, 0.0, 1e-8, 1.0, -5, None) == -2
    with pytest.raises(N.NativeError):
        N.check(-2)


def test_hundred_free_running_steps_stay_identical_to_reference(qmaps):
    """The bar of the headline configuration: 100 optimizer steps on identical seeded inputs, free
    running (no state is copied between the two implementations): codes, scales and parameters are
    still bit-identical after the last step, so 'codes equal up to 1e-6 ties, parameters within 1e-6
    relative' holds with zero differences."""
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    shape = (1024, 1536)
    n = shape[0] * shape[1]
    torch.manual_seed(0)
    p_ref = (torch.randn(shape, device=device()) * 0.02).view(-1)
    p_my = p_ref.clone()
    st_ref, st_my = fused_state(n), fused_state(n)
    for s in range(1, 101):
        g = student_t(shape, s * 100003).view(-1)
        mine_step(N, p_my, g, st_my, qm, qv, s)
        ref_step(ref, p_ref, g, st_ref, qm, qv, s)
    torch.cuda.synchronize()
    assert_same(p_my, st_my, p_ref, st_ref, "after 100 steps")
    assert float((p_my - p_ref).abs().max()) == 0.0


def test_largest_tensor_of_the_7b_list_matches_reference(qmaps):
    """The 32000 x 4096 embedding (131 M elements, 1 024 000 groups) at full size, three steps."""
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        pytest.skip("oracle/_ref was not built")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    shape = (32000, 4096)
    n = shape[0] * shape[1]
    torch.manual_seed(0)
    p_ref = (torch.randn(shape, device=device()) * 0.02).view(-1)
    p_my = p_ref.clone()
    st_ref, st_my = fused_state(n), fused_state(n)
    for s in range(1, 4):
        g = student_t(shape, s * 100003 + 7).view(-1)
        mine_step(N, p_my, g, st_my, qm, qv, s)
        ref_step(ref, p_ref, g, st_ref, qm, qv, s)
        del g
    torch.cuda.synchronize()
    assert_same(p_my, st_my, p_ref, st_ref, "embedding-sized tensor")


def test_full_7b_list_one_launch_equals_per_tensor_launches(qmaps):
    """The headline workload at full size (6.74e9 parameters, 290 tensors): the single multi-tensor
    launch and 290 single-tensor launches on a second copy give identical parameters, codes and
    scales (compared through per-tensor integer checksums), for two consecutive steps."""
    from gpu_helpers import llama7b_shapes
    from lpmm import _kernels as K
    free, _ = torch.cuda.mem_get_info()
    if free < 120 * 2 ** 30:
        pytest.skip("needs about 110 GB of free device memory")
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    shapes = llama7b_shapes()
    gen = torch.Generator(device=device())
    gen.manual_seed(0)

    def build():
        out = []
        for s in shapes:
            n = int(np.prod(s))
            if n > 4096:
                st = fused_state(n)
                out.append([None, None, st[0], st[1], st[2], st[3]])
            else:
                out.append([None, None, torch.zeros(s, device=device()), torch.zeros(s, device=device()), None, None])
        return out

    a, b = build(), build()
    for ea, eb, s in zip(a, b, shapes):
        ea[0] = torch.empty(s, device=device()).normal_(0, 0.02, generator=gen)
        eb[0] = ea[0].clone()
        g = torch.empty(s, device=device()).normal_(0, 1e-3, generator=gen)
        ea[1] = eb[1] = g
    tl = K.TensorList([tuple(e) for e in a])

    def checksum(t):
        return int(t.contiguous().view(torch.uint8).view(-1).to(torch.int64).sum()) if t.dtype == torch.int8 else \
            int(t.contiguous().view(torch.int32).view(-1).to(torch.int64).sum())

    for step in (1, 2):
        K.adamw4bit_multi_tensor(tl, qm, qv, HYPER["beta1"], HYPER["beta2"], HYPER["lr"], HYPER["weight_decay"], HYPER["eps"],
                                 float(step))
        for e in b:
            if e[4] is not None:
                mine_step(N, e[0].view(-1), e[1].view(-1), e[2:6], qm, qv, step)
            else:
                K.adamw_single_tensor(e[0], e[1], e[2], e[3], HYPER["beta1"], HYPER["beta2"], HYPER["lr"],
                                      HYPER["weight_decay"], HYPER["eps"], float(step))
        torch.cuda.synchronize()
    for i, (ea, eb) in enumerate(zip(a, b)):
        for j in (0, 2, 3, 4, 5):
            if ea[j] is not None:
                assert checksum(ea[j]) == checksum(eb[j]), f"tensor {i}, field {j}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_list_longer_than_one_descriptor_window_equals_per_tensor_steps(qmaps, dtype):
    """450 tensors (4-bit, fp32-state, ragged) in one call: more than one launch's descriptor table holds (400), so the
    list is walked in two windows; a group range that crosses the window boundary; both element types.  Against the
    same tensors stepped one call each."""
    from lpmm import _kernels as K
    N = _lib()
    qm, qv, _ = device_qmaps(qmaps)
    shapes = [((41, 128) if i % 4 == 0 else (5000,) if i % 4 == 1 else (3000,) if i % 4 == 2 else (128 * 33 + 5,)) for i in range(450)]

    def build():
        torch.manual_seed(17)
        out = []
        for s in shapes:
            n = int(np.prod(s))
            p = (torch.randn(s, device=device()) * 0.02).to(dtype)
            if n > 4096:
                st = fused_state(n)
                out.append([p, None, st[0], st[1], st[2], st[3]])
            else:
                out.append([p, None, torch.zeros(s, device=device()), torch.zeros(s, device=device()), None, None])
        return out

    a, b, c = build(), build(), build()
    for s in range(1, 4):
        grads = [student_t(sh, 700 + 13 * s + i).to(dtype) for i, sh in enumerate(shapes)]
        for lst in (a, b, c):
            for e, g in zip(lst, grads):
                e[1] = g
        K.adamw4bit_multi_tensor(K.TensorList([tuple(e) for e in a]), qm, qv, HYPER["beta1"], HYPER["beta2"], HYPER["lr"],
                                 HYPER["weight_decay"], HYPER["eps"], float(s), dtype=dtype)
        for e in b:  # one call per tensor
            K.adamw4bit_multi_tensor(K.TensorList([tuple(e)]), qm, qv, HYPER["beta1"], HYPER["beta2"], HYPER["lr"],
                                     HYPER["weight_decay"], HYPER["eps"], float(s), dtype=dtype)
        tl = K.TensorList([tuple(e) for e in c])
        cut = tl.total_groups * 7 // 8 + 3  # inside the second window
        for lo, hi in ((0, cut), (cut, tl.total_groups)):
            K.adamw4bit_multi_tensor(tl, qm, qv, HYPER["beta1"], HYPER["beta2"], HYPER["lr"], HYPER["weight_decay"],
                                     HYPER["eps"], float(s), lo, hi, dtype=dtype)
    torch.cuda.synchronize()
    for i, (ea, eb, ec) in enumerate(zip(a, b, c)):
        for j in (0, 2, 3, 4, 5):
            if ea[j] is None:
                continue
            x, y, z = (t[j].contiguous().view(-1).view(torch.uint8) for t in (ea, eb, ec))
            assert torch.equal(x, y) and torch.equal(x, z), f"tensor {i}, field {j}"
