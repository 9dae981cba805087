"""The multi-tensor forms of the non-fused step on a B200.  ``lpmm_b200_adamw4bit_unfused_multi_tensor``
-- a whole group/group list in one launch -- and the rank-1 matrices of a list stepped together
(``csrc/rank1_multi.cu``, reached through ``lpmm_b200_adamw4bit_unfused_step_many``): the optimizer (``lpmm.optim.AdamW(qconfig=None)``, which reaches it from a
tensor's second step on) against the torch-op restatement of the reference, and the entry point itself
against per-tensor calls of ``lpmm_b200_adamw4bit_unfused_step``, on unaligned views and in group ranges."""
import ctypes

import pytest
import torch

from gpu_helpers import bits_equal, device, student_t
from test_gpu_unfused import _check_adamw, _run_pair_adamw

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hyper", [dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01),
                                   dict(lr=3e-4, betas=(0.8, 0.95), eps=1e-6, weight_decay=0.0),
                                   dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-30, weight_decay=0.1)])
def test_optimizer_group_config_ragged_list(qmaps, hyper):
    """Ragged shapes, 20 % exact zeros, 7 steps (6 of them through the multi-tensor launch); eps = 1e-30
    takes the IEEE sqrt / division instantiation."""
    shapes = [(300, 130), (4097,), (127,), (64, 128), (5000, 1), (3, 3, 24, 24), (4096,), (9000,), (1000, 768)]
    kw = dict(qconfig=None, **hyper)
    torch.manual_seed(21)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i, zero_fraction=0.2) for i, sh in enumerate(shapes)], 7, kw,
        qmaps, "group")
    _check_adamw(opt, params, o_states, o_params, "group")


@pytest.mark.parametrize("hyper", [dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01),
                                   dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-30, weight_decay=0.1)])
def test_optimizer_rank1_config_many_matrices(qmaps, hyper):
    """default.yml on a list with several matrices whose rows are multiples of 8 (stepped together from
    the second step on: one table, three launches), next to shapes that stay on per-tensor launches (odd
    row length, 4-D, vectors): wide rows that span several statistics tiles, very narrow rows, rows that
    do not fill a 128-element unit, 20 % exact zeros."""
    shapes = [(1000, 768), (768, 3072), (130, 4104), (4097, 8), (333, 1024), (1024,), (3, 3, 64, 64), (70, 61),
              (5000, 16), (4100,)]
    kw = dict(qconfig="default.yml", **hyper)
    torch.manual_seed(31)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i, zero_fraction=0.2) for i, sh in enumerate(shapes)], 7, kw,
        qmaps, "rank1")
    _check_adamw(opt, params, o_states, o_params, "rank1")


def test_optimizer_factored_many_matrices(qmaps):
    """factor_second_moment=True on a list with several matrices (stepped together from the second step
    on: partial sums, reduction, row means and update in four launches), fp32 and 4-bit first moments,
    next to shapes that stay on per-tensor launches (odd row length, 4-D) and vectors.  Accumulators and
    parameters to 1e-6 relative (fixed summation order, not torch's); first-moment codes identical."""
    shapes = [(1000, 768), (768, 3072), (130, 4104), (40, 8), (333, 1024), (1024,), (2, 3, 32, 32), (70, 61),
              (5000, 16), (4100,), (64, 64)]
    kw = dict(qconfig=None, factor_second_moment=True, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(41)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i) for i, sh in enumerate(shapes)], 7, kw, qmaps, "group")
    _check_adamw(opt, params, o_states, o_params, "group", factored=True)


@pytest.mark.parametrize("cfg,v_scale", [(None, "group"), ("default.yml", "rank1")])
def test_a_parameter_that_skips_a_step_keeps_its_own_step_count(qmaps, cfg, v_scale):
    """One parameter has no gradient at the third step: afterwards its step counter (hence its bias
    corrections) lags behind the others.  The list step must not put it into a launch that assumes a
    common step count; results equal the restated reference stepping each tensor with its own counter."""
    import os
    import lpmm
    from lpmm.config import CONFIG_DIR
    from oracle import torch_ref as T
    from golden_cases import THRESHOLD
    shapes = [(96, 64), (64, 128), (130, 72), (200,)]
    hyper = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(51)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    params = [torch.nn.Parameter(p.clone()) for p in p0s]
    opt = lpmm.optim.AdamW(params, qconfig=os.path.join(CONFIG_DIR, cfg) if cfg else None, **hyper)
    qm, qv = torch.from_numpy(qmaps["m"]).to(device()), torch.from_numpy(qmaps["v"]).to(device())
    o_params = [p.clone() for p in p0s]
    o_states = [dict() for _ in shapes]
    counts = [0] * len(shapes)
    for s in range(1, 7):
        for i, p in enumerate(params):
            skip = (s == 3 and i == 1)
            p.grad = None if skip else student_t(p.shape, 40 * s + i)
        opt.step()
        for i, op in enumerate(o_params):
            if s == 3 and i == 1:
                continue
            counts[i] += 1
            quant = op.numel() > THRESHOLD
            T.adamw_step(op, student_t(op.shape, 40 * s + i), o_states[i], qm, qv, m_quant=quant, v_quant=quant,
                         v_scale_type=v_scale, beta1=0.9, beta2=0.999, lr=1e-3, weight_decay=0.01, eps=1e-8,
                         step=float(counts[i]))
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        assert float(opt.state[p]["step"]) == counts[i]
        assert bits_equal(p.detach(), o_params[i]), f"tensor {i}: parameters differ"
        if p.numel() > THRESHOLD:
            assert torch.equal(opt.state[p]["exp_avg"].view(torch.uint8), o_states[i]["m"].view(torch.uint8))
            assert torch.equal(opt.state[p]["exp_avg_sq"].view(torch.uint8), o_states[i]["v"].view(torch.uint8))


def _vp(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else None)


def test_entry_point_equals_per_tensor_calls_on_unaligned_views_and_ranges(qmaps):
    from lpmm import _kernels, _native as N
    qm = torch.from_numpy(qmaps["m"]).to(device())
    qv = torch.from_numpy(qmaps["v"]).to(device())
    sizes = [128 * 40 + 5, 4097, 128 * 64, 333, 100]
    kinds = [N.KIND_Q4, N.KIND_Q4, N.KIND_Q4, N.KIND_Q4, N.KIND_FP32]

    def build(seed):
        torch.manual_seed(seed)
        out, keep = [], []
        for i, n in enumerate(sizes):
            base = torch.randn(n + 3, device=device()) * 0.02
            gbase = torch.randn(n + 3, device=device()) * 1e-3
            off = 1 if i % 2 == 0 else 0  # odd float offset: not 32-byte aligned
            p, g = base[off:off + n], gbase[off:off + n]
            groups = (n + 127) // 128
            if kinds[i] == N.KIND_Q4:
                m = torch.randint(-128, 128, (_kernels.packed_len(groups * 128),), dtype=torch.int8, device=device())
                v = torch.randint(-128, 128, (_kernels.packed_len(groups * 128),), dtype=torch.int8, device=device())
                sm = torch.rand(groups, 1, device=device()) * 1e-3
                sv = torch.rand(groups, 1, device=device()) * 1e-6
            else:
                m, v, sm, sv = torch.randn(n, device=device()) * 1e-3, torch.rand(n, device=device()) * 1e-6, None, None
            out.append((p, g, m, v, sm, sv))
            keep += [base, gbase]
        return out, keep

    hyper = (0.9, 0.999, 1e-3, 0.01, 1e-8, 7.0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def multi(entries, lo=0, hi=-1):
        tl = _kernels.TensorList(entries)
        N.check(N.lib.lpmm_b200_adamw4bit_unfused_multi_tensor(tl.array, tl.n, _vp(qm), _vp(qv), *hyper, lo, hi, stream))
        return tl

    ea, _ka = build(9)
    ta = multi(ea)
    eb, _kb = build(9)
    total = ta.total_groups
    cuts = [0, total // 3 + 1, 2 * total // 3, total]
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        multi(eb, lo, hi)
    ec, _kc = build(9)
    for (p, g, m, v, sm, sv), kind in zip(ec, kinds):
        t = N.StepTensor()
        t.p, t.g, t.numel, t.ndim, t.first = p.data_ptr(), g.data_ptr(), p.numel(), 1, 0
        t.shape[0] = p.numel()
        mode = N.STATE_GROUP4 if kind == N.KIND_Q4 else N.STATE_FP32
        t.m_mode = t.v_mode = mode
        t.m, t.v = m.data_ptr(), v.data_ptr()
        if sm is not None:
            t.m_max1, t.v_max1 = sm.data_ptr(), sv.data_ptr()
        N.check(N.lib.lpmm_b200_adamw4bit_unfused_step(ctypes.byref(t), _vp(qm), _vp(qv), *hyper, None, 0, stream))
    torch.cuda.synchronize()
    for i, (a, b, c) in enumerate(zip(ea, eb, ec)):
        n = a[0].numel()
        nbytes = (n + 127) // 128 * 64
        for other, what in ((b, "group ranges"), (c, "per-tensor calls")):
            assert bits_equal(a[0], other[0]), f"tensor {i}: parameters vs {what}"
            if kinds[i] == N.KIND_Q4:
                assert torch.equal(a[2][:nbytes], other[2][:nbytes]), f"tensor {i}: first-moment codes vs {what}"
                assert torch.equal(a[3][:nbytes], other[3][:nbytes]), f"tensor {i}: second-moment codes vs {what}"
                assert bits_equal(a[4], other[4]) and bits_equal(a[5], other[5]), f"tensor {i}: scales vs {what}"
            else:
                assert bits_equal(a[2], other[2]) and bits_equal(a[3], other[3]), f"tensor {i}: fp32 moments vs {what}"


@pytest.mark.parametrize("kw", [dict(qconfig="default.yml"), dict(qconfig=None, factor_second_moment=True)],
                         ids=["rank1", "factored"])
def test_list_wide_steps_can_be_captured_into_a_cuda_graph(kw):
    """The list-wide rank-1 and factored steps upload nothing (their descriptors travel in the launch parameters), so
    a step captured into a CUDA graph and replayed once equals the same step launched directly, bit for bit, and
    the captured step took the list-wide kernels (a handful of graph nodes, not a chain per tensor)."""
    import os
    import lpmm
    from lpmm.config import CONFIG_DIR
    shapes = [(1024, 768), (768, 3072), (130, 4104), (333, 1024), (1024,), (5000, 16), (512, 512), (256, 1280)]
    kw = dict(kw, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    if isinstance(kw.get("qconfig"), str):
        kw["qconfig"] = os.path.join(CONFIG_DIR, kw["qconfig"])
    torch.manual_seed(51)
    init = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    pa = [torch.nn.Parameter(x.clone()) for x in init]
    pb = [torch.nn.Parameter(x.clone()) for x in init]
    oa, ob = lpmm.optim.AdamW(pa, **kw), lpmm.optim.AdamW(pb, **kw)
    for p in pa + pb:
        p.grad = torch.zeros_like(p)
    for s in range(1, 4):  # eager steps: states initialised, descriptors cached, scratch allocated
        for i, (a, b) in enumerate(zip(pa, pb)):
            g = student_t(shapes[i], 100003 * s + i)
            a.grad.copy_(g)
            b.grad.copy_(g)
        oa.step()
        ob.step()
    for i, (a, b) in enumerate(zip(pa, pb)):
        g = student_t(shapes[i], 100003 * 4 + i)
        a.grad.copy_(g)
        b.grad.copy_(g)
    torch.cuda.synchronize()
    oa.step()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ob.step()
    graph.replay()
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(zip(pa, pb)):
        assert bits_equal(a.detach(), b.detach()), f"tensor {i}: parameters"
        sa, sb = oa.state[a], ob.state[b]
        assert torch.equal(sa["exp_avg"].view(torch.uint8).view(-1), sb["exp_avg"].view(torch.uint8).view(-1)), f"tensor {i}"
        if "exp_avg_sq" in sa:
            assert torch.equal(sa["exp_avg_sq"].view(torch.uint8).view(-1), sb["exp_avg_sq"].view(torch.uint8).view(-1))
        else:
            assert bits_equal(sa["exp_avg_sq_row"], sb["exp_avg_sq_row"]) and bits_equal(sa["exp_avg_sq_col"], sb["exp_avg_sq_col"])


@pytest.mark.parametrize("kw,v_scale,factored", [(dict(qconfig="default.yml"), "rank1", False),
                                                 (dict(qconfig=None, factor_second_moment=True), "group", True)],
                         ids=["rank1", "factored"])
def test_lists_longer_than_one_descriptor_window(qmaps, kw, v_scale, factored):
    """300 matrices in one parameter group: more than the launch parameters hold descriptors for (268 rank-1 / 224
    factored), so the list is stepped in two windows; wide rows (multiples of 128) and narrow ones mixed, so that
    both update kernels run in both windows."""
    shapes = [((40, 128) if i % 3 else (136, 40)) for i in range(300)]
    kw = dict(kw, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(61)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i) for i, sh in enumerate(shapes)], 4, kw, qmaps, v_scale)
    _check_adamw(opt, params, o_states, o_params, v_scale, factored=factored)


WIDE_SHAPES = [(1000, 768), (768, 3072), (130, 4096), (4097, 8), (333, 1024), (1024,), (3, 3, 64, 64), (70, 61),
               (5000, 16), (4100,), (64, 128)]


@pytest.mark.parametrize("kw,v_scale,factored", [(dict(qconfig=None), "group", False),
                                                 (dict(qconfig="default.yml"), "rank1", False),
                                                 (dict(qconfig=None, factor_second_moment=True), "group", True)],
                         ids=["group", "rank1", "factored"])
def test_tolerance_mode_of_the_list_wide_kernels_against_the_oracle(qmaps, kw, v_scale, factored):
    """``exact_params=False`` on the non-fused step: the list-wide kernels take the approximate square root and
    reciprocal in the parameter update.  Moments do not depend on the parameters, so after 7 steps every code, scale,
    per-axis maximum and accumulator still equals the restated reference's exactly (the accumulators to their usual
    summation-order tolerance); the parameters stay within 1e-6 relative.  Matrices with rows that are multiples of
    128 (the wide update kernels) next to narrow and odd shapes (exact kernels)."""
    kw = dict(kw, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, exact_params=False)
    torch.manual_seed(71)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in WIDE_SHAPES]
    opt, params, o_states, o_params = _run_pair_adamw(
        WIDE_SHAPES, p0s, lambda s: [student_t(sh, s * 100003 + i, zero_fraction=0.2) for i, sh in enumerate(WIDE_SHAPES)],
        7, kw, qmaps, v_scale)
    _check_adamw(opt, params, o_states, o_params, v_scale, factored=factored, p_exact=False)
    for p, op in zip(params, o_params):  # element-wise too: a few ulps of the parameter or of the step taken
        err = (p.detach() - op).abs()
        assert bool((err <= 2e-6 * op.abs() + 5e-8).all())


@pytest.mark.parametrize("kw", [dict(qconfig=None), dict(qconfig="default.yml"),
                                dict(qconfig=None, factor_second_moment=True),
                                dict(qconfig="default.yml", fused=True, fused_rank1=True)],
                         ids=["group", "rank1", "factored", "fused_rank1"])
def test_tolerance_mode_of_the_list_wide_kernels_against_the_exact_mode(kw):
    """The same list stepped by two optimizers, one exact and one in tolerance mode: all state tensors bit-identical
    after 6 steps, parameters within 1e-6 relative, and not all parameters bit-identical (the flag reached the
    kernels)."""
    import os
    import lpmm
    from lpmm.config import CONFIG_DIR
    kw = dict(kw, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    if isinstance(kw.get("qconfig"), str):
        kw["qconfig"] = os.path.join(CONFIG_DIR, kw["qconfig"])
    torch.manual_seed(81)
    init = [torch.randn(s, device=device()) * 0.02 for s in WIDE_SHAPES]
    pa = [torch.nn.Parameter(x.clone()) for x in init]
    pb = [torch.nn.Parameter(x.clone()) for x in init]
    oa, ob = lpmm.optim.AdamW(pa, **kw), lpmm.optim.AdamW(pb, exact_params=False, **kw)
    for s in range(1, 7):
        for i, (a, b) in enumerate(zip(pa, pb)):
            g = student_t(WIDE_SHAPES[i], 100003 * s + i)
            a.grad, b.grad = g, g.clone()
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    differing = 0
    for i, (a, b) in enumerate(zip(pa, pb)):
        rel = ((a.detach() - b.detach()).norm() / a.detach().norm()).item()
        assert rel <= 1e-6, f"tensor {i}: {rel}"
        differing += int(not bits_equal(a.detach(), b.detach()))
        sa, sb = oa.state[a], ob.state[b]
        for key in ("exp_avg", "exp_avg_sq", "exp_avg_sq_row", "exp_avg_sq_col"):
            if key in sa and torch.is_tensor(sa[key]) and sa[key].numel():
                assert torch.equal(sa[key].reshape(-1).view(torch.uint8), sb[key].reshape(-1).view(torch.uint8)), f"tensor {i}: {key}"
        for q in ("exp_avg_qstate", "exp_avg_sq_qstate"):
            oh_a, oh_b = sa.get(q, {}).get("overhead", {}), sb.get(q, {}).get("overhead", {})
            if oh_a.get("max1") is not None:
                assert bits_equal(oh_a["max1"], oh_b["max1"]), f"tensor {i}: {q} scales"
            if oh_a.get("max_dims") is not None:
                for x, y in zip(oh_a["max_dims"], oh_b["max_dims"]):
                    assert bits_equal(x, y), f"tensor {i}: {q} per-axis maxima"
    assert differing > 0
