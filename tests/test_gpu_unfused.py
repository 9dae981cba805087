"""The optimizers of the Python surface (``lpmm.optim.AdamW`` non-fused and factored, ``lpmm.optim.SGD``)
on a B200 against the torch-op restatement of the reference's Python path run on the same GPU
(``oracle/torch_ref.py``, itself pinned to the reference's Python on CPU).  Codes, scales and
per-axis maxima must be bit-identical; parameters bit-identical except in the factored mode,
where row/column means are summed in a different (fixed) order: 1e-6 relative there."""
import os

import numpy as np
import pytest
import torch

from golden_cases import CASES, THRESHOLD, layout
from gpu_helpers import bits_equal, device, nibbles, student_t

pytestmark = pytest.mark.gpu


def _golden(golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"python_{name}.npz"))
    return {k: z[k] for k in z.files}


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device())


def _make_opt(kind, params, kw):
    import lpmm
    from lpmm.config import CONFIG_DIR
    kw = dict(kw)
    if isinstance(kw.get("qconfig"), str):
        kw["qconfig"] = os.path.join(CONFIG_DIR, kw["qconfig"])
    return getattr(lpmm.optim, kind)(params, **kw)


def _default_quant(i, numel):
    return numel > THRESHOLD, numel > THRESHOLD


def _run_pair_adamw(shapes, p0s, grads_of_step, steps, kw, qmaps, v_scale, maps=("m", "v"), m_gp=128, quant_of=None,
                    overrides=()):
    """Returns (optimizer, params, oracle states, oracle params).  ``quant_of(i, numel)`` -> (first moment
    quantized, second moment quantized) of tensor i (default: both iff numel > 4096); ``overrides``:
    (tensor index, enable) pairs passed to ``override_quantize_enable`` before the first step."""
    from oracle import torch_ref as T
    quant_of = quant_of or _default_quant
    qm, qv = _dev(qmaps[maps[0]]), _dev(qmaps[maps[1]])
    params = [torch.nn.Parameter(p.clone()) for p in p0s]
    opt = _make_opt("AdamW", params, kw)
    holder = torch.nn.Module()
    for i, enable in overrides:
        holder.register_parameter(f"p{i}", params[i])
        opt.override_quantize_enable(holder, f"p{i}", enable)
    o_params = [p.clone() for p in p0s]
    o_states = [dict() for _ in p0s]
    factored = kw.get("factor_second_moment", False)
    for i, sh in enumerate(shapes):
        if factored and len(sh) >= 2:
            o_states[i] = {"row": torch.zeros(sh[:-1], device=device()), "col": torch.zeros(sh[:-2] + sh[-1:], device=device())}
    b1, b2 = kw["betas"]
    for s in range(1, steps + 1):
        grads = grads_of_step(s)
        for p, g in zip(params, grads):
            p.grad = g.clone()
        opt.step()
        for i, (op, g) in enumerate(zip(o_params, grads)):
            mq, vq = quant_of(i, op.numel())
            common = dict(beta1=b1, beta2=b2, lr=kw["lr"], weight_decay=kw["weight_decay"], eps=kw["eps"], step=float(s))
            if factored and op.dim() >= 2:
                T.factored_step(op, g, o_states[i], qm, m_quant=mq, m_gp_sz=m_gp, **common)
            else:
                T.adamw_step(op, g, o_states[i], qm, qv, m_quant=mq, v_quant=vq, v_scale_type=v_scale,
                             m_gp_sz=m_gp, **common)
    torch.cuda.synchronize()
    return opt, params, o_states, o_params


def _check_group_state(mine_codes, mine_max1, o_codes, o_md, n, what, gp=128):
    groups = (n + gp - 1) // gp
    assert mine_codes.numel() == o_codes.numel(), f"{what}: packed length"
    assert torch.equal(mine_codes.view(torch.uint8), o_codes.view(torch.uint8)), f"{what}: codes (incl. padding) differ"
    assert bits_equal(mine_max1.reshape(-1), o_md["max1"].reshape(-1)), f"{what}: scales differ"
    assert mine_max1.numel() == groups


def _check_adamw(opt, params, o_states, o_params, v_scale, factored=False, p_exact=True, m_gp=128, quant_of=None,
                 acc_tol=1e-6):
    """``acc_tol``: relative tolerance (of the largest entry) on the factored row / column accumulators, whose sums
    are taken in another order than torch's."""
    quant_of = quant_of or _default_quant
    for i, p in enumerate(params):
        st, os_, op = opt.state[p], o_states[i], o_params[i]
        quant, v_quant = quant_of(i, p.numel())
        fac = factored and p.dim() >= 2
        if fac or not p_exact:
            rel = ((p.detach() - op).norm() / op.norm()).item()
            assert rel <= 1e-6, f"tensor {i}: params rel err {rel}"
        else:
            assert bits_equal(p.detach(), op), f"tensor {i}: params differ"
        if quant:
            _check_group_state(st["exp_avg"], st["exp_avg_qstate"]["overhead"]["max1"], os_["m"], os_["m_md"], p.numel(),
                               f"tensor {i} exp_avg", m_gp)
        else:
            assert bits_equal(st["exp_avg"], os_["m"]), f"tensor {i}: fp32 exp_avg differs"
        if fac:
            for mine, orc in ((st["exp_avg_sq_row"], os_["row"]), (st["exp_avg_sq_col"], os_["col"])):
                rel = ((mine - orc).abs().max() / orc.abs().max()).item()
                assert rel <= acc_tol, f"tensor {i}: accumulator rel err {rel}"
            continue
        if not v_quant:
            assert bits_equal(st["exp_avg_sq"], os_["v"]), f"tensor {i}: fp32 exp_avg_sq differs"
        elif v_scale == "rank1" and p.dim() >= 2:
            oh = st["exp_avg_sq_qstate"]["overhead"]
            assert st["exp_avg_sq"].numel() == os_["v"].numel()
            assert torch.equal(st["exp_avg_sq"].view(torch.uint8), os_["v"].view(torch.uint8)), f"tensor {i}: v codes"
            for d in range(p.dim()):
                assert oh["max_dims"][d].shape == os_["v_md"]["max_dims"][d].shape
                assert bits_equal(oh["max_dims"][d], os_["v_md"]["max_dims"][d]), f"tensor {i}: axis {d} maxima"
        else:
            _check_group_state(st["exp_avg_sq"], st["exp_avg_sq_qstate"]["overhead"]["max1"], os_["v"], os_["v_md"],
                               p.numel(), f"tensor {i} exp_avg_sq")


def _codes(t, n, bits):
    """The first n codes of a packed tensor as uint8."""
    return nibbles(t, n) if bits == 4 else t.view(torch.uint8)[:n]


@pytest.mark.parametrize("name", ["adamw_rank1", "adamw_group", "adamw_rank1_ragged", "adamw_8bit", "adamw_5bit",
                                  "adamw_m_group_512", "adamw_m_group_4096"])
def test_adamw_unfused_on_golden_inputs(golden_dir, qmaps, name):
    G = _golden(golden_dir, name)
    _, kw, shapes = CASES[name]
    L = layout(name)
    v_scale = L["v_scale"]
    steps = int(G["steps"])
    p0s = [_dev(G[f"p0.{i}"]) for i in range(len(shapes))]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [_dev(G[f"g{s}.{i}"]) for i in range(len(shapes))], steps, kw, qmaps, v_scale,
        maps=L["maps"], m_gp=L["m_gp"])
    _check_adamw(opt, params, o_states, o_params, v_scale, m_gp=L["m_gp"])
    # and against what the reference's Python produced on CPU: same codes up to fp ties, same params to 1e-6
    for i, p in enumerate(params):
        ref_p = _dev(G[f"p.{i}"])
        assert ((p.detach() - ref_p).norm() / ref_p.norm()).item() <= 1e-6
        if p.numel() > THRESHOLD:
            n = p.numel()
            assert opt.state[p]["exp_avg"].numel() == G[f"s.{i}.exp_avg"].size, "packed length differs from the CPU run"
            mism = (_codes(opt.state[p]["exp_avg"], n, L["bits"])
                    != _codes(_dev(G[f"s.{i}.exp_avg"]), n, L["bits"])).float().mean().item()
            # wider maps have closer midpoints, so the last-bit differences between CPU and GPU torch ops
            # flip proportionally more codes
            assert mism <= (1e-3 if L["bits"] == 4 else 2e-2), f"tensor {i}: {mism} of first-moment codes differ from the CPU run"


def test_adamw_unfused_larger_ragged_shapes(qmaps):
    """The ragged shape list of the tail/fallback configuration: conv weights, matrices whose sizes
    are not multiples of 128, vectors around the 4096 threshold, a column vector; 20 % exact zeros."""
    from lpmm.config import CONFIG_DIR  # noqa: F401
    shapes = [(3, 3, 64, 64), (1000, 768), (768, 3072), (4097,), (127,), (4096,), (50000, 1)]
    kw = dict(qconfig="default.yml", lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(0)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i, zero_fraction=0.2) for i, sh in enumerate(shapes)], 6, kw,
        qmaps, "rank1")
    _check_adamw(opt, params, o_states, o_params, "rank1")


@pytest.mark.parametrize("cfg,bits,m_gp", [("default_8b.yml", 8, 128), ("default_6b.yml", 6, 128),
                                           ("default_7b.yml", 7, 128), ("1st_moment_group_256.yml", 4, 256),
                                           ("1st_moment_group_1024.yml", 4, 1024),
                                           ("1st_moment_group_2048.yml", 4, 2048),
                                           ("1st_moment_group_4096.yml", 4, 4096)])
def test_adamw_wider_codes_and_larger_groups_ragged_shapes(qmaps, golden_dir, cfg, bits, m_gp):
    """Every remaining configuration file on ragged shapes (group padding that crosses a 2048-row,
    tensors shorter than one group, a column vector), 20 % exact zeros where the format allows
    it: with one code per byte an all-zero group becomes NaN in the reference (its 0/0 is stored
    as 255, which the unpack kernel reads past the end of a map of fewer than 256 entries), so those
    cases use dense gradients."""
    shapes = [(3, 3, 64, 64), (1000, 768), (4097,), (6000,), (4096,), (50000, 1), (777, 13)]
    kw = dict(qconfig=cfg, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    maps = ("m", "v") if bits == 4 else (f"nonlinear_{bits}", f"power1_{bits}")
    if bits not in (4,) and maps[0] not in qmaps:
        pytest.skip("map fixture missing")
    torch.manual_seed(5)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    zf = 0.2 if bits == 4 else 0.0
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i, zero_fraction=zf) for i, sh in enumerate(shapes)], 5, kw,
        qmaps, "rank1", maps=maps, m_gp=m_gp)
    _check_adamw(opt, params, o_states, o_params, "rank1", m_gp=m_gp)


def test_adamw_group_config_matrix(qmaps):
    shapes = [(4096, 512), (333, 77)]
    kw = dict(qconfig=None, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(1)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i) for i, sh in enumerate(shapes)], 5, kw, qmaps, "group")
    _check_adamw(opt, params, o_states, o_params, "group")


def test_adamw_factored_on_golden_inputs(golden_dir, qmaps):
    G = _golden(golden_dir, "adamw_factored")
    _, kw, shapes = CASES["adamw_factored"]
    steps = int(G["steps"])
    p0s = [_dev(G[f"p0.{i}"]) for i in range(len(shapes))]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [_dev(G[f"g{s}.{i}"]) for i in range(len(shapes))], steps, kw, qmaps, "group")
    _check_adamw(opt, params, o_states, o_params, "group", factored=True)


def test_adamw_factored_gpt2_like_shapes(qmaps):
    shapes = [(5025, 1024), (1024, 3072), (1024,)]
    kw = dict(qconfig=None, factor_second_moment=True, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(2)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    opt, params, o_states, o_params = _run_pair_adamw(
        shapes, p0s, lambda s: [student_t(sh, s * 100003 + i) for i, sh in enumerate(shapes)], 4, kw, qmaps, "group")
    _check_adamw(opt, params, o_states, o_params, "group", factored=True)


@pytest.mark.parametrize("name", ["sgd_momentum", "sgd_nesterov", "sgd_8bit", "sgd_group_1024"])
def test_sgd_on_golden_inputs(golden_dir, qmaps, name):
    from oracle import torch_ref as T
    G = _golden(golden_dir, name)
    _, kw, shapes = CASES[name]
    L = layout(name)
    steps = int(G["steps"])
    qm = _dev(qmaps[L["maps"][0]])
    params = [torch.nn.Parameter(_dev(G[f"p0.{i}"])) for i in range(len(shapes))]
    opt = _make_opt("SGD", params, kw)
    o_params = [_dev(G[f"p0.{i}"]) for i in range(len(shapes))]
    o_states = [dict() for _ in shapes]
    for s in range(1, steps + 1):
        for i, p in enumerate(params):
            g = _dev(G[f"g{s}.{i}"])
            p.grad = g.clone()
            T.sgd_step(o_params[i], g, o_states[i], qm, quant=p.numel() > THRESHOLD, weight_decay=kw["weight_decay"],
                       momentum=kw["momentum"], lr=kw["lr"], dampening=kw.get("dampening", 0),
                       nesterov=kw.get("nesterov", False), maximize=False, gp_sz=L["m_gp"])
        opt.step()
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        assert bits_equal(p.detach(), o_params[i]), f"tensor {i}: params differ"
        st = opt.state[p]
        if p.numel() > THRESHOLD:
            _check_group_state(st["momentum_buffer"], st["momentum_buffer_qstate"]["overhead"]["max1"], o_states[i]["buf"],
                               o_states[i]["buf_md"], p.numel(), f"tensor {i} buffer", L["m_gp"])
        else:
            assert bits_equal(st["momentum_buffer"], o_states[i]["buf"])
        ref_p = _dev(G[f"p.{i}"])
        assert ((p.detach() - ref_p).norm() / ref_p.norm()).item() <= 1e-6


def test_state_dict_round_trip_keeps_codes_and_continues(qmaps):
    """state_dict -> load_state_dict into a fresh optimizer, then one more step on both: identical."""
    import lpmm
    from lpmm.config import CONFIG_DIR
    shapes = [(96, 64), (5000,), (100,)]
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, qconfig=os.path.join(CONFIG_DIR, "default.yml"))
    torch.manual_seed(3)
    pa = [torch.nn.Parameter(torch.randn(s, device=device()) * 0.02) for s in shapes]
    oa = lpmm.optim.AdamW(pa, **kw)
    for s in range(1, 4):
        for i, p in enumerate(pa):
            p.grad = student_t(p.shape, 900 + 10 * s + i)
        oa.step()
    sd = oa.state_dict()
    assert "qconfig" in sd
    assert sd["state"][0]["exp_avg"].dtype == torch.int8
    pb = [torch.nn.Parameter(p.detach().clone()) for p in pa]
    ob = lpmm.optim.AdamW(pb, **kw)
    ob.load_state_dict(sd)
    assert ob.state[pb[0]]["exp_avg"].dtype == torch.int8
    for i, (a, b) in enumerate(zip(pa, pb)):
        g = student_t(a.shape, 990 + i)
        a.grad, b.grad = g.clone(), g.clone()
    oa.step()
    ob.step()
    torch.cuda.synchronize()
    for a, b in zip(pa, pb):
        assert bits_equal(a.detach(), b.detach())
        assert torch.equal(oa.state[a]["exp_avg"], ob.state[b]["exp_avg"])


@pytest.mark.parametrize("cfg,v_scale", [(None, "group"), ("default.yml", "rank1")])
def test_fp32_moment_met_by_a_quantizing_step_is_quantised_in_place(qmaps, cfg, v_scale):
    """A checkpoint saved with a tensor's moments in fp32 (its quantization was overridden off) and loaded into an
    optimizer that quantizes that tensor: the initialised fp32 states are quantised as they are on the first step --
    never replaced by fresh storage that would then be read as the previous moment.  Oracle: the fp32 moments
    quantised with the restated reference quantizer, then one more restated step."""
    import lpmm
    from oracle import torch_ref as T
    shape = (96, 64)  # 6144 elements
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    qm, qv = _dev(qmaps["m"]), _dev(qmaps["v"])
    torch.manual_seed(12)
    p0 = torch.randn(shape, device=device()) * 0.02
    p = torch.nn.Parameter(p0.clone())
    opt = _make_opt("AdamW", [p], dict(kw, qconfig=cfg))
    holder = torch.nn.Module()
    holder.register_parameter("w", p)
    opt.override_quantize_enable(holder, "w", False)
    op, st = p0.clone(), {}
    common = dict(beta1=0.9, beta2=0.999, lr=1e-3, weight_decay=0.01, eps=1e-8)
    for s in (1, 2):
        g = student_t(shape, 700 + s)
        p.grad = g.clone()
        opt.step()
        T.adamw_step(op, g, st, qm, qv, m_quant=False, v_quant=False, v_scale_type=v_scale, step=float(s), **common)
    assert opt.state[p]["exp_avg"].dtype == torch.float32 and bits_equal(opt.state[p]["exp_avg"], st["m"])
    p2 = torch.nn.Parameter(p.detach().clone())
    opt2 = _make_opt("AdamW", [p2], dict(kw, qconfig=cfg))   # no override: both moments are to be 4-bit
    opt2.load_state_dict(opt.state_dict())
    assert opt2.state[p2]["exp_avg"].dtype == torch.float32
    st["m"], st["m_md"] = T.vectorwise_quant(st["m"], qm, "group")
    st["v"], st["v_md"] = T.vectorwise_quant(st["v"], qv, v_scale)
    g = student_t(shape, 703)
    p2.grad = g.clone()
    opt2.step()
    T.adamw_step(op, g, st, qm, qv, m_quant=True, v_quant=True, v_scale_type=v_scale, step=3.0, **common)
    torch.cuda.synchronize()
    s2 = opt2.state[p2]
    assert s2["exp_avg"].dtype == torch.int8 and s2["exp_avg_sq"].dtype == torch.int8
    assert bits_equal(p2.detach(), op)
    _check_group_state(s2["exp_avg"], s2["exp_avg_qstate"]["overhead"]["max1"], st["m"], st["m_md"], p2.numel(), "exp_avg")
    if v_scale == "group":
        _check_group_state(s2["exp_avg_sq"], s2["exp_avg_sq_qstate"]["overhead"]["max1"], st["v"], st["v_md"], p2.numel(),
                           "exp_avg_sq")
    else:
        assert torch.equal(s2["exp_avg_sq"].view(torch.uint8), st["v"].view(torch.uint8))
        for d in range(2):
            assert bits_equal(s2["exp_avg_sq_qstate"]["overhead"]["max_dims"][d], st["v_md"]["max_dims"][d])
