"""The torch-op restatement (oracle/torch_ref.py) against golden vectors produced by the
reference's own Python on CPU: bit-exact parameters, codes, scales and accumulators."""
import os

import numpy as np
import pytest
import torch

from golden_cases import CASES, OVERRIDES, THRESHOLD, layout
from oracle import torch_ref as T


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"python_{name}.npz"))
    return {k: z[k] for k in z.files}


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def _same_codes(a, b, numel_codes):
    a = np.asarray(a).view(np.uint8)[:numel_codes]
    b = np.asarray(b).view(np.uint8)[:numel_codes]
    return np.array_equal(a, b)


def quant_flags(name, i, numel):
    """(first moment quantized, second moment quantized) of tensor i of a golden case: the threshold rule
    (reference optimizer.py:156-163), M.ENABLE False in the 2nd_moment_only configurations, and the case's
    override_quantize_enable calls (reference adamw.py:143-144)."""
    over = dict(OVERRIDES.get(name, []))
    if i in over:
        return over[i], over[i]
    big = numel > THRESHOLD
    cfg = CASES[name][1].get("qconfig")
    m_enabled = not (isinstance(cfg, str) and cfg.startswith("2nd_moment_only"))
    return big and m_enabled, big


@pytest.mark.parametrize("name", ["adamw_rank1", "adamw_group", "adamw_rank1_ragged", "adamw_8bit", "adamw_5bit",
                                  "adamw_m_group_512", "adamw_m_group_4096", "adamw_2nd_only_rank1",
                                  "adamw_2nd_only_group", "adamw_override"])
def test_adamw_unfused_matches_reference_python(golden_dir, qmaps, name):
    G = _load(golden_dir, name)
    _, kw, shapes = CASES[name]
    L = layout(name)
    v_scale = L["v_scale"]
    qm, qv = _t(qmaps[L["maps"][0]]), _t(qmaps[L["maps"][1]])
    steps = int(G["steps"])
    for i, shape in enumerate(shapes):
        p = _t(G[f"p0.{i}"]).clone()
        quant, v_quant = quant_flags(name, i, p.numel())
        st = {}
        for s in range(1, steps + 1):
            T.adamw_step(p, _t(G[f"g{s}.{i}"]), st, qm, qv, m_quant=quant, v_quant=v_quant, v_scale_type=v_scale,
                         beta1=0.9, beta2=0.999, lr=1e-3, weight_decay=0.01, eps=1e-8, step=float(s),
                         m_gp_sz=L["m_gp"])
        assert np.array_equal(p.numpy(), G[f"p.{i}"]), f"params of tensor {i}"
        if quant:
            # last byte is not written by the reference
            assert st["m"].numel() == G[f"s.{i}.exp_avg"].size
            assert _same_codes(st["m"].numpy(), G[f"s.{i}.exp_avg"], G[f"s.{i}.exp_avg"].size - 1)
            assert np.array_equal(st["m_md"]["max1"].numpy(), G[f"s.{i}.exp_avg_qstate.overhead.max1"])
        else:
            assert np.array_equal(st["m"].numpy(), G[f"s.{i}.exp_avg"])
        if v_quant:
            assert st["v"].numel() == G[f"s.{i}.exp_avg_sq"].size
            assert _same_codes(st["v"].numpy(), G[f"s.{i}.exp_avg_sq"], G[f"s.{i}.exp_avg_sq"].size - 1)
            if v_scale == "rank1" and len(shape) > 1:
                for d in range(len(shape)):
                    assert np.array_equal(st["v_md"]["max_dims"][d].numpy(),
                                          G[f"s.{i}.exp_avg_sq_qstate.overhead.max_dims.{d}"])
            else:
                assert np.array_equal(st["v_md"]["max1"].numpy(), G[f"s.{i}.exp_avg_sq_qstate.overhead.max1"])
        else:
            assert np.array_equal(st["v"].numpy(), G[f"s.{i}.exp_avg_sq"])


def test_adamw_factored_matches_reference_python(golden_dir, qmaps):
    G = _load(golden_dir, "adamw_factored")
    _, kw, shapes = CASES["adamw_factored"]
    qm, qv = _t(qmaps["m"]), _t(qmaps["v"])
    steps = int(G["steps"])
    for i, shape in enumerate(shapes):
        p = _t(G[f"p0.{i}"]).clone()
        quant = p.numel() > THRESHOLD
        if len(shape) >= 2:
            st = {"row": torch.zeros(shape[:-1]), "col": torch.zeros(shape[:-2] + shape[-1:])}
            for s in range(1, steps + 1):
                T.factored_step(p, _t(G[f"g{s}.{i}"]), st, qm, m_quant=quant, beta1=0.9, beta2=0.999, lr=1e-3,
                                weight_decay=0.01, eps=1e-8, step=float(s))
            assert np.array_equal(st["row"].numpy(), G[f"s.{i}.exp_avg_sq_row"])
            assert np.array_equal(st["col"].numpy(), G[f"s.{i}.exp_avg_sq_col"])
        else:
            st = {}
            for s in range(1, steps + 1):
                T.adamw_step(p, _t(G[f"g{s}.{i}"]), st, qm, qv, m_quant=quant, v_quant=quant, v_scale_type="group",
                             beta1=0.9, beta2=0.999, lr=1e-3, weight_decay=0.01, eps=1e-8, step=float(s))
        assert np.array_equal(p.numpy(), G[f"p.{i}"]), f"params of tensor {i}"
        if quant:
            assert _same_codes(st["m"].numpy(), G[f"s.{i}.exp_avg"], G[f"s.{i}.exp_avg"].size - 1)
        else:
            assert np.array_equal(st["m"].numpy(), G[f"s.{i}.exp_avg"])


@pytest.mark.parametrize("name", ["sgd_momentum", "sgd_nesterov", "sgd_8bit", "sgd_group_1024"])
def test_sgd_matches_reference_python(golden_dir, qmaps, name):
    G = _load(golden_dir, name)
    _, kw, shapes = CASES[name]
    L = layout(name)
    qm = _t(qmaps[L["maps"][0]])
    steps = int(G["steps"])
    for i, shape in enumerate(shapes):
        p = _t(G[f"p0.{i}"]).clone()
        quant = p.numel() > THRESHOLD
        st = {}
        for s in range(1, steps + 1):
            T.sgd_step(p, _t(G[f"g{s}.{i}"]), st, qm, quant=quant, weight_decay=kw["weight_decay"],
                       momentum=kw["momentum"], lr=kw["lr"], dampening=kw.get("dampening", 0),
                       nesterov=kw.get("nesterov", False), maximize=False, gp_sz=L["m_gp"])
        assert np.array_equal(p.numpy(), G[f"p.{i}"])
        if quant:
            assert _same_codes(st["buf"].numpy(), G[f"s.{i}.momentum_buffer"], G[f"s.{i}.momentum_buffer"].size - 1)
            assert np.array_equal(st["buf_md"]["max1"].numpy(), G[f"s.{i}.momentum_buffer_qstate.overhead.max1"])
        else:
            assert np.array_equal(st["buf"].numpy(), G[f"s.{i}.momentum_buffer"])
