"""Checkpoint interoperability: an optimizer ``state_dict`` in the reference's layout -- here rebuilt
from the golden vectors its own Python produced on CPU (packed codes, ``max1`` / ``max_dims``,
``scaled_shape``, ``dtype``, ``stride``, fp32 states, CPU ``step``) -- is loaded into this package's
``lpmm.optim.AdamW`` on a B200 and stepped once more; the result must equal the torch-op
restatement continuing from the same state on the same GPU, bit for bit."""
import os

import numpy as np
import pytest
import torch

from golden_cases import CASES, THRESHOLD, layout
from gpu_helpers import bits_equal, device, student_t

pytestmark = pytest.mark.gpu


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


@pytest.mark.parametrize("name", ["adamw_rank1", "adamw_group", "adamw_8bit", "adamw_5bit", "adamw_m_group_512",
                                  "adamw_m_group_4096"])
def test_reference_layout_state_dict_loads_and_continues(golden_dir, qmaps, name):
    import lpmm
    from lpmm.config import CONFIG_DIR, get_config
    from oracle import torch_ref as T
    z = np.load(os.path.join(golden_dir, f"python_{name}.npz"))
    G = {k: z[k] for k in z.files}
    _, kw, shapes = CASES[name]
    L = layout(name)
    rank1 = L["v_scale"] == "rank1"
    cfg_path = os.path.join(CONFIG_DIR, kw["qconfig"]) if kw["qconfig"] else None
    steps = int(G["steps"])
    qm_cpu, qv_cpu = _t(qmaps[L["maps"][0]]), _t(qmaps[L["maps"][1]])

    # ---- a state_dict as the reference writes it (CPU tensors, as torch.save / torch.load would give)
    state, o_states = {}, []
    for i, shape in enumerate(shapes):
        n = int(np.prod(shape))
        quant = n > THRESHOLD
        st = {"step": torch.tensor(float(steps))}
        o = {}
        for key, qmap, nm in (("exp_avg", qm_cpu, "m"), ("exp_avg_sq", qv_cpu, "v")):
            st[key] = _t(G[f"s.{i}.{key}"]).clone()
            oh = {}
            if quant:
                pre = f"s.{i}.{key}_qstate.overhead"
                oh = {"dtype": torch.float32, "stride": torch.empty(shape).stride(),
                      "scaled_shape": torch.Size(G[f"{pre}.scaled_shape"].tolist())}
                if f"{pre}.max1" in G:
                    oh["max1"] = _t(G[f"{pre}.max1"]).clone()
                else:
                    oh.update(max1=None, dim=len(shape),
                              max_dims=[_t(G[f"{pre}.max_dims.{d}"]).clone() for d in range(len(shape))])
                if f"{pre}.dim" in G:
                    oh["dim"] = int(G[f"{pre}.dim"])
                st[key][-1] = 0  # the reference leaves the trailing byte unwritten
            st[f"{key}_qstate"] = {"enable": quant, "overhead": oh, "qmap": qmap.clone()}
            o[nm] = st[key].clone().to(device())
            if quant:
                o[f"{nm}_md"] = {k: ([x.to(device()) for x in v] if isinstance(v, list) else
                                     (v.to(device()) if isinstance(v, torch.Tensor) else v)) for k, v in oh.items()}
        state[i] = st
        o_states.append(o)
    sd = {"state": state, "qconfig": get_config(cfg_path),
          "param_groups": [dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, fused=False, use_first_moment=True,
                                factor_second_moment=False, params=list(range(len(shapes))))]}

    params = [torch.nn.Parameter(_t(G[f"p.{i}"]).to(device())) for i in range(len(shapes))]
    opt = lpmm.optim.AdamW(params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, qconfig=cfg_path)
    opt.load_state_dict(sd)
    assert opt.state[params[0]]["exp_avg"].dtype == torch.int8 and opt.state[params[0]]["exp_avg"].is_cuda
    assert opt.state[params[0]]["step"].device.type == "cpu"

    qm, qv = qm_cpu.to(device()), qv_cpu.to(device())
    o_params = [p.detach().clone() for p in params]
    grads = [student_t(s, 31337 + i) for i, s in enumerate(shapes)]
    for p, g in zip(params, grads):
        p.grad = g.clone()
    opt.step()
    for i, (op, g) in enumerate(zip(o_params, grads)):
        quant = op.numel() > THRESHOLD
        T.adamw_step(op, g, o_states[i], qm, qv, m_quant=quant, v_quant=quant, v_scale_type="rank1" if rank1 else "group",
                     beta1=0.9, beta2=0.999, lr=1e-3, weight_decay=0.01, eps=1e-8, step=float(steps + 1),
                     m_gp_sz=L["m_gp"])
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        assert bits_equal(p.detach(), o_params[i]), f"tensor {i}: params differ after the resumed step"
        st = opt.state[p]
        assert float(st["step"]) == steps + 1
        if p.numel() > THRESHOLD:
            assert torch.equal(st["exp_avg"].view(torch.uint8), o_states[i]["m"].view(torch.uint8))
            assert torch.equal(st["exp_avg_sq"].view(torch.uint8), o_states[i]["v"].view(torch.uint8))
        else:
            assert bits_equal(st["exp_avg"], o_states[i]["m"]) and bits_equal(st["exp_avg_sq"], o_states[i]["v"])
