"""Stochastic rounding ('real-sr') on a B200 against the reference's own compiled pack kernel
(``oracle/_ref``): with torch's default CUDA generator in the same state, the packed codes are identical
bit for bit, the generator ends at the same offset, and optimizers configured with stochastic rounding
reproduce the torch-op restatement of the reference's step that packs with the reference's kernel.
Skipped where the reference extension was not built."""
import os

import pytest
import torch

from golden_cases import THRESHOLD
from gpu_helpers import bits_equal, device, device_map, load_reference_extension, student_t

pytestmark = pytest.mark.gpu


def _ref():
    ref = load_reference_extension("quantization")
    if ref is None:
        pytest.skip("the reference's quantization extension (oracle/_ref) is not built")
    return ref


def _gen():
    return torch.cuda.default_generators[device().index or 0]


@pytest.mark.parametrize("bits,name", [(4, "m"), (4, "v"), (8, "nonlinear_8"), (5, "power1_5")])
def test_stochastic_pack_equals_reference_kernel(qmaps, bits, name):
    from lpmm.cpp_extension import quantization as mine
    ref = _ref()
    qmap = device_map(qmaps, name)
    lo, hi = float(qmap[0]), float(qmap[-1])
    torch.manual_seed(5)
    x = (torch.rand(7, 2048, device=device()) * (hi - lo) * 1.1 + lo - 0.05 * (hi - lo)).contiguous()
    x[0, :16] = qmap[:16]  # exact map values
    x[1, :5] = torch.tensor([0.0, -0.0, 1.0, 2.0, -2.0], device=device())
    torch.manual_seed(1234)
    r = ref.pack_nonlinear(x, qmap, bits, True)
    torch.cuda.synchronize()
    r_off = _gen().get_offset()
    torch.manual_seed(1234)
    m = mine.pack_nonlinear(x, qmap, bits, True)
    torch.cuda.synchronize()
    assert _gen().get_offset() == r_off, "the generator must end where the reference leaves it"
    assert torch.equal(m[:-1], r[:-1]), "stochastic codes differ from the reference's kernel"
    # a second call continues the stream
    r2 = ref.pack_nonlinear(x, qmap, bits, True)
    torch.manual_seed(1234)
    mine.pack_nonlinear(x, qmap, bits, True)
    m2 = mine.pack_nonlinear(x, qmap, bits, True)
    torch.cuda.synchronize()
    assert torch.equal(m2[:-1], r2[:-1]) and not torch.equal(m2[:-1], m[:-1])


@pytest.mark.parametrize("shape", [(4097,), (300, 130), (3, 3, 24, 24), (9000,)])
@pytest.mark.parametrize("scale_type,which,gp_sz", [("group", "m", 128), ("rank1", "v", 128), ("group", "m", 512)])
def test_vectorwise_quant_real_sr_equals_restated_reference(qmaps, shape, scale_type, which, gp_sz):
    import lpmm.functional as F
    from oracle import torch_ref as T
    ref = _ref()
    qmap = device_map(qmaps, which)
    x = student_t(shape, 91)
    if which == "v":
        x = x * x
    kw = dict(b=4, quant_type="nonlinear" if which == "m" else "power-1", round_type="real-sr", gp_sz=gp_sz,
              signed=(which == "m"), scale_type=scale_type)
    torch.manual_seed(77)
    codes, md = F.vectorwise_quant(x, qmap=qmap, shape=x.shape, **kw)
    torch.cuda.synchronize()
    off = _gen().get_offset()
    torch.manual_seed(77)
    o_codes, o_md = T.vectorwise_quant(x, qmap, scale_type, gp_sz, ref.pack_nonlinear, True)
    torch.cuda.synchronize()
    assert _gen().get_offset() == off
    assert codes.numel() == o_codes.numel()
    assert torch.equal(codes.view(torch.uint8), o_codes.view(torch.uint8)), "stochastic codes differ"
    if "max1" in o_md and o_md["max1"] is not None:
        assert bits_equal(md["max1"], o_md["max1"])


def _sr_config(tmp_path, m_round, v_round, v_scale):
    path = os.path.join(tmp_path, "sr.yml")
    with open(path, "w") as f:
        f.write(f"""QUANT:
  M: {{ENABLE: true, BITS: 4, GROUP_SIZE: 128, SCALE_TYPE: {{DEFAULT: group}}, QUANT_TYPE: {{DEFAULT: nonlinear}}, ROUND_TYPE: {m_round}}}
  SQM: {{ENABLE: true, BITS: 4, GROUP_SIZE: 128, SCALE_TYPE: {{DEFAULT: {v_scale}}}, QUANT_TYPE: {{DEFAULT: power-1}}, ROUND_TYPE: {v_round}}}
""")
    return path


@pytest.mark.parametrize("m_round,v_round,v_scale", [("real-sr", "real-sr", "rank1"), ("real-sr", "real-nearest", "group"),
                                                     ("real-nearest", "real-sr", "rank1")])
def test_adamw_with_stochastic_rounding_follows_the_reference_stream(qmaps, tmp_path, m_round, v_round, v_scale):
    """Three steps of AdamW with 'real-sr' states: parameters, codes and scales equal the restated reference
    whose packing is done by the reference's kernel, both starting from the same generator state (a
    nearest-rounded state advances the generator as well, as in the reference)."""
    import lpmm
    from oracle import torch_ref as T
    ref = _ref()
    qm, qv = device_map(qmaps, "m"), device_map(qmaps, "v")
    shapes = [(72, 64), (4097,), (100,), (3, 3, 24, 24)]
    hyper = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    torch.manual_seed(3)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    grads = [[student_t(s, 500 * k + i) for i, s in enumerate(shapes)] for k in range(3)]

    params = [torch.nn.Parameter(p.clone()) for p in p0s]
    opt = lpmm.optim.AdamW(params, qconfig=_sr_config(str(tmp_path), m_round, v_round, v_scale), **hyper)
    torch.manual_seed(2024)
    for k in range(3):
        for p, g in zip(params, grads[k]):
            p.grad = g.clone()
        opt.step()
    torch.cuda.synchronize()
    end = _gen().get_offset()

    o_params = [p.clone() for p in p0s]
    o_states = [dict() for _ in shapes]
    torch.manual_seed(2024)
    for k in range(3):
        for i, op in enumerate(o_params):
            quant = op.numel() > THRESHOLD
            T.adamw_step(op, grads[k][i], o_states[i], qm, qv, m_quant=quant, v_quant=quant, v_scale_type=v_scale,
                         beta1=0.9, beta2=0.999, lr=1e-3, weight_decay=0.01, eps=1e-8, step=float(k + 1),
                         ref_pack=ref.pack_nonlinear, m_stochastic=m_round == "real-sr", v_stochastic=v_round == "real-sr")
    torch.cuda.synchronize()
    assert _gen().get_offset() == end
    for i, p in enumerate(params):
        assert bits_equal(p.detach(), o_params[i]), f"tensor {i}: parameters differ"
        st = opt.state[p]
        if p.numel() > THRESHOLD:
            assert torch.equal(st["exp_avg"].view(torch.uint8), o_states[i]["m"].view(torch.uint8)), f"tensor {i}: m codes"
            assert torch.equal(st["exp_avg_sq"].view(torch.uint8), o_states[i]["v"].view(torch.uint8)), f"tensor {i}: v codes"
            assert bits_equal(st["exp_avg_qstate"]["overhead"]["max1"], o_states[i]["m_md"]["max1"])
        else:
            assert bits_equal(st["exp_avg"], o_states[i]["m"]) and bits_equal(st["exp_avg_sq"], o_states[i]["v"])


def test_sgd_with_stochastic_rounding_follows_the_reference_stream(qmaps, tmp_path):
    import lpmm
    from oracle import torch_ref as T
    ref = _ref()
    qm = device_map(qmaps, "m")
    shapes = [(72, 64), (4097,), (100,)]
    kw = dict(lr=1e-2, momentum=0.9, weight_decay=1e-4)
    torch.manual_seed(4)
    p0s = [torch.randn(s, device=device()) * 0.02 for s in shapes]
    grads = [[student_t(s, 700 * k + i) for i, s in enumerate(shapes)] for k in range(3)]
    params = [torch.nn.Parameter(p.clone()) for p in p0s]
    opt = lpmm.optim.SGD(params, qconfig=_sr_config(str(tmp_path), "real-sr", "real-nearest", "group"), **kw)
    torch.manual_seed(99)
    for k in range(3):
        for p, g in zip(params, grads[k]):
            p.grad = g.clone()
        opt.step()
    o_params = [p.clone() for p in p0s]
    o_states = [dict() for _ in shapes]
    torch.manual_seed(99)
    for k in range(3):
        for i, op in enumerate(o_params):
            T.sgd_step(op, grads[k][i], o_states[i], qm, quant=op.numel() > THRESHOLD, weight_decay=1e-4, momentum=0.9,
                       lr=1e-2, dampening=0, nesterov=False, maximize=False, ref_pack=ref.pack_nonlinear, stochastic=True)
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        assert bits_equal(p.detach(), o_params[i]), f"tensor {i}: parameters differ"
        if p.numel() > THRESHOLD:
            assert torch.equal(opt.state[p]["momentum_buffer"].view(torch.uint8), o_states[i]["buf"].view(torch.uint8))
