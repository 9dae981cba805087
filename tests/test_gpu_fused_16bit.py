"""The fused step for bf16 / fp16 parameters and gradients (``lpmm_b200_adamw4bit_multi_tensor_16bit``,
``lpmm.optim.AdamW(fused=True)`` on 16-bit parameters) on a B200.

The reference cannot run this combination (its launcher asks the fp32 scales for half pointers, bf16 is
not dispatched), so the step is defined through the fp32 one: widen parameters and gradients, take the
fp32 fused step, round the parameters to nearest-even.  The oracle is exactly that with the C
restatement of the reference kernel (``oracle/lpmm_oracle.c``) and the device's bias corrections:
parameters, codes and scales must be bit-identical."""
import ctypes

import numpy as np
import pytest
import torch

from gpu_helpers import bits_equal, device, nibbles, student_t
from golden_cases import THRESHOLD

pytestmark = pytest.mark.gpu


def _device_bias_corrections(beta1, beta2, step):
    from lpmm import _native as N
    out = torch.zeros(2, device=device())
    N.check(N.lib.lpmm_b200_bias_corrections(beta1, beta2, float(step), ctypes.c_void_p(out.data_ptr()),
                                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    return tuple(float(x) for x in out.cpu().numpy())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hyper", [dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01),
                                   dict(lr=1e-2, betas=(0.8, 0.95), eps=1e-30, weight_decay=0.1)])
def test_fused_16bit_optimizer_against_widened_fp32_oracle(qmaps, dtype, hyper):
    """Full and ragged groups, an odd numel, a view that is only 2-byte aligned, small tensors with fp32
    moments, 20 % exact zeros; eps = 1e-30 takes the IEEE branch.  fp16 gradients are scaled so that a
    good part of them is subnormal in fp16."""
    import lpmm
    from oracle import cpu as O
    shapes = [(300, 256), (128 * 41 + 6,), (4097,), (64, 64), (1000,), (5000, 3), (12345,)]
    torch.manual_seed(81)
    base = torch.randn(200000, device=device()).mul(0.02).to(dtype)
    p0s = [torch.randn(s, device=device()).mul(0.02).to(dtype) for s in shapes]
    p0s.append(base[1:1 + 128 * 700 + 5])  # 2-byte aligned view: the scalar path
    params = [torch.nn.Parameter(p.clone() if i < len(shapes) else p) for i, p in enumerate(p0s)]
    opt = lpmm.optim.AdamW(params, fused=True, **hyper)
    qm, qv = qmaps["m"], qmaps["v"]
    host = []
    for p in p0s:
        n = p.numel()
        quant = n > THRESHOLD
        host.append(dict(p=p.detach().float().cpu().numpy().reshape(-1).copy(), quant=quant,
                         m=np.zeros((n + 1) // 2, np.uint8) if quant else np.zeros(n, np.float32),
                         v=np.zeros((n + 1) // 2, np.uint8) if quant else np.zeros(n, np.float32),
                         ms=np.zeros((n + 127) // 128, np.float32), vs=np.zeros((n + 127) // 128, np.float32)))
    b1, b2 = hyper["betas"]
    gscale = 1e-3 if dtype == torch.bfloat16 else 3e-5
    for s in range(1, 6):
        grads = [student_t(tuple(p.shape), s * 7919 + i, zero_fraction=0.2, scale=gscale).to(dtype)
                 for i, p in enumerate(p0s)]
        for p, g in zip(params, grads):
            p.grad = g
        opt.step()
        c = _device_bias_corrections(b1, b2, s)
        for h, g in zip(host, grads):
            gn = g.float().cpu().numpy().reshape(-1).copy()
            if h["quant"]:
                O.adamw4bit(h["p"], gn, h["m"], h["v"], h["ms"], h["vs"], qm, qv, b1, b2, hyper["lr"],
                            hyper["weight_decay"], hyper["eps"], float(s), c=c)
            else:
                O.adamw_fp32(h["p"], gn, h["m"], h["v"], b1, b2, hyper["lr"], hyper["weight_decay"], hyper["eps"],
                             float(s), c=c)
            # the parameter is stored in 16 bits: round to nearest-even, continue from the rounded value
            h["p"] = torch.from_numpy(h["p"]).to(dtype).float().numpy()
    torch.cuda.synchronize()
    for i, (p, h) in enumerate(zip(params, host)):
        st = opt.state[p]
        n = p.numel()
        assert p.dtype == dtype
        assert bits_equal(p.detach().float().cpu().reshape(-1), torch.from_numpy(h["p"])), f"tensor {i}: params"
        if h["quant"]:
            for name, codes, scales in (("exp_avg", h["m"], h["ms"]), ("exp_avg_sq", h["v"], h["vs"])):
                assert st[name].dtype == torch.int8 and st[name].numel() == (n + 1) // 2
                assert np.array_equal(st[name].view(torch.uint8).cpu().numpy(), codes), f"tensor {i}: {name} codes"
                mx = st[f"{name}_qstate"]["overhead"]["max1"]
                assert mx.dtype == torch.float32
                assert bits_equal(mx.cpu().reshape(-1), torch.from_numpy(scales)), f"tensor {i}: {name} scales"
        else:
            assert st["exp_avg"].dtype == torch.float32
            assert bits_equal(st["exp_avg"].cpu().reshape(-1), torch.from_numpy(h["m"]))
            assert bits_equal(st["exp_avg_sq"].cpu().reshape(-1), torch.from_numpy(h["v"]))


def test_fused_16bit_state_dict_round_trip_keeps_fp32_scales(qmaps):
    import lpmm
    torch.manual_seed(5)
    w = torch.nn.Parameter(torch.randn(128, 96, device=device()).mul(0.02).bfloat16())
    b = torch.nn.Parameter(torch.randn(96, device=device()).mul(0.02).bfloat16())
    opt = lpmm.optim.AdamW([w, b], fused=True)
    for s in range(3):
        w.grad = student_t((128, 96), s).bfloat16()
        b.grad = student_t((96,), s + 50).bfloat16()
        opt.step()
    sd = opt.state_dict()
    w2 = torch.nn.Parameter(w.detach().clone())
    b2 = torch.nn.Parameter(b.detach().clone())
    opt2 = lpmm.optim.AdamW([w2, b2], fused=True)
    opt2.load_state_dict(sd)
    assert opt2.state[w2]["exp_avg_qstate"]["overhead"]["max1"].dtype == torch.float32
    assert opt2.state[b2]["exp_avg"].dtype == torch.float32
    for o, (x, y) in ((opt, (w, b)), (opt2, (w2, b2))):
        x.grad = student_t((128, 96), 99).bfloat16()
        y.grad = student_t((96,), 98).bfloat16()
        o.step()
    torch.cuda.synchronize()
    assert bits_equal(w.detach().float(), w2.detach().float()) and bits_equal(b.detach().float(), b2.detach().float())
    assert torch.equal(opt.state[w]["exp_avg_sq"], opt2.state[w2]["exp_avg_sq"])
