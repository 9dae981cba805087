"""``lpmm.optim.SGD`` with one multi-tensor launch per parameter group (its normal mode) on a B200:
bit-identical parameters, codes and scales to the per-tensor path and to the torch-op restatement of
the reference's ``_single_tensor_sgd4bit`` (``oracle/torch_ref.py``), for every option combination,
ragged and unaligned tensors, and group ranges (shards) of the list."""
import ctypes

import pytest
import torch

from golden_cases import THRESHOLD
from gpu_helpers import bits_equal, device, student_t

pytestmark = pytest.mark.gpu

SHAPES = [(300, 130), (4097,), (127,), (64, 128), (5000, 1), (3, 3, 24, 24), (4096,), (9000,)]


def _params(seed):
    torch.manual_seed(seed)
    return [torch.randn(s, device=device()) * 0.02 for s in SHAPES]


def _run(kw, steps, fused, zero_fraction=0.0):
    import lpmm
    params = [torch.nn.Parameter(p.clone()) for p in _params(11)]
    opt = lpmm.optim.SGD(params, fused=fused, **kw)
    opt._fused = fused  # False: the per-tensor launches (what LPMM_SGD_PER_TENSOR=1 selects)
    for s in range(1, steps + 1):
        for i, p in enumerate(params):
            p.grad = student_t(p.shape, 1000 * s + i, zero_fraction=zero_fraction)
        opt.step()
    torch.cuda.synchronize()
    return opt, params


@pytest.mark.parametrize("kw", [
    dict(lr=1e-2, momentum=0.9, weight_decay=1e-4),
    dict(lr=1e-2, momentum=0.8, nesterov=True, weight_decay=0.0),
    dict(lr=3e-3, momentum=0.95, dampening=0.1, weight_decay=1e-2, maximize=True),
])
def test_fused_sgd_equals_per_tensor_path_and_restated_reference(qmaps, kw):
    from oracle import torch_ref as T
    steps = 5
    of, pf = _run(kw, steps, True, zero_fraction=0.2)
    ou, pu = _run(kw, steps, False, zero_fraction=0.2)
    qm = torch.from_numpy(qmaps["m"]).to(device())
    o_params = _params(11)
    o_states = [dict() for _ in SHAPES]
    for s in range(1, steps + 1):
        for i, op in enumerate(o_params):
            T.sgd_step(op, student_t(op.shape, 1000 * s + i, zero_fraction=0.2), o_states[i], qm,
                       quant=op.numel() > THRESHOLD, weight_decay=kw["weight_decay"], momentum=kw["momentum"],
                       lr=kw["lr"], dampening=kw.get("dampening", 0), nesterov=kw.get("nesterov", False),
                       maximize=kw.get("maximize", False))
    for i, (a, b) in enumerate(zip(pf, pu)):
        assert bits_equal(a.detach(), b.detach()), f"tensor {i}: fused and per-tensor parameters differ"
        assert bits_equal(a.detach(), o_params[i]), f"tensor {i}: parameters differ from the restated reference"
        sa, sb = of.state[a], ou.state[b]
        assert sa["momentum_buffer"].dtype == sb["momentum_buffer"].dtype
        assert torch.equal(sa["momentum_buffer"].view(torch.uint8), sb["momentum_buffer"].view(torch.uint8)), \
            f"tensor {i}: buffers (incl. padding) differ"
        if a.numel() > THRESHOLD:
            assert torch.equal(sa["momentum_buffer"].view(torch.uint8), o_states[i]["buf"].view(torch.uint8))
            assert bits_equal(sa["momentum_buffer_qstate"]["overhead"]["max1"].reshape(-1),
                              o_states[i]["buf_md"]["max1"].reshape(-1)), f"tensor {i}: scales differ"
        else:
            assert bits_equal(sa["momentum_buffer"], o_states[i]["buf"])
    assert of.state_dict()["param_groups"][0].keys() == ou.state_dict()["param_groups"][0].keys()


def test_fused_sgd_unaligned_views_and_group_ranges(qmaps):
    """Tensors carved at odd offsets (scalar path) and the list stepped as three group ranges equal
    the list stepped in one launch."""
    from lpmm import _kernels, _native as N
    qm = torch.from_numpy(qmaps["m"]).to(device())
    sizes = [128 * 40 + 5, 4097, 128 * 64, 333]

    def build(seed):
        torch.manual_seed(seed)
        entries, keep = [], []
        for i, n in enumerate(sizes):
            base = torch.randn(n + 3, device=device()) * 0.02
            gbase = torch.randn(n + 3, device=device()) * 1e-3
            off = 1 if i % 2 == 0 else 0  # odd float offset: not 32-byte aligned
            p, g = base[off:off + n], gbase[off:off + n]
            groups = (n + 127) // 128
            buf = torch.randint(-128, 128, (_kernels.packed_len(groups * 128),), dtype=torch.int8, device=device())
            sc = torch.rand(groups, 1, device=device()) * 1e-3
            entries.append((p, g, buf, buf, sc, None))
            keep += [base, gbase]
        return entries, keep

    hyper = dict(weight_decay=1e-3, momentum=0.9, lr=1e-2, dampening=0.0, nesterov=True, maximize=False)
    ea, _ka = build(5)
    eb, _kb = build(5)
    ta, tb = _kernels.TensorList(ea), _kernels.TensorList(eb)
    _kernels.sgd4bit_multi_tensor(ta, qm, **hyper)
    total = tb.total_groups
    cuts = [0, total // 3 + 1, 2 * total // 3, total]
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        _kernels.sgd4bit_multi_tensor(tb, qm, group_begin=lo, group_end=hi, **hyper)
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(zip(ea, eb)):
        n = a[0].numel()
        assert bits_equal(a[0], b[0]), f"tensor {i}: parameters"
        assert torch.equal(a[2][: (n + 127) // 128 * 64], b[2][: (n + 127) // 128 * 64]), f"tensor {i}: codes"
        assert bits_equal(a[4], b[4]), f"tensor {i}: scales"
    # and one per-tensor launch on a third copy gives the same
    ec, _kc = build(5)
    for (p, g, buf, _, sc, _n) in ec:
        N.check(N.lib.lpmm_b200_sgd4bit_step(ctypes.c_void_p(p.data_ptr()), ctypes.c_void_p(g.data_ptr()), p.numel(),
                                             ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(sc.data_ptr()),
                                             N.STATE_GROUP4, 0, ctypes.c_void_p(qm.data_ptr()), 1e-3, 0.9, 1e-2, 0.0, 1, 0,
                                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    for i, (a, c) in enumerate(zip(ea, ec)):
        n = a[0].numel()
        assert bits_equal(a[0], c[0]), f"tensor {i}: parameters vs per-tensor launch"
        assert torch.equal(a[2][: (n + 127) // 128 * 64], c[2][: (n + 127) // 128 * 64]), f"tensor {i}: codes vs per-tensor launch"
        assert bits_equal(a[4], c[4])


def test_fused_sgd_argument_errors(qmaps):
    from lpmm import _kernels, _native as N
    qm = torch.from_numpy(qmaps["m"]).to(device())
    p = torch.zeros(256, device=device())
    buf = torch.zeros(_kernels.packed_len(256), dtype=torch.int8, device=device())
    sc = torch.zeros(2, 1, device=device())
    tl = _kernels.TensorList([(p, p.clone(), buf, buf, sc, None)])
    base = dict(weight_decay=0.0, lr=1e-2, dampening=0.0, nesterov=False, maximize=False)
    with pytest.raises(N.NativeError):
        _kernels.sgd4bit_multi_tensor(tl, qm, momentum=0.0, **base)  # nothing to step without a buffer
    with pytest.raises(N.NativeError):
        _kernels.sgd4bit_multi_tensor(tl, qm, momentum=0.9, group_begin=3, group_end=2, **base)
    with pytest.raises(N.NativeError):
        _kernels.sgd4bit_multi_tensor(tl, None, momentum=0.9, **base)
