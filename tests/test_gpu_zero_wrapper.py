"""``lpmm.optim.ZeroAdamW`` on one GPU (a world of one rank: the sharding arithmetic, the adoption of the parameters
into the flat buffer, per-group hyper-parameters, the state_dict layout) against ``lpmm.optim.AdamW(fused=True)``:
identical parameters and identical ``state_dict()`` after 5 steps, for fp32 and 16-bit parameters, and a checkpoint
of either optimizer continues in the other."""
import pytest
import torch

from gpu_helpers import device, student_t
from test_zero_cpu import _assert_same_tree

pytestmark = pytest.mark.gpu

SHAPES = [(300, 128), (4096,), (5000,), (77, 129), (128,), (64, 64, 3), (512, 1024)]


def _model(dtype):
    torch.manual_seed(0)
    return [torch.nn.Parameter((torch.randn(s, device=device()) * 0.02).to(dtype)) for s in SHAPES]


def _groups(params):
    return [dict(params=params[:3], weight_decay=0.01), dict(params=params[3:], weight_decay=0.1, lr=2e-3)]


def _steps(opt, params, dtype, first, last):
    for s in range(first, last + 1):
        if s == 3:
            opt.param_groups[1]["lr"] = 5e-4
        for i, p in enumerate(params):
            p.grad = student_t(tuple(p.shape), 100003 * s + i, scale=1e-3 if dtype != torch.float16 else 3e-5).to(dtype)
        opt.step()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("exact", [True, False])
def test_one_rank_wrapper_equals_the_unsharded_fused_optimizer(dtype, exact):
    import lpmm
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8)
    pa, pb = _model(dtype), _model(dtype)
    za = lpmm.optim.ZeroAdamW(_groups(pa), exact_params=exact, **kw)
    ob = lpmm.optim.AdamW(_groups(pb), fused=True, exact_params=exact, **kw)
    assert all(p.data_ptr() == v.data_ptr() for p, v in zip(pa, za.engine.params)), "parameters were not adopted"
    _steps(za, pa, dtype, 1, 5)
    _steps(ob, pb, dtype, 1, 5)
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(zip(pa, pb)):
        assert torch.equal(a.detach().view(-1).view(torch.uint8), b.detach().view(-1).view(torch.uint8)), f"tensor {i}"
    sa, sb = za.state_dict(), ob.state_dict()
    _assert_same_tree(sa, sb)
    # each optimizer continues from the other's checkpoint
    pc, pd = [torch.nn.Parameter(p.detach().clone()) for p in pa], [torch.nn.Parameter(p.detach().clone()) for p in pb]
    zc = lpmm.optim.ZeroAdamW(_groups(pc), exact_params=exact, **kw)
    od = lpmm.optim.AdamW(_groups(pd), fused=True, exact_params=exact, **kw)
    zc.load_state_dict(sb)
    od.load_state_dict(sa)
    for opt, ps in ((za, pa), (ob, pb), (zc, pc), (od, pd)):
        _steps(opt, ps, dtype, 6, 7)
    torch.cuda.synchronize()
    for i in range(len(SHAPES)):
        ref = pa[i].detach().view(-1).view(torch.uint8)
        for other in (pb, pc, pd):
            assert torch.equal(ref, other[i].detach().view(-1).view(torch.uint8)), f"tensor {i} after the resume"


def test_wrapper_needs_every_gradient():
    import lpmm
    ps = _model(torch.float32)
    z = lpmm.optim.ZeroAdamW(ps)
    for p in ps[1:]:
        p.grad = torch.zeros_like(p)
    with pytest.raises(RuntimeError):
        z.step()
