"""``step_from_host`` (gradients arriving from pinned host memory, updated chunk by chunk while the copies run) gives the
results of copying everything and calling ``step()``, bit for bit: ``lpmm.optim.AdamW`` with fused, non-fused and
mixed parameter groups, skipped parameters and chunk sizes that cut the list into many launches; and the ZeRO-1 engine
on a world of one rank."""
import pytest
import torch

from gpu_helpers import device, student_t
from test_zero_cpu import _assert_same_tree

pytestmark = pytest.mark.gpu

SHAPES = [(300, 128), (4096,), (5000,), (77, 129), (128,), (64, 64, 3), (512, 1024), (1000, 768), (4097,)]


def _model(dtype=torch.float32):
    torch.manual_seed(0)
    return [torch.nn.Parameter((torch.randn(s, device=device()) * 0.02).to(dtype)) for s in SHAPES]


def _host_grads(step, dtype=torch.float32, skip=()):
    return [None if i in skip else student_t(s, 100003 * step + i).to(dtype).cpu().pin_memory()
            for i, s in enumerate(SHAPES)]


def _same(pa, pb, oa, ob):
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(zip(pa, pb)):
        assert torch.equal(a.detach().view(-1).view(torch.uint8), b.detach().view(-1).view(torch.uint8)), f"tensor {i}"
    _assert_same_tree(oa.state_dict(), ob.state_dict())


@pytest.mark.parametrize("chunk", [1 << 12, 1 << 20, 256 << 20])
@pytest.mark.parametrize("groups", ["fused", "fused_bf16", "mixed", "nonfused"])
def test_adamw_step_from_host_equals_copy_then_step(chunk, groups):
    import lpmm
    dtype = torch.bfloat16 if groups == "fused_bf16" else torch.float32
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)

    def make(params):
        if groups in ("fused", "fused_bf16"):
            return lpmm.optim.AdamW([dict(params=params[:4]), dict(params=params[4:], lr=2e-3)], fused=True, **kw)
        if groups == "mixed":
            return lpmm.optim.AdamW([dict(params=params[:4], fused=True), dict(params=params[4:], fused=False)], **kw)
        return lpmm.optim.AdamW(params, **kw)

    pa, pb = _model(dtype), _model(dtype)
    oa, ob = make(pa), make(pb)
    for s in range(1, 7):
        skip = (2,) if s == 4 else ()  # a parameter of the first group sits out one step: that group's plan is dropped
        hg = _host_grads(s, dtype, skip)
        oa.step_from_host(hg, chunk_bytes=chunk)
        for p, h in zip(pb, hg):
            p.grad = None if h is None else h.to(device())
        ob.step()
    _same(pa, pb, oa, ob)
    if groups.startswith("fused"):
        assert 1 in oa._plans, "the second group did not keep its plan: the streamed path was not taken"


def test_adamw_step_from_host_validates_its_arguments():
    import lpmm
    pa = _model()
    oa = lpmm.optim.AdamW(pa, fused=True)
    with pytest.raises(ValueError):
        oa.step_from_host([None])
    hg = _host_grads(1)
    hg[0] = hg[0][:-1]
    with pytest.raises(RuntimeError):
        oa.step_from_host(hg)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk", [1 << 12, 1 << 20])
def test_zero1_engine_step_from_host_equals_copy_then_step(dtype, chunk):
    from lpmm.zero import Zero1FusedAdamW
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, rank=0, world=1, dtype=dtype)
    za, zb = Zero1FusedAdamW(SHAPES, device(), **kw), Zero1FusedAdamW(SHAPES, device(), **kw)
    za.init_params_normal_(0.02, seed=0)
    zb.init_params_normal_(0.02, seed=0)
    for s in range(1, 5):
        grads = [student_t(sh, 100003 * s + i).to(dtype) for i, sh in enumerate(SHAPES)]
        zb.set_grad_shard_from_full(grads)
        host = zb.grad_shard.cpu().pin_memory()
        zb.step()
        za.step_from_host(host, chunk_bytes=chunk)
    torch.cuda.synchronize()
    assert torch.equal(za.flat.view(torch.uint8), zb.flat.view(torch.uint8))
    for name in ("m_codes", "v_codes", "m_scale", "v_scale", "m32", "v32"):
        assert torch.equal(getattr(za, name).view(torch.uint8), getattr(zb, name).view(torch.uint8)), name
    with pytest.raises(RuntimeError):
        za.step_from_host(host[:-1])


@pytest.mark.parametrize("chunk", [1 << 12, 256 << 20])
def test_zero_wrapper_step_from_host_equals_step(chunk):
    """``lpmm.optim.ZeroAdamW.step_from_host`` on one rank, two parameter groups (a launch never spans two groups)."""
    import lpmm
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8)
    groups = lambda ps: [dict(params=ps[:3], weight_decay=0.01), dict(params=ps[3:], weight_decay=0.1, lr=2e-3)]
    pa, pb = _model(), _model()
    za, zb = lpmm.optim.ZeroAdamW(groups(pa), **kw), lpmm.optim.ZeroAdamW(groups(pb), **kw)
    for s in range(1, 5):
        hg = _host_grads(s)
        za.step_from_host(hg, chunk_bytes=chunk)
        for p, h in zip(pb, hg):
            p.grad = h.to(device())
        zb.step()
    _same(pa, pb, za, zb)
    with pytest.raises(ValueError):
        za.step_from_host(hg[:-1])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_narrowing_kernel_equals_torch_conversion(dtype):
    """``lpmm_b200_narrow_fp32`` through the C ABI on aligned and unaligned views, sizes around the vector width,
    values that need rounding, infinities and NaN: bit-identical to ``.to(dtype)``."""
    import ctypes
    from lpmm import _native as N
    dt = N.DTYPE_BF16 if dtype == torch.bfloat16 else N.DTYPE_FP16
    torch.manual_seed(3)
    base = torch.randn(1 << 16, device=device()) * 3.0
    base[::97] = float("inf")
    base[1::193] = float("nan")
    base[2::389] = 1e-30
    out = torch.zeros((1 << 16) + 16, dtype=dtype, device=device())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for off_s, off_d, n in ((0, 0, 1 << 16), (1, 0, 1000), (3, 5, 4097), (8, 8, 12345), (0, 1, 77), (5, 0, 7), (0, 0, 0)):
        src, dst = base[off_s:off_s + n], out[off_d:off_d + n]
        dst.zero_()
        N.check(N.lib.lpmm_b200_narrow_fp32(ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()), n, dt, st))
        torch.cuda.synchronize()
        want = src.to(dtype)
        nan = torch.isnan(want)
        assert torch.equal(torch.isnan(dst), nan), (off_s, off_d, n)     # a NaN stays a NaN (payload not compared)
        assert torch.equal(dst.view(torch.int16)[~nan], want.view(torch.int16)[~nan]), (off_s, off_d, n)
    assert N.lib.lpmm_b200_narrow_fp32(None, None, 5, dt, st) == -1
    assert N.lib.lpmm_b200_narrow_fp32(None, None, 5, 9, st) == -3


def test_one_rank_engine_with_fp32_master_and_bf16_replicas():
    from lpmm.zero import Zero1FusedAdamW
    kw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, rank=0, world=1)
    za = Zero1FusedAdamW(SHAPES, device(), replica_dtype=torch.bfloat16, **kw)
    zb = Zero1FusedAdamW(SHAPES, device(), **kw)
    za.init_params_normal_(0.02, seed=0)
    zb.init_params_normal_(0.02, seed=0)
    for s in range(1, 4):
        grads = [student_t(sh, 100003 * s + i) for i, sh in enumerate(SHAPES)]
        for z in (za, zb):
            z.set_grad_shard_from_full(grads)
            z.step()
    torch.cuda.synchronize()
    assert torch.equal(za.flat.view(torch.int32), zb.flat.view(torch.int32))
    assert torch.equal(za.replica.view(torch.int16), zb.flat.to(torch.bfloat16).view(torch.int16))
    assert za.replica_params[3].shape == tuple(SHAPES[3])
    with pytest.raises(ValueError):
        Zero1FusedAdamW(SHAPES, device(), dtype=torch.bfloat16, replica_dtype=torch.bfloat16, **kw)
