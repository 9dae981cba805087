"""``lpmm.functional`` and the ``lpmm.cpp_extension.quantization`` stand-ins on a B200: against the
reference's own compiled pack/unpack kernels when ``oracle/_ref`` is present, against the torch-op
restatement otherwise and always.  Codes and scales bit-identical; dequantized values bit-identical."""
import numpy as np
import pytest
import torch

from gpu_helpers import bits_equal, device, device_map, device_qmaps, load_reference_extension, student_t

pytestmark = pytest.mark.gpu


def _special_values(qmap):
    q = qmap.cpu()
    mids = (q[:-1] + q[1:]) * 0.5
    up = torch.nextafter(mids, torch.full_like(mids, 2.0))
    dn = torch.nextafter(mids, torch.full_like(mids, -2.0))
    extra = torch.tensor([0.0, -0.0, 1.0, -1.0, 2.0, -2.0, 1e-30, -1e-30, float("inf"), float("-inf"), float("nan"), 1.1249,
                          0.5, 1e-8])
    return torch.cat([q, mids, up, dn, extra])


@pytest.mark.parametrize("which", ["m", "v"])
def test_pack_unpack_match_reference_kernels(qmaps, which):
    from lpmm.cpp_extension import quantization as mine
    ref = load_reference_extension("quantization")
    qm, qv, _ = device_qmaps(qmaps)
    qmap = qm if which == "m" else qv
    torch.manual_seed(0)
    x = torch.cat([_special_values(qmap), torch.rand(2048 * 5) * 2.2 - 1.1])
    x = torch.cat([x, torch.zeros((-x.numel()) % 2048)]).to(device()).view(-1, 2048)
    packed = mine.pack_nonlinear(x, qmap, 4, False)
    assert packed.dtype == torch.int8 and packed.numel() == x.numel() // 2 + 1 and int(packed[-1]) == 0
    from oracle import torch_ref as T
    assert torch.equal(packed, T.pack_nonlinear(x, qmap)), "codes differ from the restated rule"
    out = mine.unpack_nonlinear(packed, qmap, 4, x.shape[0], 2048)
    assert out.shape == x.shape and bits_equal(out, T.unpack_nonlinear(packed, qmap, x.shape[0], 2048))
    if ref is not None:
        r_packed = ref.pack_nonlinear(x, qmap, 4, False)
        torch.cuda.synchronize()
        assert torch.equal(packed[:-1], r_packed[:-1]), "codes differ from the reference's kernel"
        assert bits_equal(out, ref.unpack_nonlinear(r_packed, qmap, 4, x.shape[0], 2048))


@pytest.mark.parametrize("which", ["m", "v", "power2"])
@pytest.mark.parametrize("n,offset", [(2048 * 3 + 46, 0), (6, 0), (2048 + 32, 4), (32, 0), (2048 * 2, 8), (2048 * 40 + 8, 0)])
def test_pack_unpack_sizes_and_alignments_through_the_c_abi(qmaps, which, n, offset):
    """The 4-bit pack / unpack take wide accesses (8 values per lane) for whole units of 8 values in 32-byte aligned
    buffers and a byte-wise path for the rest, for shorter inputs and for other alignments: every combination
    against the restated rule, special values included."""
    import ctypes
    from lpmm import _native as N
    from oracle import torch_ref as T
    qm, qv, q2 = device_qmaps(qmaps)
    qmap = {"m": qm, "v": qv, "power2": q2}[which]
    torch.manual_seed(n + offset)
    vals = torch.cat([_special_values(qmap), torch.rand(max(n, 64)) * 2.2 - 1.1])
    vals = vals[torch.randperm(vals.numel())][:n].contiguous()
    buf = torch.zeros(n + 16, device=device())
    x = buf[offset: offset + n]
    x.copy_(vals.to(device()))
    obuf = torch.full((n // 2 + 1 + 64,), 77, dtype=torch.int8, device=device())
    out = obuf[4 * offset: 4 * offset + n // 2 + 1]
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    N.check(N.lib.lpmm_b200_pack_nonlinear(vp(x), n, vp(qmap), 4, vp(out), st))
    torch.cuda.synchronize()
    assert torch.equal(out, T.pack_nonlinear(x.contiguous().view(1, -1), qmap)), "codes"
    assert int(obuf[4 * offset + n // 2 + 1]) == 77, "wrote past the trailing byte"
    back = torch.full((n + 16,), -5.0, device=device())
    dst = back[offset: offset + n]
    N.check(N.lib.lpmm_b200_unpack_nonlinear(vp(out), vp(qmap), 4, n, vp(dst), st))
    torch.cuda.synchronize()
    assert bits_equal(dst, T.unpack_nonlinear(out, qmap, 1, n).view(-1))
    assert float(back[offset + n]) == -5.0 and (offset == 0 or float(back[offset - 1]) == -5.0)


@pytest.mark.parametrize("bits", [5, 6, 7, 8])
@pytest.mark.parametrize("kind", ["nonlinear", "power1"])
def test_pack_unpack_one_code_per_byte_match_reference_kernels(qmaps, bits, kind):
    """Maps of 5 to 8 bits (pack_nonlinear_8bit / unpack_nonlinear_8bit in the reference).  NaN is
    left out of the comparison with the reference's kernel: it stores 255 there, which its unpack
    kernel then reads from beyond a map of fewer than 256 entries; the 255 itself is checked
    against the restated rule."""
    from lpmm.cpp_extension import quantization as mine
    from oracle import torch_ref as T
    ref = load_reference_extension("quantization")
    qmap = device_map(qmaps, f"{kind}_{bits}")
    assert qmap.numel() == 1 << bits
    torch.manual_seed(bits)
    special = _special_values(qmap)
    x = torch.cat([special[~torch.isnan(special)], torch.rand(2048 * 5) * 2.2 - 1.1])
    x = torch.cat([x, torch.zeros((-x.numel()) % 2048)]).to(device()).view(-1, 2048)
    packed = mine.pack_nonlinear(x, qmap, bits, False)
    assert packed.dtype == torch.int8 and packed.numel() == x.numel() + 1 and int(packed[-1]) == 0
    assert torch.equal(packed, T.pack_nonlinear(x, qmap)), "codes differ from the restated rule"
    out = mine.unpack_nonlinear(packed, qmap, bits, x.shape[0], 2048)
    assert out.shape == x.shape and bits_equal(out, T.unpack_nonlinear(packed, qmap, x.shape[0], 2048))
    if ref is not None:
        r_packed = ref.pack_nonlinear(x, qmap, bits, False)
        torch.cuda.synchronize()
        assert torch.equal(packed[:-1], r_packed[:-1]), "codes differ from the reference's kernel"
        assert bits_equal(out, ref.unpack_nonlinear(r_packed, qmap, bits, x.shape[0], 2048))
    xn = x.clone()
    xn[0, :7] = float("nan")
    pn = mine.pack_nonlinear(xn, qmap, bits, False)
    assert torch.equal(pn, T.pack_nonlinear(xn, qmap)) and (pn[:7].view(torch.uint8) == 255).all()
    back = mine.unpack_nonlinear(pn, qmap, bits, x.shape[0], 2048)
    if bits < 8:
        assert torch.isnan(back[0, :7]).all()
    else:
        assert bits_equal(back[0, :7], qmap[255].expand(7).contiguous())


def test_pack_argument_checks(qmaps):
    from lpmm.cpp_extension import quantization as mine
    qm, _, _ = device_qmaps(qmaps)
    x = torch.zeros(2, 2048, device=device())
    with pytest.raises(RuntimeError):
        mine.pack_nonlinear(x.cpu(), qm, 4, False)
    with pytest.raises(RuntimeError):
        mine.pack_nonlinear(x.view(-1), qm, 4, False)
    with pytest.raises(RuntimeError):
        mine.pack_nonlinear(x, qm, 9, False)
    assert mine.pack_nonlinear(x, qm, 4, True).numel() == x.numel() // 2 + 1  # stochastic rounding is built
    with pytest.raises(RuntimeError):
        mine.unpack_nonlinear(torch.zeros(10, device=device()), qm, 4, 1, 2048)


_META = dict(b=4, quant_type=None, round_type="real-nearest", gp_sz=128, signed=None)


@pytest.mark.parametrize("shape", [(4096,), (4097,), (127,), (300, 130), (3, 3, 24, 24), (5000, 1), (2, 3, 4, 5, 6)])
@pytest.mark.parametrize("scale_type,which", [("group", "m"), ("rank1", "v"), ("group", "v")])
def test_vectorwise_quant_dequant_match_restated_reference(qmaps, shape, scale_type, which):
    import lpmm.functional as F
    from oracle import torch_ref as T
    qm, qv, _ = device_qmaps(qmaps)
    qmap = qm if which == "m" else qv
    x = student_t(shape, 77, zero_fraction=0.1)
    if which == "v":
        x = x * x
    kw = dict(_META, quant_type="nonlinear" if which == "m" else "power-1", signed=(which == "m"), scale_type=scale_type)
    codes, md = F.vectorwise_quant(x, qmap=qmap, shape=x.shape, **kw)
    o_codes, o_md = T.vectorwise_quant(x, qmap, scale_type)
    assert codes.dtype == torch.int8 and codes.numel() == o_codes.numel()
    assert torch.equal(codes.view(torch.uint8), o_codes.view(torch.uint8)), "codes differ"
    assert md["scaled_shape"] == o_md["scaled_shape"] and md["dtype"] == x.dtype and md["stride"] == x.stride()
    if scale_type == "rank1" and len(shape) > 1:
        assert md["dim"] == len(shape) and md["max1"] is None
        for a, b in zip(md["max_dims"], o_md["max_dims"]):
            assert a.shape == b.shape and bits_equal(a, b)
    else:
        assert bits_equal(md["max1"], o_md["max1"]) and md["max1"].shape == o_md["max1"].shape
    back = F.vectorwise_dequant(codes, qmap=qmap, shape=x.shape, **{**kw, **md})
    o_back = T.vectorwise_dequant(o_codes, qmap, scale_type, x.shape, o_md)
    assert back.shape == x.shape and bits_equal(back, o_back)


@pytest.mark.parametrize("shape", [(4097,), (127,), (300, 130), (3, 3, 24, 24), (5000, 1), (9000,)])
@pytest.mark.parametrize("bits,gp_sz,scale_type,kind", [
    (8, 128, "group", "nonlinear"), (8, 128, "rank1", "power1"), (5, 128, "group", "nonlinear"),
    (6, 128, "rank1", "power1"), (7, 128, "group", "power1"), (4, 256, "group", "m"), (4, 512, "group", "m"),
    (4, 1024, "group", "v"), (4, 2048, "group", "m"), (4, 4096, "group", "m"), (8, 4096, "group", "nonlinear"),
    (5, 512, "group", "nonlinear")])
def test_vectorwise_quant_dequant_wider_codes_and_larger_groups(qmaps, shape, bits, gp_sz, scale_type, kind):
    import lpmm.functional as F
    from oracle import torch_ref as T
    name = kind if bits == 4 else f"{kind}_{bits}"
    qmap = device_map(qmaps, name)
    unsigned = kind in ("v", "power1")
    x = student_t(shape, 78)  # dense: with one code per byte an all-zero group is NaN in the reference as well
    if unsigned:
        x = x * x
    kw = dict(_META, b=bits, gp_sz=gp_sz, quant_type="power-1" if unsigned else "nonlinear", signed=not unsigned,
              scale_type=scale_type)
    codes, md = F.vectorwise_quant(x, qmap=qmap, shape=x.shape, **kw)
    o_codes, o_md = T.vectorwise_quant(x, qmap, scale_type, gp_sz)
    assert codes.dtype == torch.int8 and codes.numel() == o_codes.numel()
    assert torch.equal(codes.view(torch.uint8), o_codes.view(torch.uint8)), "codes differ"
    assert md["scaled_shape"] == o_md["scaled_shape"]
    if scale_type == "rank1" and len(shape) > 1:
        for a, b in zip(md["max_dims"], o_md["max_dims"]):
            assert a.shape == b.shape and bits_equal(a, b)
    else:
        assert bits_equal(md["max1"], o_md["max1"]) and md["max1"].shape == o_md["max1"].shape
    back = F.vectorwise_dequant(codes, qmap=qmap, shape=x.shape, **{**kw, **md})
    o_back = T.vectorwise_dequant(o_codes, qmap, scale_type, x.shape, o_md)
    assert back.shape == x.shape and bits_equal(back, o_back)


def test_vectorwise_quant_rejects_what_is_not_built(qmaps):
    import lpmm.functional as F
    qm, _, _ = device_qmaps(qmaps)
    x = torch.randn(4096, device=device())
    base = dict(_META, quant_type="nonlinear", signed=True, scale_type="group", qmap=qm, shape=x.shape)
    with pytest.raises(NotImplementedError):
        F.vectorwise_quant(x, **{**base, "b": 2})
    with pytest.raises(NotImplementedError):
        F.vectorwise_quant(x, **{**base, "gp_sz": 64})
    with pytest.raises(RuntimeError):
        F.vectorwise_quant(x, **{**base, "b": 8})  # a 16-entry map is not an 8-bit map
    with pytest.raises(NotImplementedError):
        F.vectorwise_quant(x, **{**base, "round_type": "sr"})
    with pytest.raises(NotImplementedError):
        F.vectorwise_quant(x, **{**base, "scale_type": "dim0"})
    with pytest.raises(ValueError):
        F.vectorwise_quant(x, **{**base, "quant_type": "bogus"})
