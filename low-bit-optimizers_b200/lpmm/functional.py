"""Quantization maps and the quantize / dequantize front end (reference: lpmm/functional.py).

The maps are built with the same torch calls as the reference so their fp32 values are
identical (functional.py:244-315, 644-656).  ``vectorwise_quant`` / ``vectorwise_dequant`` keep the
reference's signature and metadata dictionaries for the configurations of the low-bit optimizers
-- ``scale_type`` 'group' (128 ... 4096) or 'rank1', ``quant_type`` 'nonlinear' or 'power-*',
``round_type`` 'real-nearest' or 'real-sr', 4 to 8 bits -- and run on the CUDA library; anything else
raises.
"""
import torch

from . import _kernels

__all__ = [
    "vectorwise_quant", "vectorwise_dequant", "create_general_qmap", "create_dynamic_map", "create_pow_map",
    "group_tensor", "recon_grouped_tensor", "get_sm3_statistics", "init_lpmm_generator",
]

lpmm_generator = None


def init_lpmm_generator(gpu, seed):
    """Per-rank torch generator for stochastic rounding (reference functional.py:17-23).  Kept for
    interface parity: the round-to-nearest modes implemented here never draw from it."""
    global lpmm_generator
    if lpmm_generator is None:
        lpmm_generator = torch.Generator(device=gpu)
        lpmm_generator.manual_seed(3407 if seed is None else seed)


# ----------------------------------------------------------------------------------------------
# quantization maps
# ----------------------------------------------------------------------------------------------
def _interval_means(n_points):
    edges = torch.linspace(0.1, 1, n_points)
    return (edges[:-1] + edges[1:]) / 2.0


def create_dynamic_map(signed=True, max_exponent_bits=7, total_bits=8):
    """Dynamic-exponent map: for each exponent level i the interval [0.1, 1] * 10^(i - E + 1) is cut
    into more and more equal pieces and the piece centres become code values; 0 and 1 are added
    (reference functional.py:272-315)."""
    mantissa_bits = total_bits - (1 if signed else 0)
    extra = 2 ** (mantissa_bits - max_exponent_bits) - 1
    if not signed:
        extra *= 2
    values = []
    for level in range(max_exponent_bits):
        pieces = 2 ** (level + mantissa_bits - max_exponent_bits + (0 if signed else 1))
        magnitude = 10 ** (level - (max_exponent_bits - 1))
        blocks = [_interval_means(pieces + 1)]
        if extra > 0:
            blocks.append(_interval_means(extra + 1))
        for centres in blocks:
            values += (magnitude * centres).tolist()
            if signed:
                values += (-magnitude * centres).tolist()
    values += [0, 1.0]
    values.sort()
    return torch.Tensor(values)


def create_pow_map(b, signed, p):
    """Evenly spaced points raised to the p-th power; the unsigned variant leaves out zero
    (reference functional.py:644-656)."""
    if signed:
        pts = torch.linspace(-1, 1, 2 ** b)
        return pts if p == 1 else pts.sign() * (pts.abs() ** p)
    pts = torch.linspace(0, 1, 2 ** b + 1)[1:]
    return pts if p == 1 else pts ** p


def create_general_qmap(quant_type, bit, signed):
    """Map for (quant_type, bits, signed) (reference functional.py:244-268)."""
    if bit == 1:
        return torch.Tensor([-1.0, 1.0]) if signed else torch.Tensor([0.0, 1.0])
    if quant_type == "linear":
        return None
    if quant_type == "nonlinear":
        return create_dynamic_map(signed, bit - 1, bit if signed else bit - 1)
    if quant_type == "nonlinear-nozero":
        q = create_dynamic_map(signed, bit - 1, bit if signed else bit - 1)
        if not signed:
            q[0] = q[1]
        return q
    if quant_type in ("power-1", "power-2", "power-3"):
        return create_pow_map(bit, signed, int(quant_type[-1]))
    raise ValueError(f"Not support {quant_type} quant type.")


# ----------------------------------------------------------------------------------------------
# grouping helpers (pure shape work; reference functional.py:404-431, 503-531)
# ----------------------------------------------------------------------------------------------
def group_tensor(input, gp_sz):
    if not gp_sz > 0:
        raise ValueError(f"group size need to be a positive integer, but found {gp_sz}")
    flat = input.flatten()
    rem = flat.shape[0] % gp_sz
    if rem:
        flat = torch.cat([flat, flat.new_zeros(gp_sz - rem)])
    return flat.view(-1, gp_sz)


def recon_grouped_tensor(grouped_tensor, shape):
    return grouped_tensor.flatten()[: shape.numel()].view(shape)


def get_sm3_statistics(x, **kwargs):
    """Per-axis maxima of |x|: entry i keeps axis i and reduces all others (keepdim).  Runs on the
    CUDA library for CUDA tensors."""
    return _kernels.axis_absmax(x)


def _compute_sm3_scale_tensor(max_dims):
    st = max_dims[0].clone()
    for other in max_dims[1:]:
        st = torch.min(st, other)
    return st


# ----------------------------------------------------------------------------------------------
# quantize / dequantize
# ----------------------------------------------------------------------------------------------
_MAP_TYPES = ("nonlinear", "power-1", "power-2", "power-3", "nonlinear-nozero")


def _resolve_qmap(kwargs):
    qmap = kwargs["qmap"]
    if not isinstance(qmap, torch.Tensor):
        qmap = qmap[(kwargs["b"], kwargs["signed"])][kwargs["quant_type"]]
    return qmap


def _check_supported(kwargs):
    if kwargs["quant_type"] not in _MAP_TYPES:
        raise ValueError(f"Not support {kwargs['quant_type']} quant type.")
    if kwargs["b"] not in _kernels.SUPPORTED_BITS:
        raise NotImplementedError(f"code widths {_kernels.SUPPORTED_BITS} are built in this implementation")
    if kwargs["round_type"] not in ("real-nearest", "real-sr"):
        raise NotImplementedError("only round_type 'real-nearest' and 'real-sr' are built in this implementation")
    if kwargs["scale_type"] not in ("group", "rank1"):
        raise NotImplementedError("only scale_type 'group' and 'rank1' are built in this implementation")


def vectorwise_quant(x, **kwargs):
    """Quantize ``x`` -> ``(packed int8 codes, generated metadata)`` (reference functional.py:26-59).

    The codes use the reference's layout: the normalised tensor regrouped into zero-padded rows of
    2048, two 4-bit codes (or one wider code) per byte, one trailing byte (functional.py:359-369,
    quantization_kernel.cu:475-477, 552-554; the trailing byte, uninitialised there, is 0 here)."""
    _check_supported(kwargs)
    qmap = _resolve_qmap(kwargs)
    x = x.detach()
    md = {"dtype": x.dtype, "stride": x.stride()}
    xc = x.contiguous()
    # 'real-sr': the (seed, offset) the reference's pack kernel would take from torch's CUDA generator;
    # ``mimic_rng`` (set by the optimizers when any state is stochastic) advances the generator for a
    # nearest-rounded state too, as the reference's pack call does, so that later draws line up
    sr = None
    if kwargs["round_type"] == "real-sr":
        sr = _kernels.philox_inputs(xc.device, kwargs["b"])
    elif kwargs.get("mimic_rng"):
        _kernels.philox_inputs(xc.device, kwargs["b"])
    if kwargs["scale_type"] == "group" or x.dim() == 1:
        gp_sz = kwargs["gp_sz"] if kwargs["scale_type"] == "group" else 128  # rank1 on vectors: 128 (functional.py:193)
        if kwargs["scale_type"] == "rank1":
            md["dim"] = x.dim()
        codes, max1 = _kernels.quant_group(xc, qmap, gp_sz, kwargs["b"], sr)
        md["max1"] = max1
        md["scaled_shape"] = torch.Size([max1.shape[0], gp_sz])
    else:
        md["dim"] = x.dim()
        codes, max_dims = _kernels.quant_rank1(xc, qmap, kwargs["b"], sr)
        md["max_dims"] = max_dims
        md["max1"] = None
        md["scaled_shape"] = x.shape
    return codes, md


def vectorwise_dequant(qx, denormalized=True, **kwargs):
    """Inverse of ``vectorwise_quant`` (reference functional.py:62-151)."""
    _check_supported(kwargs)
    qmap = _resolve_qmap(kwargs)
    dtype, stride, shape = kwargs["dtype"], kwargs["stride"], kwargs["shape"]
    grouped = kwargs["scale_type"] == "group" or kwargs.get("dim") == 1
    if not denormalized:
        n = kwargs["scaled_shape"].numel()
        return _kernels.dequant_plain(qx, qmap, n, kwargs["b"]).view(kwargs["scaled_shape"])
    if grouped:
        gp_sz = kwargs["scaled_shape"][1]
        x = _kernels.dequant_group(qx, qmap, kwargs["max1"], shape.numel(), gp_sz, kwargs["b"]).view(shape)
    else:
        x = _kernels.dequant_rank1(qx, qmap, kwargs["max_dims"], shape, kwargs["b"])
    if x.stride() != stride:
        out = torch.empty_strided(x.shape, stride, dtype=dtype, layout=torch.strided, device=x.device)
        out.copy_(x)
        return out
    return x.to(dtype=dtype)
