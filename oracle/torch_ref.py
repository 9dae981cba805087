"""torch-op restatement of the reference's non-fused Python path.  TEST INFRASTRUCTURE ONLY.

The reference's non-fused optimizers are sequences of torch element-wise ops around two extension
calls (pack/unpack).  This module restates those sequences op for op, so that running it on a
device reproduces what the reference computes on that device:

* on CPU, in a container that holds the reference checkout, it is compared bit for bit with the
  reference's own Python (tests/test_oracle_python_path.py, fixtures under tests/golden/ made by
  tests/golden/make_python_golden.py) -- that pins it;
* on a GPU it is the parity target of the CUDA kernels (same torch CUDA kernels the reference
  would run), with the pack/unpack pair replaced by the bucketize form below, itself checked
  against the reference's compiled pack/unpack kernels when those are available.

Every function cites the reference lines it follows (paths within thu-ml/low-bit-optimizers).
"""
import math

import torch

PACK_ROW = 2048  # functional.py:362


# ---- maps and the nearest-code rule ----------------------------------------------------------
def midpoints(qmap):
    return (qmap[:-1] + qmap[1:]) * 0.5


def codes_of(x, qmap):
    """quantize_bsearch<false> (quantization_kernel.cu:397-427): #midpoints < x.  A NaN makes the
    search return -1, stored as 15 by the 4-bit kernel (mask, :454) and as 255 by the
    one-code-per-byte kernel (cast, :533)."""
    c = torch.bucketize(x, midpoints(qmap), right=False)
    nan_code = 15 if qmap.numel() == 16 else 255
    c = torch.where(torch.isnan(x), torch.full_like(c, nan_code), c)
    return c.to(torch.uint8)


def pack_nonlinear(data, qmap):
    """pack_nonlinear(data[G, S], qmap, bits, False) with bits = log2(len(qmap)): two codes per byte for
    4 bits (quantization_kernel.cu:430-513), one per byte for 5 ... 8 (:515-591), plus the trailing
    byte (uninitialised in the reference, 0 here)."""
    c = codes_of(data.reshape(-1), qmap)
    packed = (c[0::2] | (c[1::2] << 4)).to(torch.uint8) if qmap.numel() == 16 else c
    out = torch.zeros(packed.numel() + 1, dtype=torch.uint8, device=data.device)
    out[:-1] = packed
    return out.view(torch.int8)


def unpack_nonlinear(packed, qmap, num_groups, group_size):
    """unpack_nonlinear (quantization_kernel.cu:604-653, 655-693): float[num_groups, group_size].  A
    byte beyond a map of fewer than 8 bits (the 255 of a NaN) decodes to NaN."""
    n = num_groups * group_size
    if qmap.numel() == 16:
        b = packed.view(torch.uint8)[: n // 2].to(torch.int64)
        idx = torch.stack([b & 15, b >> 4], dim=1).reshape(-1)
        return qmap[idx].reshape(num_groups, group_size)
    idx = packed.view(torch.uint8)[:n].to(torch.int64)
    ext = torch.cat([qmap, torch.full((256 - qmap.numel(),), float("nan"), dtype=qmap.dtype, device=qmap.device)])
    return ext[idx].reshape(num_groups, group_size)


# ---- grouping (functional.py:404-431) -------------------------------------------------------
def group_tensor(x, gp_sz):
    flat = x.flatten()
    rem = flat.shape[0] % gp_sz
    if rem:
        flat = torch.cat([flat, torch.zeros(gp_sz - rem, dtype=x.dtype, device=x.device)])
    return flat.view(-1, gp_sz)


def recon(grouped, shape):
    return grouped.flatten()[: shape.numel()].view(shape)


def max_except_dim(t, dim):
    """_max_reduce_except_dim (functional.py:521-531)."""
    r = t
    for d in range(t.dim()):
        if d != dim:
            r = r.max(dim=d, keepdim=True).values
    return r


def scale_tensor(max_dims):
    """_compute_sm3_scale_tensor (functional.py:503-509)."""
    st = max_dims[0].clone()
    for m in max_dims[1:]:
        st = torch.min(st, m)
    return st


# ---- vectorwise_quant / vectorwise_dequant for the optimizer's configurations ---------------
def vectorwise_quant(x, qmap, scale_type, gp_sz=128, ref_pack=None, stochastic=False):
    """functional.py:26-59 with quant_scaling (154-241) and nonlinear_quant (359-369).

    ``ref_pack``: the reference's own compiled ``pack_nonlinear`` (CUDA only).  When given it does the
    packing, with ``stochastic`` as its flag -- it draws from torch's default CUDA generator (and
    advances it even when not stochastic), which is what 'real-sr' configurations are checked against."""
    md = {"dtype": x.dtype, "stride": x.stride()}
    qx = x.detach()
    if scale_type == "group" or (scale_type == "rank1" and qx.dim() == 1):
        if scale_type == "rank1":
            md["dim"] = qx.dim()
            gp_sz = 128
        qx = group_tensor(qx, gp_sz)
        max1 = max_except_dim(qx.abs(), 0)
        qx = qx.div(max1)
        md["max1"] = max1
    elif scale_type == "rank1":
        md["dim"] = qx.dim()
        a = qx.abs()
        max_dims = [max_except_dim(a, i) for i in range(a.dim())]
        qx = qx.div(scale_tensor(max_dims))
        md["max_dims"] = max_dims
        md["max1"] = None
    else:
        raise NotImplementedError(scale_type)
    md["scaled_shape"] = qx.shape
    grouped = group_tensor(qx, PACK_ROW)
    if ref_pack is not None:
        bits = int(math.log2(qmap.numel()))
        packed = ref_pack(grouped.contiguous(), qmap, bits, bool(stochastic))
        packed[-1] = 0  # the byte the reference leaves unwritten
        return packed, md
    return pack_nonlinear(grouped, qmap), md


def vectorwise_dequant(q, qmap, scale_type, shape, md):
    """functional.py:62-151 with nonlinear_dequant (393-400)."""
    ss = md["scaled_shape"]
    x = recon(unpack_nonlinear(q, qmap, (ss.numel() + PACK_ROW - 1) // PACK_ROW, PACK_ROW), ss)
    if scale_type == "group" or md.get("dim") == 1:
        x = recon(x.mul(md["max1"]), shape)
    else:
        x = x.mul(scale_tensor(md["max_dims"]))
    if x.stride() != md["stride"]:
        out = torch.empty_strided(x.shape, md["stride"], dtype=md["dtype"], device=x.device)
        out.copy_(x)
        return out
    return x.to(dtype=md["dtype"])


# ---- non-fused AdamW (adamw.py:332-436) -----------------------------------------------------
def adamw_step(p, g, st, qmap_m, qmap_v, *, m_quant, v_quant, v_scale_type, beta1, beta2, lr, weight_decay, eps,
               step, m_gp_sz=128, v_gp_sz=128, ref_pack=None, m_stochastic=False, v_stochastic=False,
               arithmetic="torch", c=None):
    """One tensor of _single_tensor_adamw4bit.  ``st`` is a dict: 'm', 'v' hold either None (not yet
    initialised), an fp32 tensor (not quantized) or packed codes with 'm_md' / 'v_md' metadata.

    ``arithmetic="fused"``: between the reference's dequantisation and quantisation, the element-wise
    update of its fused kernels (fused_adamw_kernel.cu:69-77 = 121-128) through the C restatement
    (``cpu.adamw_fp32``), ``c`` = the device's (1 - beta1^t, sqrt(1 - beta2^t)).  The reference has no step
    that combines the two; this composition of its parts is what the library's fused step on rank-1 states is
    checked against."""
    if arithmetic == "torch":
        p.mul_(1 - lr * weight_decay)                                    # :369
    if st.get("m") is None:
        m = torch.zeros_like(p)                                          # :394-395
    elif m_quant:
        m = vectorwise_dequant(st["m"], qmap_m, "group", p.shape, st["m_md"])    # :396-399
    else:
        m = st["m"]
    if st.get("v") is None:
        v = torch.zeros_like(p)                                          # :402-403
    elif v_quant:
        v = vectorwise_dequant(st["v"], qmap_v, v_scale_type, p.shape, st["v_md"])
    else:
        v = st["v"]
    if arithmetic == "fused":
        from . import cpu
        host = [t.detach().cpu().contiguous().numpy().reshape(-1).copy() for t in (p, g, m, v)]
        cpu.adamw_fp32(*host, beta1, beta2, lr, weight_decay, eps, step, c=c)
        p.copy_(torch.from_numpy(host[0]).view(p.shape))
        m = torch.from_numpy(host[2]).view(p.shape).to(p.device)
        v = torch.from_numpy(host[3]).view(p.shape).to(p.device)
    else:
        m.lerp_(g, 1 - beta1)                                            # :412
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)                    # :413
        bc1 = 1 - beta1 ** step                                          # :416-419
        bc2 = 1 - beta2 ** step
        step_size = lr / bc1
        bc2_sqrt = math.sqrt(bc2)
        denom = (v.sqrt() / bc2_sqrt).add_(eps)                          # :421
        p.addcdiv_(m, denom, value=-step_size)                           # :422
    if m_quant:
        st["m"], st["m_md"] = vectorwise_quant(m, qmap_m, "group", m_gp_sz, ref_pack, m_stochastic)   # :425-428
    else:
        st["m"] = m
    if v_quant:
        st["v"], st["v_md"] = vectorwise_quant(v, qmap_v, v_scale_type, v_gp_sz, ref_pack, v_stochastic)  # :431-434
    else:
        st["v"] = v


# ---- factored second moment (adamw.py:571-627) ----------------------------------------------
def approx_sq_grad(row, col):
    r = (row / row.mean(dim=-1, keepdim=True)).unsqueeze(-1)
    return torch.mul(r, col.unsqueeze(-2))


def factored_step(p, g, st, qmap_m, *, m_quant, beta1, beta2, lr, weight_decay, eps, step, m_gp_sz=128):
    """param decay (adamw.py:369/478) followed by _single_quantized_factored_update (579-627).
    st: 'm' as above, 'row', 'col' fp32 accumulators."""
    p.mul_(1 - lr * weight_decay)
    if st.get("m") is None:
        m = torch.zeros_like(p)
    elif m_quant:
        m = vectorwise_dequant(st["m"], qmap_m, "group", p.shape, st["m_md"])
    else:
        m = st["m"]
    m.lerp_(g, 1 - beta1)                                                # :607
    update = g ** 2                                                      # :608
    st["row"].mul_(beta2).add_(update.mean(dim=-1), alpha=1 - beta2)     # :609
    st["col"].mul_(beta2).add_(update.mean(dim=-2), alpha=1 - beta2)     # :610
    v = approx_sq_grad(st["row"], st["col"])                             # :611
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    step_size = lr / bc1
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)                        # :618
    p.addcdiv_(m, denom, value=-step_size)                               # :619
    if m_quant:
        st["m"], st["m_md"] = vectorwise_quant(m, qmap_m, "group", m_gp_sz)   # :622-625
    else:
        st["m"] = m


# ---- SGD with momentum (sgd.py:133-187) -----------------------------------------------------
def sgd_step(p, g, st, qmap, *, quant, weight_decay, momentum, lr, dampening, nesterov, maximize, gp_sz=128,
             ref_pack=None, stochastic=False):
    d_p = g if not maximize else -g
    if weight_decay != 0:
        d_p = d_p.add(p, alpha=weight_decay)                             # :156
    if momentum != 0:
        if st.get("buf") is None:
            buf = torch.clone(d_p).detach()                              # :164
        else:
            buf = vectorwise_dequant(st["buf"], qmap, "group", p.shape, st["buf_md"]) if quant else st["buf"]
            buf.mul_(momentum).add_(d_p, alpha=1 - dampening)            # :174
        d_p = d_p.add(buf, alpha=momentum) if nesterov else buf          # :177-180
    p.add_(d_p, alpha=-lr)                                               # :182
    if momentum != 0:
        if quant:
            st["buf"], st["buf_md"] = vectorwise_quant(buf, qmap, "group", gp_sz, ref_pack, stochastic)   # :185-187
        else:
            st["buf"] = buf
