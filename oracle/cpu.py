"""numpy front end of ``lpmm_oracle.c`` (the C restatement of the reference's kernels).

TEST INFRASTRUCTURE ONLY.  ``build()`` compiles the C file with gcc (``-ffp-contract=off`` so no
multiply-add is fused behind the source's back) into ``oracle/_build/liblpmm_oracle.so``.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "lpmm_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "liblpmm_oracle.so")

_lib = None


def build(force=False):
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared", "-o", LIB, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        f, i64, i32, vp = ctypes.c_float, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.lpmm_oracle_code.restype = i32
        L.lpmm_oracle_code.argtypes = [vp, i32, f]
        L.lpmm_oracle_pack4.argtypes = [vp, i64, vp, vp]
        L.lpmm_oracle_unpack4.argtypes = [vp, i64, vp, vp]
        L.lpmm_oracle_pack8.argtypes = [vp, i64, vp, i32, vp]
        L.lpmm_oracle_unpack8.argtypes = [vp, i64, vp, i32, vp]
        L.lpmm_oracle_bias_corrections.argtypes = [f, f, f, vp]
        L.lpmm_oracle_adamw4bit_c.argtypes = [vp] * 8 + [f] * 7 + [i64, i32]
        L.lpmm_oracle_adamw4bit.argtypes = [vp] * 8 + [f] * 6 + [i64, i32]
        L.lpmm_oracle_adamw_fp32_c.argtypes = [vp] * 4 + [f] * 7 + [i64, i32]
        L.lpmm_oracle_adamw_fp32.argtypes = [vp] * 4 + [f] * 6 + [i64, i32]
        L.lpmm_oracle_threads.restype = i32
        L.lpmm_oracle_set_threads.argtypes = [i32]
        for n in ("lpmm_oracle_pack4", "lpmm_oracle_unpack4", "lpmm_oracle_pack8", "lpmm_oracle_unpack8", "lpmm_oracle_bias_corrections",
                  "lpmm_oracle_adamw4bit_c", "lpmm_oracle_adamw4bit", "lpmm_oracle_adamw_fp32_c",
                  "lpmm_oracle_adamw_fp32", "lpmm_oracle_set_threads"):
            getattr(L, n).restype = None
        _lib = L
    return _lib


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def threads():
    return lib().lpmm_oracle_threads()


def set_threads(n):
    lib().lpmm_oracle_set_threads(int(n))


def code(qmap, x, bits=4):
    qmap = _f32(qmap)
    return lib().lpmm_oracle_code(_ptr(qmap), bits, float(np.float32(x)))


def codes(qmap, xs):
    """Codes (uint8, one per element) of a float32 array; length must be even."""
    xs = _f32(xs).ravel()
    assert xs.size % 2 == 0
    packed = np.empty(xs.size // 2, np.uint8)
    qmap = _f32(qmap)
    lib().lpmm_oracle_pack4(_ptr(xs), xs.size, _ptr(qmap), _ptr(packed))
    out = np.empty(xs.size, np.uint8)
    out[0::2] = packed & 15
    out[1::2] = packed >> 4
    return out


def pack4(data, qmap):
    """``pack_nonlinear(data[G, S], qmap, 4, False)``: uint8[G*S/2 + 1], last byte 0."""
    data = _f32(data)
    n = data.size
    assert n % 2 == 0
    packed = np.zeros(n // 2 + 1, np.uint8)
    qmap = _f32(qmap)
    lib().lpmm_oracle_pack4(_ptr(data), n, _ptr(qmap), _ptr(packed))
    return packed


def unpack4(packed, qmap, num_groups, group_size):
    """``unpack_nonlinear(packed, qmap, 4, num_groups, group_size)`` -> float32[G, S]."""
    packed = np.ascontiguousarray(packed).view(np.uint8)
    n = num_groups * group_size
    out = np.empty(n, np.float32)
    qmap = _f32(qmap)
    lib().lpmm_oracle_unpack4(_ptr(packed), n, _ptr(qmap), _ptr(out))
    return out.reshape(num_groups, group_size)


def pack8(data, qmap, bits):
    """``pack_nonlinear(data[G, S], qmap, bits, False)`` for 5 <= bits <= 8: uint8[G*S + 1], last byte 0."""
    data = _f32(data)
    qmap = _f32(qmap)
    assert 5 <= bits <= 8 and qmap.size == 1 << bits
    packed = np.zeros(data.size + 1, np.uint8)
    lib().lpmm_oracle_pack8(_ptr(data), data.size, _ptr(qmap), bits, _ptr(packed))
    return packed


def unpack8(packed, qmap, bits, num_groups, group_size):
    """``unpack_nonlinear(packed, qmap, bits, num_groups, group_size)`` for 5 <= bits <= 8."""
    packed = np.ascontiguousarray(packed).view(np.uint8)
    qmap = _f32(qmap)
    assert 5 <= bits <= 8 and qmap.size == 1 << bits
    n = num_groups * group_size
    out = np.empty(n, np.float32)
    lib().lpmm_oracle_unpack8(_ptr(packed), n, _ptr(qmap), bits, _ptr(out))
    return out.reshape(num_groups, group_size)


def bias_corrections(beta1, beta2, step):
    out = np.empty(2, np.float32)
    lib().lpmm_oracle_bias_corrections(beta1, beta2, step, _ptr(out))
    return float(out[0]), float(out[1])


def adamw4bit(p, g, mq, vq, ms, vs, qmap_m, qmap_v, beta1, beta2, lr, wd, eps, step, variant=0, c=None):
    """Fused 4-bit AdamW step, in place on the numpy arrays (p, ms, vs float32; mq, vq uint8).
    ``c=(c1, c2s)`` overrides the host-powf bias corrections."""
    assert p.dtype == np.float32 and g.dtype == np.float32 and ms.dtype == np.float32 and vs.dtype == np.float32
    assert mq.dtype == np.uint8 and vq.dtype == np.uint8
    for a in (p, g, mq, vq, ms, vs):
        assert a.flags.c_contiguous
    qm, qv = _f32(qmap_m), _f32(qmap_v)
    n = p.size
    assert mq.size >= (n + 1) // 2 and ms.size >= (n + 127) // 128
    if c is None:
        lib().lpmm_oracle_adamw4bit(_ptr(p), _ptr(g), _ptr(mq), _ptr(vq), _ptr(ms), _ptr(vs), _ptr(qm), _ptr(qv),
                                    beta1, beta2, lr, wd, eps, step, n, variant)
    else:
        lib().lpmm_oracle_adamw4bit_c(_ptr(p), _ptr(g), _ptr(mq), _ptr(vq), _ptr(ms), _ptr(vs), _ptr(qm), _ptr(qv),
                                      beta1, beta2, lr, wd, eps, c[0], c[1], n, variant)


def adamw_fp32(p, g, m, v, beta1, beta2, lr, wd, eps, step, variant=0, c=None):
    for a in (p, g, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    n = p.size
    if c is None:
        lib().lpmm_oracle_adamw_fp32(_ptr(p), _ptr(g), _ptr(m), _ptr(v), beta1, beta2, lr, wd, eps, step, n, variant)
    else:
        lib().lpmm_oracle_adamw_fp32_c(_ptr(p), _ptr(g), _ptr(m), _ptr(v), beta1, beta2, lr, wd, eps, c[0], c[1], n,
                                       variant)
