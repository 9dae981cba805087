"""Shared pieces of the GPU parity tests."""
import ctypes
import importlib.util
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HYPER = dict(beta1=0.9, beta2=0.999, lr=1e-3, weight_decay=0.01, eps=1e-8)


def device():
    return torch.device("cuda:0")


def load_reference_extension(name):
    """The reference's own compiled extension (``oracle/_ref``), or None when it was not built."""
    path = os.path.join(ROOT, "oracle", "_ref", name, name + ".so")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_qbuf = None


def device_qmaps(qmaps):
    """Both maps carved out of the middle of one buffer.  The reference's search reads qmap[-1]
    for a NaN input (fused_adamw_kernel.cu:46 with lo == 0; harmless garbage it never uses), which
    faults if the map happens to start a device allocation."""
    global _qbuf
    if _qbuf is None:
        _qbuf = torch.zeros(256, dtype=torch.float32, device=device())
        _qbuf[64:80] = torch.from_numpy(qmaps["m"])
        _qbuf[128:144] = torch.from_numpy(qmaps["v"])
        _qbuf[192:208] = torch.from_numpy(qmaps["power2"])
    return _qbuf[64:80], _qbuf[128:144], _qbuf[192:208]


_wide_bufs = {}


def device_map(qmaps, name):
    """One map of the fixture on the device, carved out of the middle of a larger zero buffer (the
    reference's kernels may read one entry before a map and, for the byte 255 of a map with fewer
    than 256 entries, up to 255 entries after its start)."""
    if name not in _wide_bufs:
        a = torch.from_numpy(np.ascontiguousarray(qmaps[name]))
        buf = torch.zeros(64 + 512, dtype=torch.float32, device=device())
        buf[64:64 + a.numel()] = a
        _wide_bufs[name] = buf
    return _wide_bufs[name][64:64 + len(qmaps[name])]


def student_t(shape, seed, dev=None, zero_fraction=0.0, scale=1e-3):
    """Seeded Student-t(3) gradients with 1 % of rows (>= 2-D) scaled by 50."""
    dev = dev or device()
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    z = torch.randn((4,) + tuple(shape), generator=g, device=dev)
    t = z[0] / torch.sqrt((z[1] ** 2 + z[2] ** 2 + z[3] ** 2) / 3.0) * scale
    if len(shape) >= 2:
        k = max(1, round(0.01 * shape[0]))
        rows = torch.randperm(shape[0], generator=g, device=dev)[:k]
        t[rows] *= 50.0
    if zero_fraction > 0:
        t[torch.rand(shape, generator=g, device=dev) < zero_fraction] = 0.0
    return t.contiguous()


def fused_state(n, dev=None):
    dev = dev or device()
    return [torch.zeros((n + 1) // 2, dtype=torch.int8, device=dev), torch.zeros((n + 1) // 2, dtype=torch.int8, device=dev),
            torch.zeros((n + 127) // 128, dtype=torch.float32, device=dev),
            torch.zeros((n + 127) // 128, dtype=torch.float32, device=dev)]


def vp(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(None)


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def nibbles(t, n):
    """The first n 4-bit codes of a packed tensor, one per uint8."""
    b = t.view(torch.uint8)
    out = torch.stack([b & 15, b >> 4], dim=1).reshape(-1)
    return out[:n]


def bits_equal(a, b):
    """Bit-for-bit equality of two float tensors (NaNs with equal payload compare equal)."""
    return bool(torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32)))


def llama7b_shapes(layers=32, hidden=4096, inter=11008, vocab=32000):
    shapes = [(vocab, hidden)]
    for _ in range(layers):
        shapes += [(hidden, hidden)] * 4 + [(inter, hidden)] * 2 + [(hidden, inter)] + [(hidden,)] * 2
    shapes += [(vocab, hidden)]
    return shapes
