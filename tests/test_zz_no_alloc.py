"""The allocation-free factored step (``lpmm_b200_adamw4bit_factored_step_noalloc``), for callers
that have no way to hand the library a scratch buffer because they may not allocate device memory
themselves.  Called through the C ABI on a B200, twice in a row, and compared with the ordinary
entry point given a caller-allocated scratch buffer: both run the same kernels, so parameters,
codes, scales and the row/column accumulators must be bit-identical after each call.  Also checks
that a tensor too large for the built-in scratch is refused with a clear status.

This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from gpu_helpers import bits_equal, device, student_t, vp, stream

pytestmark = pytest.mark.gpu


def _step_tensor(N, p, g, m, m_max1, row, col, first):
    t = N.StepTensor()
    t.p, t.g, t.numel, t.ndim, t.first = p.data_ptr(), g.data_ptr(), p.numel(), p.dim(), int(first)
    for i, d in enumerate(p.shape):
        t.shape[i] = d
    t.m_mode, t.v_mode = N.STATE_GROUP4, N.STATE_FACTORED
    t.m, t.m_max1 = m.data_ptr(), m_max1.data_ptr()
    t.row, t.col = row.data_ptr(), col.data_ptr()
    return t


def _fresh(shape, seed):
    from lpmm import _kernels as K
    torch.manual_seed(seed)
    n = int(np.prod(shape))
    groups = (n + 127) // 128
    return dict(p=torch.randn(shape, device=device()) * 0.02,
                m=torch.zeros(K.packed_len(groups * 128), dtype=torch.int8, device=device()),
                m_max1=torch.zeros(groups, 1, device=device()),
                row=torch.zeros(shape[:-1], device=device()), col=torch.zeros(shape[:-2] + shape[-1:], device=device()))


@pytest.mark.parametrize("shape", [(300, 200), (2, 3, 70, 64)])
def test_noalloc_factored_step_equals_ordinary_entry_point(qmaps, shape):
    from lpmm import _native as N
    qm = torch.from_numpy(qmaps["m"]).to(device())
    a, b = _fresh(shape, 11), _fresh(shape, 11)
    shp = (ctypes.c_int64 * len(shape))(*shape)
    need = int(N.lib.lpmm_b200_factored_scratch_bytes(shp, len(shape)))
    assert 0 < need <= N.STATIC_SCRATCH_BYTES
    scratch = torch.empty(need, dtype=torch.uint8, device=device())
    hyper = (0.9, 0.999, 1e-3, 0.01, 1e-8)
    for step in (1, 2):                                   # two calls in a row through each entry point
        g = student_t(shape, 4000 + step)
        ta = _step_tensor(N, a["p"], g, a["m"], a["m_max1"], a["row"], a["col"], first=(step == 1))
        tb = _step_tensor(N, b["p"], g, b["m"], b["m_max1"], b["row"], b["col"], first=(step == 1))
        N.check(N.lib.lpmm_b200_adamw4bit_factored_step_noalloc(ctypes.byref(ta), vp(qm), *hyper, float(step), stream()))
        N.check(N.lib.lpmm_b200_adamw4bit_unfused_step(ctypes.byref(tb), vp(qm), None, *hyper, float(step), vp(scratch),
                                                       scratch.numel(), stream()))
        torch.cuda.synchronize()
        assert bits_equal(a["p"], b["p"]), f"step {step}: parameters differ"
        assert torch.equal(a["m"], b["m"]), f"step {step}: first-moment codes differ"
        for k in ("m_max1", "row", "col"):
            assert bits_equal(a[k], b[k]), f"step {step}: {k} differs"
    assert float(a["row"].abs().max()) > 0 and float(a["col"].abs().max()) > 0


def test_noalloc_refuses_what_does_not_fit_and_wrong_modes(qmaps):
    from lpmm import _native as N
    t = N.StepTensor()
    t.ndim, t.v_mode = 2, N.STATE_FACTORED
    t.shape[0], t.shape[1] = 64 * 600, 4096               # 600 row tiles x 4096 columns x 4 B > 8 MiB
    t.numel = t.shape[0] * t.shape[1]
    rc = N.lib.lpmm_b200_adamw4bit_factored_step_noalloc(ctypes.byref(t), None, 0.9, 0.999, 1e-3, 0.0, 1e-8, 1.0, None)
    assert rc == -6
    assert b"limit" in N.lib.lpmm_b200_strerror(rc)
    t.v_mode = N.STATE_GROUP4
    assert N.lib.lpmm_b200_adamw4bit_factored_step_noalloc(ctypes.byref(t), None, 0.9, 0.999, 1e-3, 0.0, 1e-8, 1.0, None) == -3
    assert N.lib.lpmm_b200_adamw4bit_factored_step_noalloc(None, None, 0.9, 0.999, 1e-3, 0.0, 1e-8, 1.0, None) == -1
