"""The short arithmetic sequences of the step kernels against the IEEE instructions and the reference's search, on a
B200 (``lpmm_b200_test_exactness``): 2^28 seeded pseudo-random and adversarial operands per check (around every
midpoint of the maps, at the 2^-60 / 2^60 guards, perfect squares, zeros), zero mismatches required."""
import ctypes

import pytest
import torch

from gpu_helpers import device, device_qmaps, stream, vp

pytestmark = pytest.mark.gpu

N_SAMPLES = 1 << 28
NAMES = {0: "shared-reciprocal division", 1: "code of a shared-reciprocal quotient", 2: "short square root",
         3: "short division", 4: "code of an arbitrary float"}


def _run(check, qmap, seed):
    from lpmm import _native as N
    out = torch.zeros(2, dtype=torch.int64, device=device())
    N.check(N.lib.lpmm_b200_test_exactness(check, vp(qmap), seed, N_SAMPLES, vp(out), stream()))
    torch.cuda.synchronize()
    bad, tested = (int(x) for x in out.cpu())
    return bad, tested


@pytest.mark.parametrize("check", [0, 2, 3])
def test_short_sequences_equal_ieee_results(check):
    bad, tested = _run(check, None, 1234 + check)
    print(f"{NAMES[check]}: {bad} mismatches in {tested} operands")
    assert tested > N_SAMPLES // 2
    assert bad == 0


@pytest.mark.parametrize("check", [1, 4])
@pytest.mark.parametrize("which", ["m", "v", "power2"])
def test_codes_equal_the_reference_search(qmaps, check, which):
    """'m': the signed nonlinear map (table), 'v': the linear map k/16 (closed form), 'power2': another unsigned map
    (table)."""
    qm, qv, q2 = device_qmaps(qmaps)
    qmap = {"m": qm, "v": qv, "power2": q2}[which]
    bad, tested = _run(check, qmap, 99 + check)
    print(f"{NAMES[check]}, map {which}: {bad} mismatches in {tested} operands")
    assert tested > N_SAMPLES // 8
    assert bad == 0


def test_bad_arguments():
    from lpmm import _native as N
    assert N.lib.lpmm_b200_test_exactness(7, None, 0, 10, None, None) == -3
    assert N.lib.lpmm_b200_test_exactness(1, None, 0, 10, None, None) == -1
