"""The C oracle (oracle/lpmm_oracle.c) against golden vectors produced by the reference's own
compiled CUDA kernels on a B200 (tests/golden/fused_golden.npz): bit-exact codes, scales, params."""
import os

import numpy as np
import pytest

from oracle import cpu as O


@pytest.fixture(scope="module")
def G(golden_dir):
    z = np.load(os.path.join(golden_dir, "fused_golden.npz"))
    return {k: z[k] for k in z.files}


def test_quantization_maps_match_reference(qmaps, G):
    assert np.array_equal(G["qmap_m"], qmaps["m"]) and np.array_equal(G["qmap_v"], qmaps["v"])
    assert np.array_equal(qmaps["v"], (np.arange(1, 17) / 16).astype(np.float32))
    assert qmaps["m"][7] == 0.0 and qmaps["m"][15] == 1.0 and qmaps["m"][0] == np.float32(-0.8875)


@pytest.mark.parametrize("step", [1, 2, 3, 4])
def test_fused_4bit_step_matches_reference_kernel(G, step):
    b1, b2, lr, wd, eps = (float(x) for x in G["hyper"])
    pre = {k: G[f"q4.s{step}.pre.{k}"].copy() for k in ("p", "m", "v", "ms", "vs")}
    c = G[f"q4.s{step}.c"]
    O.adamw4bit(pre["p"], G[f"q4.s{step}.g"], pre["m"].view(np.uint8), pre["v"].view(np.uint8), pre["ms"], pre["vs"],
                G["qmap_m"], G["qmap_v"], b1, b2, lr, wd, eps, float(step), c=(float(c[0]), float(c[1])))
    for k in ("m", "v"):
        assert np.array_equal(pre[k].view(np.uint8), G[f"q4.s{step}.post.{k}"].view(np.uint8)), k
    for k in ("ms", "vs", "p"):
        assert np.array_equal(pre[k].view(np.int32), G[f"q4.s{step}.post.{k}"].view(np.int32)), k


@pytest.mark.parametrize("step", [1, 2, 3, 4])
def test_fused_4bit_step_with_host_powf_is_within_tolerance(G, step):
    """With the host's own powf the bias corrections may differ in the last bit: codes and scales
    still match exactly (they do not depend on them), parameters to 1e-6 relative."""
    b1, b2, lr, wd, eps = (float(x) for x in G["hyper"])
    pre = {k: G[f"q4.s{step}.pre.{k}"].copy() for k in ("p", "m", "v", "ms", "vs")}
    O.adamw4bit(pre["p"], G[f"q4.s{step}.g"], pre["m"].view(np.uint8), pre["v"].view(np.uint8), pre["ms"], pre["vs"],
                G["qmap_m"], G["qmap_v"], b1, b2, lr, wd, eps, float(step))
    assert np.array_equal(pre["m"].view(np.uint8), G[f"q4.s{step}.post.m"].view(np.uint8))
    assert np.array_equal(pre["v"].view(np.uint8), G[f"q4.s{step}.post.v"].view(np.uint8))
    ref = G[f"q4.s{step}.post.p"]
    assert np.linalg.norm(pre["p"] - ref) / np.linalg.norm(ref) <= 1e-6


@pytest.mark.parametrize("step", [1, 2, 3, 4])
def test_fused_fp32_step_matches_reference_kernel(G, step):
    b1, b2, lr, wd, eps = (float(x) for x in G["hyper"])
    p, m, v = (G[f"f32.s{step}.pre.{k}"].copy() for k in ("p", "m", "v"))
    c = G[f"q4.s{step}.c"]
    O.adamw_fp32(p, G[f"f32.s{step}.g"], m, v, b1, b2, lr, wd, eps, float(step), c=(float(c[0]), float(c[1])))
    assert np.array_equal(m.view(np.int32), G[f"f32.s{step}.post.m"].view(np.int32))
    assert np.array_equal(v.view(np.int32), G[f"f32.s{step}.post.v"].view(np.int32))
    assert np.array_equal(p.view(np.int32), G[f"f32.s{step}.post.p"].view(np.int32))


def test_code_rule_edges(qmaps):
    q = qmaps["m"]
    mids = (q[:-1] + q[1:]) * np.float32(0.5)
    for i, mid in enumerate(mids):
        assert O.code(q, mid) == i                               # a tie goes to the lower code
        assert O.code(q, np.nextafter(mid, np.float32(2))) == i + 1
        assert O.code(q, np.nextafter(mid, np.float32(-2))) == i
    for i, val in enumerate(q):
        assert O.code(q, val) == i
    assert O.code(q, float("nan")) == 15 and O.code(q, -5.0) == 0 and O.code(q, 5.0) == 15
    qv = qmaps["v"]
    assert O.code(qv, 0.0) == 0 and O.code(qv, 1.0) == 15 and O.code(qv, 3.0 / 32) == 0
    assert O.code(qv, np.nextafter(np.float32(3.0 / 32), np.float32(1))) == 1


def test_pack_unpack_layout(qmaps):
    q = qmaps["m"]
    x = np.array([q[3], q[12], -1.0, 1.0, 0.0, 0.001, 0.2, -0.2], np.float32)
    packed = O.pack4(x.reshape(1, 8), q)
    assert packed.size == 5 and packed[-1] == 0
    assert packed[0] == (3 | (12 << 4))                          # element 2k in the low nibble
    back = O.unpack4(packed, q, 1, 8)
    assert np.array_equal(back[0, :2], np.array([q[3], q[12]], np.float32))
