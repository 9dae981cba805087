"""Generate golden vectors of the FUSED step by running the reference's own compiled CUDA kernels.

Needs a GPU and ``oracle/_ref`` (``python oracle/build_ref.py`` in a container that holds the
reference checkout).  Run on the GPU box:

    python tests/golden/make_fused_golden.py [output_dir]

Writes ``fused_golden.npz``: for four consecutive steps of ``adamw4bit_single_tensor`` on a ragged
tensor (128*37 + 70 elements, so the last group is partial) and of ``adamw_single_tensor`` on a
1000-element tensor: the gradient, the state before and after the step, and the two bias
corrections the device computed (so a CPU model can be fed the device's powf).  Step 3 zeroes the
gradient of the first third of the tensor and step >= 3 of one whole group.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "low-bit-optimizers_b200"))

from gpu_helpers import HYPER, device, device_qmaps, fused_state, load_reference_extension, stream, student_t, vp  # noqa: E402


def main(out_dir):
    from lpmm import _native as N
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        raise SystemExit("oracle/_ref/fused_adamw is missing")
    z = np.load(os.path.join(HERE, "qmaps.npz"))
    qmaps = {k: z[k] for k in z.files}
    qm, qv, _ = device_qmaps(qmaps)
    h = HYPER
    out = {"qmap_m": qmaps["m"], "qmap_v": qmaps["v"],
           "hyper": np.array([h["beta1"], h["beta2"], h["lr"], h["weight_decay"], h["eps"]], np.float64)}
    n = 128 * 37 + 70
    torch.manual_seed(n)
    p = torch.randn(n, device=device()) * 0.02
    st = fused_state(n)
    cdev = torch.zeros(2, device=device())
    for step in range(1, 5):
        g = student_t((n,), 1000 + step)
        if step == 3:
            g[: n // 3] = 0.0
        if step >= 3:
            g[128 * 20:128 * 21] = 0.0
        N.check(N.lib.lpmm_b200_bias_corrections(h["beta1"], h["beta2"], float(step), vp(cdev), stream()))
        torch.cuda.synchronize()
        out[f"q4.s{step}.c"] = cdev.cpu().numpy().copy()
        out[f"q4.s{step}.g"] = g.cpu().numpy()
        out[f"q4.s{step}.pre.p"] = p.cpu().numpy()
        for nm, t in zip(("m", "v", "ms", "vs"), st):
            out[f"q4.s{step}.pre.{nm}"] = t.cpu().numpy()
        ref.adamw4bit_single_tensor(p, g, st[0], st[1], st[2], st[3], qm, qv, h["beta1"], h["beta2"], h["lr"],
                                    h["weight_decay"], h["eps"], float(step))
        torch.cuda.synchronize()
        out[f"q4.s{step}.post.p"] = p.cpu().numpy()
        for nm, t in zip(("m", "v", "ms", "vs"), st):
            out[f"q4.s{step}.post.{nm}"] = t.cpu().numpy()
    n = 1000
    torch.manual_seed(n)
    p = torch.randn(n, device=device()) * 0.02
    m, v = torch.zeros(n, device=device()), torch.zeros(n, device=device())
    for step in range(1, 5):
        g = student_t((n,), 2000 + step)
        out[f"f32.s{step}.g"] = g.cpu().numpy()
        out[f"f32.s{step}.pre.p"], out[f"f32.s{step}.pre.m"], out[f"f32.s{step}.pre.v"] = (
            p.cpu().numpy(), m.cpu().numpy(), v.cpu().numpy())
        ref.adamw_single_tensor(p, g, m, v, h["beta1"], h["beta2"], h["lr"], h["weight_decay"], h["eps"], float(step))
        torch.cuda.synchronize()
        out[f"f32.s{step}.post.p"], out[f"f32.s{step}.post.m"], out[f"f32.s{step}.post.v"] = (
            p.cpu().numpy(), m.cpu().numpy(), v.cpu().numpy())
    path = os.path.join(out_dir, "fused_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
