"""Like-for-like step time on one B200: the reference's own fused kernels (``oracle/_ref/fused_adamw``,
its sources compiled unmodified for sm_100a) driven as ``_fused_adamw4bit`` drives them -- one launch per
tensor (lpmm/optim/adamw.py:463-561) -- against this library's one-launch step, on the same
LLaMA-7B-shaped fp32 list and the same buffers.  Not a test (pytest does not collect it); run it as

    python tests/time_reference_kernels_gpu.py [--layers 32] [--iters 10]

The figures in ``profiles/reference_kernels_vs_one_launch_step_7b_list.md`` come from it."""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "low-bit-optimizers_b200"), os.path.join(ROOT, "tests")]

from gpu_helpers import HYPER, llama7b_shapes, load_reference_extension  # noqa: E402

THRESHOLD = 4096


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    import lpmm
    from lpmm import _kernels
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        raise SystemExit("oracle/_ref/fused_adamw is not built (python -c 'import __graft_entry__ as g; g.build()')")
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    shapes = llama7b_shapes(layers=a.layers)
    qm = lpmm.functional.create_general_qmap("nonlinear", 4, True).to(dev)
    qv = lpmm.functional.create_general_qmap("power-1", 4, False).to(dev)
    # the maps sit in the middle of a buffer: the reference's search may read one entry before a map
    buf = torch.zeros(256, device=dev)
    buf[64:80], buf[128:144] = qm, qv
    qm, qv = buf[64:80], buf[128:144]
    entries = []
    for s in shapes:
        p = torch.empty(s, device=dev).normal_(0.0, 0.02)
        g = torch.empty(s, device=dev).normal_(0.0, 1e-3)
        n = p.numel()
        if n > THRESHOLD:
            entries.append((p, g, torch.zeros((n + 1) // 2, dtype=torch.int8, device=dev),
                            torch.zeros((n + 1) // 2, dtype=torch.int8, device=dev),
                            torch.zeros((n + 127) // 128, device=dev), torch.zeros((n + 127) // 128, device=dev)))
        else:
            entries.append((p, g, torch.zeros_like(p), torch.zeros_like(p), None, None))
    total = sum(e[0].numel() for e in entries)
    h = HYPER

    def step_reference(step):
        for p, g, m, v, sm, sv in entries:
            if sm is not None:
                ref.adamw4bit_single_tensor(p, g, m, v, sm, sv, qm, qv, h["beta1"], h["beta2"], h["lr"],
                                            h["weight_decay"], h["eps"], float(step))
            else:
                ref.adamw_single_tensor(p, g, m, v, h["beta1"], h["beta2"], h["lr"], h["weight_decay"], h["eps"],
                                        float(step))

    tl = _kernels.TensorList(entries)

    def step_own(step):
        _kernels.adamw4bit_multi_tensor(tl, qm, qv, h["beta1"], h["beta2"], h["lr"], h["weight_decay"], h["eps"],
                                        float(step))

    for name, fn in (("reference kernels, one launch per tensor", step_reference), ("this library, one launch", step_own)):
        for s in range(1, 4):
            fn(s)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(4, 4 + a.iters):
            fn(s)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        print(f"{name}: {len(entries)} tensors, {total} params, {ms:.3f} ms/step, {total / ms / 1e6:.1f} Gparam/s, "
              f"{total * 14.125 / ms / 1e6:.0f} GB/s of 14.125 B/param", flush=True)


if __name__ == "__main__":
    main()
