"""Step times of the secondary paths of the package on a B200: the non-fused AdamW configurations
(rank-1, group, wider codes, larger groups), the factored second moment, momentum SGD per tensor and
fused, next to the fused AdamW step on the same shapes.  Seeded synthetic inputs.

    python benchmarks/paths.py [--iters 10] [--only SUBSTRING] [--big]

One line per case: parameters, CUDA-event time per step (after 3 warm-up steps), wall time per step,
parameters per second.  ``LPMM_SGD_PER_TENSOR=1`` in the environment times the per-tensor SGD launches
instead of the multi-tensor one.  The headline benchmark of the repository is ``bench.py``; this script is
where the figures of ``profiles/unfused_rank1_factored_kernels.md`` come from.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "low-bit-optimizers_b200"))
import lpmm  # noqa: E402
from lpmm.config import CONFIG_DIR  # noqa: E402


def gpt2_medium_shapes():
    shapes = [(50257, 1024), (1024, 1024)]
    for _ in range(24):
        shapes += [(1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024)] + [(1024,)] * 4
    return shapes


def llama7b_shapes(layers=32, hidden=4096, inter=11008, vocab=32000):
    shapes = [(vocab, hidden)]
    for _ in range(layers):
        shapes += [(hidden, hidden)] * 4 + [(inter, hidden), (inter, hidden), (hidden, inter), (hidden,), (hidden,)]
    return shapes + [(hidden,), (vocab, hidden)]


LINEAR = [(4096, 4096), (4096,)]
RAGGED = [(3, 3, 64, 64), (1000, 768), (768, 3072), (4097,), (127,), (4096,), (50000, 1)]


def cfg(name):
    return os.path.join(CONFIG_DIR, name)


def cases():
    adamw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    sgd = dict(lr=1e-2, momentum=0.9, weight_decay=1e-4)
    out = [
        ("linear4096 adamw rank-1 (default.yml)", "AdamW", LINEAR, dict(adamw, qconfig=cfg("default.yml"))),
        ("linear4096 adamw group (qconfig=None)", "AdamW", LINEAR, dict(adamw, qconfig=None)),
        ("linear4096 adamw fused", "AdamW", LINEAR, dict(adamw, fused=True)),
        ("linear4096 adamw fused rank-1 (default.yml, fused_rank1)", "AdamW", LINEAR,
         dict(adamw, qconfig=cfg("default.yml"), fused=True, fused_rank1=True)),
    ]
    for c in ("default_8b.yml", "default_5b.yml", "1st_moment_group_512.yml", "1st_moment_group_4096.yml"):
        out.append((f"linear4096 adamw {c}", "AdamW", LINEAR, dict(adamw, qconfig=cfg(c))))
    out += [
        ("linear4096 sgd", "SGD", LINEAR, dict(sgd)),
        ("gpt2-medium adamw factored", "AdamW", gpt2_medium_shapes(), dict(adamw, factor_second_moment=True)),
        ("gpt2-medium adamw rank-1 (default.yml)", "AdamW", gpt2_medium_shapes(), dict(adamw, qconfig=cfg("default.yml"))),
        ("gpt2-medium adamw group (qconfig=None)", "AdamW", gpt2_medium_shapes(), dict(adamw, qconfig=None)),
        ("gpt2-medium adamw fused", "AdamW", gpt2_medium_shapes(), dict(adamw, fused=True)),
        ("gpt2-medium adamw fused rank-1 (default.yml, fused_rank1)", "AdamW", gpt2_medium_shapes(),
         dict(adamw, qconfig=cfg("default.yml"), fused=True, fused_rank1=True)),
        ("gpt2-medium adamw fused bf16 parameters:", "AdamW", gpt2_medium_shapes(),
         dict(adamw, fused=True, param_dtype=torch.bfloat16)),
        ("gpt2-medium adamw fused bf16 parameters, tolerance mode", "AdamW", gpt2_medium_shapes(),
         dict(adamw, fused=True, exact_params=False, param_dtype=torch.bfloat16)),
        ("gpt2-medium adamw factored, tolerance mode", "AdamW", gpt2_medium_shapes(),
         dict(adamw, factor_second_moment=True, exact_params=False)),
        ("gpt2-medium adamw rank-1 (default.yml), tolerance mode", "AdamW", gpt2_medium_shapes(),
         dict(adamw, qconfig=cfg("default.yml"), exact_params=False)),
        ("gpt2-medium adamw group (qconfig=None), tolerance mode", "AdamW", gpt2_medium_shapes(),
         dict(adamw, qconfig=None, exact_params=False)),
        ("gpt2-medium sgd", "SGD", gpt2_medium_shapes(), dict(sgd)),
        ("ragged adamw rank-1 (default.yml)", "AdamW", RAGGED, dict(adamw, qconfig=cfg("default.yml"))),
    ]
    return out


def big_cases():
    """The LLaMA-7B-shaped list of ``bench.py`` (61 GB of parameters, gradients and states)."""
    adamw = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    return [
        ("llama7b adamw group (qconfig=None)", "AdamW", llama7b_shapes(), dict(adamw, qconfig=None)),
        ("llama7b adamw fused", "AdamW", llama7b_shapes(), dict(adamw, fused=True)),
        ("llama7b adamw fused, tolerance mode (exact_params=False)", "AdamW", llama7b_shapes(),
         dict(adamw, fused=True, exact_params=False)),
        ("llama7b adamw fused bf16 parameters", "AdamW", llama7b_shapes(), dict(adamw, fused=True, param_dtype=torch.bfloat16)),
        ("llama7b adamw fused bf16 parameters, tolerance mode", "AdamW", llama7b_shapes(),
         dict(adamw, fused=True, exact_params=False, param_dtype=torch.bfloat16)),
        ("llama7b adamw rank-1 (default.yml)", "AdamW", llama7b_shapes(), dict(adamw, qconfig=cfg("default.yml"))),
        ("llama7b adamw fused rank-1 (default.yml, fused_rank1)", "AdamW", llama7b_shapes(),
         dict(adamw, qconfig=cfg("default.yml"), fused=True, fused_rank1=True)),
        ("llama7b adamw factored", "AdamW", llama7b_shapes(), dict(adamw, factor_second_moment=True)),
        ("llama7b adamw group (qconfig=None), tolerance mode", "AdamW", llama7b_shapes(),
         dict(adamw, qconfig=None, exact_params=False)),
        ("llama7b adamw rank-1 (default.yml), tolerance mode", "AdamW", llama7b_shapes(),
         dict(adamw, qconfig=cfg("default.yml"), exact_params=False)),
        ("llama7b adamw fused rank-1 (default.yml, fused_rank1), tolerance mode", "AdamW", llama7b_shapes(),
         dict(adamw, qconfig=cfg("default.yml"), fused=True, fused_rank1=True, exact_params=False)),
        ("llama7b adamw factored, tolerance mode", "AdamW", llama7b_shapes(),
         dict(adamw, factor_second_moment=True, exact_params=False)),
        ("llama7b sgd", "SGD", llama7b_shapes(), dict(lr=1e-2, momentum=0.9, weight_decay=1e-4)),
    ]


def run(name, kind, shapes, kw, iters):
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    kw = dict(kw)
    dtype = kw.pop("param_dtype", torch.float32)  # not an optimizer argument: element type of parameters and gradients
    params = [torch.nn.Parameter(torch.empty(s, device=dev).normal_(0.0, 0.02).to(dtype)) for s in shapes]
    for p in params:
        p.grad = torch.empty(p.shape, device=dev).normal_(0.0, 1e-3).to(dtype)
    opt = getattr(lpmm.optim, kind)(params, **kw)
    for _ in range(3):
        opt.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for _ in range(iters):
        opt.step()
    b.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / iters * 1e3
    ms = a.elapsed_time(b) / iters
    n = sum(p.numel() for p in params)
    print(f"{name}: {n} params, {ms:.3f} ms/step (wall {wall:.3f}), {n / ms / 1e6:.1f} Gparam/s", flush=True)


def copy_rate(seconds=3.0):
    """Context for the roofline fractions: torch's device-to-device copy (the kind of kernel the measured
    peak comes from) as a burst of 10 and sustained for a few seconds under the power cap."""
    dev = torch.device("cuda:0")
    n = 1 << 30
    src = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_()
    dst = torch.empty_like(src)
    nbytes = 2.0 * n * 2
    for label, iters in (("burst of 10", 10), (f"sustained, ~{seconds:.0f} s", int(seconds / (nbytes / 6.0e12)))):
        for _ in range(3):
            dst.copy_(src)
        torch.cuda.synchronize()
        if label.startswith("burst"):
            time.sleep(1.0)  # let the clocks recover
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            dst.copy_(src)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        print(f"copy_ of {n} bf16 elements ({label}, {iters} copies): {ms:.3f} ms, {nbytes / ms / 1e6:.0f} GB/s", flush=True)


def pack_rate(n=1 << 28, iters=10):
    """The standalone 4-bit pack / unpack of ``lpmm.cpp_extension.quantization`` on n normalised values (4.5 bytes
    moved per value: 4 read + 0.5 written, or the reverse), next to the copy rate above."""
    from lpmm.cpp_extension import quantization as Q
    from lpmm.functional import create_general_qmap
    dev = torch.device("cuda:0")
    qmap = create_general_qmap("nonlinear", 4, True).to(dev)
    x = (torch.rand(n // 2048, 2048, device=dev) * 2 - 1).contiguous()
    packed = Q.pack_nonlinear(x, qmap, 4, False)
    for label, fn in (("pack_nonlinear", lambda: Q.pack_nonlinear(x, qmap, 4, False)),
                      ("unpack_nonlinear", lambda: Q.unpack_nonlinear(packed, qmap, 4, n // 2048, 2048))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        print(f"{label} of {n} values (incl. the output allocation): {ms:.3f} ms, {4.5 * n / ms / 1e6:.0f} GB/s", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default=None)
    ap.add_argument("--big", action="store_true", help="the LLaMA-7B-shaped list instead (needs ~70 GB)")
    ap.add_argument("--copy", action="store_true", help="time torch's device copy instead (burst and sustained)")
    ap.add_argument("--pack", action="store_true", help="time the standalone 4-bit pack / unpack of 2^28 values instead")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    if a.copy:
        return copy_rate()
    if a.pack:
        return pack_rate()
    for name, kind, shapes, kw in (big_cases() if a.big else cases()):
        if a.only is None or a.only in name:
            run(name, kind, shapes, kw, a.iters)
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
