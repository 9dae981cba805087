"""Like-for-like step time on one B200: the reference's own fused kernels (``oracle/_ref/fused_adamw``,
its sources compiled unmodified for sm_100a) driven as ``_fused_adamw4bit`` drives them -- one launch per
tensor (lpmm/optim/adamw.py:463-561) -- against this library's one-launch step, on the same
LLaMA-7B-shaped fp32 list and the same buffers.  With ``--nonfused`` instead: the reference's non-fused step (``_single_tensor_adamw4bit``,
lpmm/optim/adamw.py:332-436) as its sequence of torch CUDA operations per parameter (``oracle/torch_ref.py``)
with the reference's compiled ``pack_nonlinear``, against ``lpmm.optim.AdamW`` of this package, on the
GPT-2-medium-shaped list, for the group and the rank-1 second-moment configuration.
As a test (``pytest -m gpu``) it runs both comparisons on reduced lists and requires this library's step to be the
faster one; run as a script it times the full lists:

    python tests/test_gpu_reference_kernels_timing.py [--layers 32] [--iters 10] [--nonfused]

The figures in ``profiles/reference_kernels_vs_one_launch_step_7b_list.md`` come from it."""
import argparse
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "low-bit-optimizers_b200"), os.path.join(ROOT, "tests")]

from gpu_helpers import HYPER, llama7b_shapes, load_reference_extension  # noqa: E402

THRESHOLD = 4096


def gpt2_medium_shapes():
    shapes = [(50257, 1024), (1024, 1024)]
    for _ in range(24):
        shapes += [(1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024)] + [(1024,)] * 4
    return shapes


def nonfused(iters, shapes=None):
    """Returns {v scale: (ms of the reference's operation sequence, ms of this package)}."""
    import lpmm
    from lpmm.config import CONFIG_DIR
    from oracle import torch_ref as T
    quant = load_reference_extension("quantization")
    if quant is None:
        raise SystemExit("oracle/_ref/quantization is not built")
    dev = torch.device("cuda:0")
    shapes = shapes or gpt2_medium_shapes()
    out = {}
    buf = torch.zeros(256, device=dev)
    buf[64:80] = lpmm.functional.create_general_qmap("nonlinear", 4, True).to(dev)
    buf[128:144] = lpmm.functional.create_general_qmap("power-1", 4, False).to(dev)
    qm, qv = buf[64:80], buf[128:144]
    kw = dict(lr=HYPER["lr"], betas=(HYPER["beta1"], HYPER["beta2"]), eps=HYPER["eps"], weight_decay=HYPER["weight_decay"])
    for v_scale, cfg in (("group", None), ("rank1", os.path.join(CONFIG_DIR, "default.yml"))):
        torch.manual_seed(0)
        ps = [torch.empty(s, device=dev).normal_(0.0, 0.02) for s in shapes]
        gs = [torch.empty(s, device=dev).normal_(0.0, 1e-3) for s in shapes]
        total = sum(p.numel() for p in ps)
        states = [dict() for _ in ps]

        def step_reference(step):
            for p, g, st in zip(ps, gs, states):
                q = p.numel() > THRESHOLD
                T.adamw_step(p, g, st, qm, qv, m_quant=q, v_quant=q, v_scale_type=v_scale, beta1=HYPER["beta1"],
                             beta2=HYPER["beta2"], lr=HYPER["lr"], weight_decay=HYPER["weight_decay"], eps=HYPER["eps"],
                             step=float(step), ref_pack=quant.pack_nonlinear)

        params = [torch.nn.Parameter(p.clone()) for p in ps]
        for p, g in zip(params, gs):
            p.grad = g
        opt = lpmm.optim.AdamW(params, qconfig=cfg, **kw)
        for name, fn in ((f"torch-op sequence of the reference + its pack kernel, v {v_scale}", step_reference),
                         (f"lpmm.optim.AdamW of this package, v {v_scale}", lambda s: opt.step())):
            for s in range(1, 4):
                fn(s)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for s in range(4, 4 + iters):
                fn(s)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            print(f"{name}: {len(ps)} tensors, {total} params, {ms:.3f} ms/step, {total / ms / 1e6:.1f} Gparam/s", flush=True)
            out.setdefault(v_scale, []).append(ms)
        del opt, params, states, ps, gs
        torch.cuda.empty_cache()
    return out


def fused(layers, iters):
    """Returns (ms of the reference's kernels launched per tensor, ms of this library's one launch)."""
    import lpmm
    from lpmm import _kernels
    ref = load_reference_extension("fused_adamw")
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    shapes = llama7b_shapes(layers=layers)
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

    res = []
    for name, fn in (("reference kernels, one launch per tensor", step_reference), ("this library, one launch", step_own)):
        for s in range(1, 4):
            fn(s)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(4, 4 + iters):
            fn(s)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        res.append(ms)
        print(f"{name}: {len(entries)} tensors, {total} params, {ms:.3f} ms/step, {total / ms / 1e6:.1f} Gparam/s, "
              f"{total * 14.125 / ms / 1e6:.0f} GB/s of 14.125 B/param", flush=True)
    return tuple(res)


def test_one_launch_step_is_faster_than_the_reference_kernels_per_tensor():
    """Two transformer layers plus embedding and head (667 M parameters), 3 timed steps each."""
    if load_reference_extension("fused_adamw") is None:
        pytest.skip("oracle/_ref was not built")
    ms_ref, ms_own = fused(2, 3)
    assert ms_own < ms_ref


def test_nonfused_step_is_faster_than_the_reference_operation_sequence():
    """Six matrices and vectors of the GPT-2-medium-shaped list, group and rank-1 second moments."""
    if load_reference_extension("quantization") is None:
        pytest.skip("oracle/_ref was not built")
    shapes = [(1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024), (1024,), (1024,)]
    for v_scale, (ms_ref, ms_own) in nonfused(3, shapes).items():
        assert ms_own < ms_ref, v_scale


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--nonfused", action="store_true")
    a = ap.parse_args()
    if a.nonfused:
        return nonfused(a.iters)
    ref = load_reference_extension("fused_adamw")
    if ref is None:
        raise SystemExit("oracle/_ref/fused_adamw is not built (python -c 'import __graft_entry__ as g; g.build()')")
    fused(a.layers, a.iters)


if __name__ == "__main__":
    main()
