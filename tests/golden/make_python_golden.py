"""Generate golden vectors by running the reference's own Python on CPU.

Run in a container that holds the reference checkout:

    python tests/golden/make_python_golden.py [--reference PATH_TO_REFERENCE_CHECKOUT]

The reference package is imported unchanged through ``oracle/ref_loader.py`` (yacs stand-in, CPU
stand-in for its pack/unpack extension).  For every case below the script records the initial
parameters, the gradients of every step, and after the last step the parameters and the complete
optimizer state (packed codes, scales / per-axis maxima, fp32 states), into
``tests/golden/python_<case>.npz``.  Inputs are seeded synthetic data: N(0, 0.02) parameters,
Student-t(3) * 1e-3 gradients with a few rows scaled by 50 and, in the ragged case, 20 % exact
zeros.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)

CASES = {
    # name: (optimizer, kwargs, shapes, steps, zero_fraction)
    "adamw_rank1": ("AdamW", dict(qconfig="default.yml", **HYPER), [(64, 96), (96,)], 4, 0.0),
    "adamw_group": ("AdamW", dict(qconfig=None, **HYPER), [(72, 64), (4097,), (127,)], 4, 0.0),
    "adamw_rank1_ragged": ("AdamW", dict(qconfig="default.yml", **HYPER),
                           [(3, 3, 24, 24), (70, 61), (4097,), (127,), (4096,), (5000, 1)], 5, 0.2),
    "adamw_factored": ("AdamW", dict(qconfig=None, factor_second_moment=True, **HYPER),
                       [(80, 64), (2, 3, 32, 32), (40, 8), (5000,)], 4, 0.0),
    "sgd_momentum": ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-4, qconfig=None), [(72, 64), (4097,), (100,)], 4, 0.0),
    "sgd_nesterov": ("SGD", dict(lr=1e-2, momentum=0.8, dampening=0.0, nesterov=True, weight_decay=0.0, qconfig=None),
                     [(5000,), (6, 700)], 3, 0.0),
    # wider codes (one per byte) and larger first-moment groups
    "adamw_8bit": ("AdamW", dict(qconfig="default_8b.yml", **HYPER), [(72, 64), (4097,), (5000, 1)], 4, 0.0),
    "adamw_5bit": ("AdamW", dict(qconfig="default_5b.yml", **HYPER), [(70, 61), (4100,)], 3, 0.0),
    "adamw_m_group_512": ("AdamW", dict(qconfig="1st_moment_group_512.yml", **HYPER), [(72, 64), (4097,), (9000,)], 4, 0.0),
    "adamw_m_group_4096": ("AdamW", dict(qconfig="1st_moment_group_4096.yml", **HYPER),
                           [(70, 61), (10000,), (5000, 1)], 3, 0.0),
    "sgd_8bit": ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-4, qconfig="default_8b.yml"), [(72, 64), (4097,)], 3, 0.0),
    "sgd_group_1024": ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=0.0, qconfig="1st_moment_group_1024.yml"),
                       [(5000,), (6, 700)], 3, 0.0),
    # first moment kept in fp32, second moment 4-bit (rank-1 / group scales)
    "adamw_2nd_only_rank1": ("AdamW", dict(qconfig="2nd_moment_only_default.yml", **HYPER),
                             [(72, 64), (4097,), (100,), (2, 3, 32, 32)], 4, 0.0),
    "adamw_2nd_only_group": ("AdamW", dict(qconfig="2nd_moment_only_group_128.yml", **HYPER), [(70, 61), (5000,)], 3, 0.0),
    # override_quantize_enable before the first step: tensor 0 (4608 elements) forced to fp32 states, tensor 1
    # (3000 elements, below the threshold) forced to quantized states
    "adamw_override": ("AdamW", dict(qconfig="default.yml", **HYPER), [(72, 64), (3000,), (5000,), (50, 40)], 4, 0.0,
                       [(0, False), (1, True), (3, True)]),
}


def make_params(shapes):
    torch.manual_seed(0)
    return [torch.nn.Parameter(torch.randn(s) * 0.02) for s in shapes]


def make_grad(shape, step, index, zero_fraction):
    g = torch.Generator()
    g.manual_seed(step * 100003 + index)
    z = torch.randn((4,) + tuple(shape), generator=g)
    t = z[0] / torch.sqrt((z[1] ** 2 + z[2] ** 2 + z[3] ** 2) / 3.0) * 1e-3
    if len(shape) >= 2:
        k = max(1, round(0.01 * shape[0]))
        rows = torch.randperm(shape[0], generator=g)[:k]
        t[rows] *= 50.0
    if zero_fraction > 0:
        t[torch.rand(shape, generator=g) < zero_fraction] = 0.0
    return t.contiguous()


def flatten_state(prefix, value, out):
    if isinstance(value, torch.Tensor):
        out[prefix] = value.detach().cpu().numpy()
    elif isinstance(value, dict):
        for k, v in value.items():
            flatten_state(f"{prefix}.{k}", v, out)
    elif isinstance(value, (list, tuple)) and value and isinstance(value[0], torch.Tensor):
        for i, v in enumerate(value):
            out[f"{prefix}.{i}"] = v.detach().cpu().numpy()
    elif isinstance(value, torch.Size):
        out[prefix] = np.array(list(value), dtype=np.int64)
    elif isinstance(value, (bool, int, float)):
        out[prefix] = np.array(value)


def run_case(lpmm, name, ref_root):
    opt_name, kwargs, shapes, steps, zf = CASES[name][:5]
    overrides = CASES[name][5] if len(CASES[name]) > 5 else []
    kwargs = dict(kwargs)
    if isinstance(kwargs.get("qconfig"), str):
        kwargs["qconfig"] = os.path.join(ref_root, "lpmm", "configs", kwargs["qconfig"])
    params = make_params(shapes)
    out = {f"p0.{i}": p.detach().numpy().copy() for i, p in enumerate(params)}
    opt = getattr(lpmm.optim, opt_name)(params, **kwargs)
    holder = torch.nn.Module()
    for i, enable in overrides:  # the reference's API takes (module, attribute name, enable)
        holder.register_parameter(f"p{i}", params[i])
        opt.override_quantize_enable(holder, f"p{i}", enable)
    for step in range(1, steps + 1):
        for i, p in enumerate(params):
            p.grad = make_grad(p.shape, step, i, zf)
            out[f"g{step}.{i}"] = p.grad.numpy().copy()
        opt.step()
    for i, p in enumerate(params):
        out[f"p.{i}"] = p.detach().numpy().copy()
        st = opt.state[p]
        for k, v in st.items():
            if k.endswith("_qstate"):
                flatten_state(f"s.{i}.{k}.overhead", {kk: vv for kk, vv in v["overhead"].items() if kk not in ("dtype", "stride")}, out)
                out[f"s.{i}.{k}.enable"] = np.array(bool(v["enable"]))
            else:
                flatten_state(f"s.{i}.{k}", v, out)
    out["steps"] = np.array(steps)
    np.savez_compressed(os.path.join(HERE, f"python_{name}.npz"), **out)
    return len(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None,
                    help="the reference checkout (default: $LPMM_REFERENCE_ROOT, else ../reference beside this repository)")
    ap.add_argument("--only", nargs="*", default=None, help="generate just these cases (and no map files)")
    a = ap.parse_args()
    from oracle.build_ref import reference_root
    from oracle.ref_loader import load_reference
    a.reference = reference_root(a.reference)
    if a.reference is None:
        raise SystemExit("no reference checkout found (give --reference or set LPMM_REFERENCE_ROOT)")
    cwd = os.getcwd()
    os.chdir("/tmp")  # the reference writes ./lpmm_config.txt on construction
    lpmm = load_reference(a.reference)
    import contextlib, io
    for name in (a.only if a.only else CASES):
        with contextlib.redirect_stdout(io.StringIO()):
            n = run_case(lpmm, name, a.reference)
        print(f"{name}: {n} arrays")
    import lpmm.functional as F
    # the maps of the wider configurations: signed 'nonlinear' and unsigned 'power-1' for 5 ... 8 bits
    wide = {}
    for b in (5, 6, 7, 8):
        wide[f"nonlinear_{b}"] = F.create_general_qmap("nonlinear", b, True).numpy()
        wide[f"power1_{b}"] = F.create_general_qmap("power-1", b, False).numpy()
    np.savez_compressed(os.path.join(HERE, "qmaps_wide.npz"), **wide)
    if a.only:
        os.chdir(cwd)
        return
    # the two quantization maps, as the reference builds them
    np.savez(os.path.join(HERE, "qmaps.npz"), m=F.create_general_qmap("nonlinear", 4, True).numpy(),
             v=F.create_general_qmap("power-1", 4, False).numpy(),
             nonlinear_unsigned=F.create_general_qmap("nonlinear", 4, False).numpy(),
             power2=F.create_general_qmap("power-2", 4, False).numpy(),
             power1_signed=F.create_general_qmap("power-1", 4, True).numpy())
    os.chdir(cwd)


if __name__ == "__main__":
    main()
