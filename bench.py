"""Benchmark of the fused 4-bit AdamW step on a LLaMA-7B-shaped fp32 parameter list.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl own|reference] [--layers L]

Prints ONE JSON line.  The workload is the 7B configuration of the 4-bit optimizer's headline
metric: a 32000x4096 embedding, 32 layers of q/k/v/o 4096x4096, gate/up 11008x4096, down
4096x11008 and two 4096 norm vectors, and a 32000x4096 head; about 6.74e9 fp32 parameters, of
which the 64 norm vectors (exactly 4096 elements) keep fp32 moments.  Data are synthetic: N(0,
0.02) parameters and Student-t(3) * 1e-3 gradients with 1 % of rows scaled by 50, seeded.

own arm      one step = ``lpmm.optim.AdamW(fused=True).step()`` over the whole list (one multi-tensor
             launch).  ``value`` is timed with parameters, gradients and states resident in HBM;
             ``e2e`` is the step with its gradients arriving from pinned host memory (``step_from_host``:
             copies on a copy stream, every chunk updated as it lands) and a device->host read of a result
             inside the timed region; ``copy_then_step_ms`` is the plain sequence timed beside it.  ``tolerance_mode``: the same
             step with ``exact_params=False`` (codes and scales bit-identical, parameters within 1e-6).
             With N > 1 the list is ZeRO-1 sharded by whole 128-element groups (``lpmm.zero``); the updated
             parameters reach the other ranks by copy-engine peer copies of every updated 1-2 GB range while the
             next range is updated (``--gather copy``, the default: the fastest of the three here), by NVLink
             stores inside the update kernel (``--gather fused``, timed beside it as ``gather_fused``) or by an
             NCCL all-gather after the update (``--gather nccl``).  The whole step is timed
             (``"scaling": "strong"``: the list is fixed, the ranks share it); extra keys give the check that
             the sharded step equals the unsharded one (``zero1_check``), the update alone per GPU
             (``local_update``), the same list with bf16 parameters (``params_bf16``) and the
             LLaMA-13B-shaped list (``llama13b``).
reference    the reference's own Python CPU path (``lpmm.optim.AdamW`` unchanged, group-128 4-bit states, its
arm          CUDA pack/unpack extension replaced by a C restatement) with all host threads on a bounded
             sample of the same list, rank 0 only; the C port of the fused kernel when that Python is absent.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "low-bit-optimizers_b200"))

HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
METRIC = "optimizer_params_updated_per_second"
UNIT = "params/s"
BYTES_Q4 = 14.125   # p 4r+4w, g 4r, m codes .5r+.5w, v codes .5r+.5w, two fp32 scales per 128 elements r+w
BYTES_FP32 = 28.0   # p, m, v read+write, g read
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of adamw4bit_multi_kernel<1,1,0> over a 667 M-parameter
# list (ncu, one launch captured), divided by its 4-bit parameters: every byte moves once, so a launch over a longer
# list moves proportionally more
NCU_TRAFFIC_PER_PARAM = 14.23


def llama7b_shapes(layers=32, hidden=4096, inter=11008, vocab=32000):
    shapes = [(vocab, hidden)]
    for _ in range(layers):
        shapes += [(hidden, hidden)] * 4 + [(inter, hidden)] * 2 + [(hidden, inter)] + [(hidden,)] * 2
    shapes += [(vocab, hidden)]
    return shapes


def numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


def algorithmic_bytes(shapes):
    nq = sum(numel(s) for s in shapes if numel(s) > 4096)
    nf = sum(numel(s) for s in shapes if numel(s) <= 4096)
    return nq * BYTES_Q4 + nf * BYTES_FP32, nq, nf


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.first = index, None, [], 0

    def mark(self):
        """Samples from here on count (called when the timed region starts; the process was started
        earlier, because nvidia-smi needs up to a second before its first line)."""
        self.first = len(self.lines)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                          "100", "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines[self.first:]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return None
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def student_t_(out, seed, rows_outliers=True):
    """Fill ``out`` with Student-t(3) * 1e-3; 1 % of rows (>= 2-D) scaled by 50."""
    import torch
    g = torch.Generator(device=out.device)
    g.manual_seed(seed)
    flat = out.view(-1)
    chunk = 1 << 26
    for lo in range(0, flat.numel(), chunk):
        hi = min(lo + chunk, flat.numel())
        z = torch.randn((4, hi - lo), generator=g, device=out.device)
        flat[lo:hi] = z[0] / torch.sqrt((z[1] ** 2 + z[2] ** 2 + z[3] ** 2) / 3.0) * 1e-3
        del z
    if rows_outliers and out.dim() >= 2:
        k = max(1, round(0.01 * out.shape[0]))
        rows = torch.randperm(out.shape[0], generator=g, device=out.device)[:k]
        out[rows] *= 50.0


# --------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own Python CPU path (or, without it, the C port) on a
# bounded sample of the list
# --------------------------------------------------------------------------------------------------
def cpu_sample_shapes():
    """One transformer layer of the list: 202 383 360 parameters (the sample of the C port)."""
    return llama7b_shapes()[1:10]


def python_sample_shapes():
    """The sample of the reference's Python path, which is an order of magnitude slower than the C port: one
    attention projection, one MLP projection and one norm vector of a layer, 61 870 080 parameters."""
    return [(4096, 4096), (11008, 4096), (4096,)]


def host_threads():
    """Every host thread this process may run on (torchrun exports OMP_NUM_THREADS=1: not that)."""
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def time_cpu_oracle(steps, warmup, sample_shapes, threads=None):
    import numpy as np
    from oracle import cpu as O
    z = np.load(os.path.join(ROOT, "tests", "golden", "qmaps.npz"))
    qm, qv = z["m"], z["v"]
    O.set_threads(threads or host_threads())
    rng = np.random.default_rng(0)
    tensors = []
    for s in sample_shapes:
        n = numel(s)
        p = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02))
        g = (rng.standard_t(3, n).astype(np.float32) * np.float32(1e-3))
        if n > 4096:
            st = (np.zeros((n + 1) // 2, np.uint8), np.zeros((n + 1) // 2, np.uint8), np.zeros((n + 127) // 128, np.float32),
                  np.zeros((n + 127) // 128, np.float32))
        else:
            st = (np.zeros(n, np.float32), np.zeros(n, np.float32))
        tensors.append((p, g, st))
    b1, b2 = HYPER["betas"]
    times = []
    for it in range(1, warmup + steps + 1):
        t0 = time.perf_counter()
        for p, g, st in tensors:
            if len(st) == 4:
                O.adamw4bit(p, g, st[0], st[1], st[2], st[3], qm, qv, b1, b2, HYPER["lr"], HYPER["weight_decay"], HYPER["eps"],
                            float(it))
            else:
                O.adamw_fp32(p, g, st[0], st[1], b1, b2, HYPER["lr"], HYPER["weight_decay"], HYPER["eps"], float(it))
        dt = time.perf_counter() - t0
        if it > warmup:
            times.append(dt)
    total = sum(numel(s) for s in sample_shapes)
    sec = sum(times) / len(times)
    return total / sec, sec, O.threads(), total


def reference_python_root():
    """Where the reference's own Python layer can be imported from on this machine: the copy that
    ``oracle/build_ref.py`` leaves under the git-ignored ``oracle/_ref/lpmm_py`` (it travels with the tree), else
    a reference checkout.  None: not available."""
    from oracle import build_ref
    if build_ref.have_python():
        return build_ref.PY_OUT
    return build_ref.reference_root()


def time_reference_python(steps, warmup, sample_shapes, ref_root, threads=None):
    """The reference's own ``lpmm.optim.AdamW`` (its Python, unchanged) on CPU tensors: ``qconfig=None``, i.e. both
    moments 4-bit with group-128 scales like the fused step, non-fused arithmetic (the reference has no CPU form
    of its fused kernel).  Its CUDA pack / unpack extension is replaced by the C oracle's CPU restatement of those
    two functions (``oracle/ref_loader.py``); everything else is the reference's torch code on the host cores.
    Must run in a process that has not imported this repository's package of the same name."""
    import contextlib
    import io
    import tempfile
    import torch
    from oracle import cpu as O
    from oracle.ref_loader import load_reference
    threads = threads or host_threads()
    torch.set_num_threads(threads)
    O.set_threads(threads)
    cwd = os.getcwd()
    os.chdir(tempfile.mkdtemp())  # the reference writes ./lpmm_config.txt on construction
    try:
        ref = load_reference(ref_root)
        torch.manual_seed(0)
        params = [torch.nn.Parameter(torch.empty(s).normal_(0, 0.02)) for s in sample_shapes]
        gen = torch.Generator().manual_seed(1)
        for p in params:
            z = torch.randn((4,) + tuple(p.shape), generator=gen)
            p.grad = z[0] / torch.sqrt((z[1] ** 2 + z[2] ** 2 + z[3] ** 2) / 3.0) * 1e-3
            del z
        with contextlib.redirect_stdout(io.StringIO()):
            opt = ref.optim.AdamW(params, qconfig=None, fused=False, **HYPER)
        times = []
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            opt.step()
            dt = time.perf_counter() - t0
            if it >= warmup:
                times.append(dt)
    finally:
        os.chdir(cwd)
    total = sum(numel(s) for s in sample_shapes)
    sec = sum(times) / len(times)
    return total / sec, sec, threads, total


def reference_measurement(steps, warmup):
    """(value, seconds per step, cpu_baseline dict): the reference's Python when it is importable here, else the
    C port."""
    root = reference_python_root()
    if root is not None:
        value, sec, threads, total = time_reference_python(steps, warmup, python_sample_shapes(), root)
        desc = (f"a 4096x4096 and an 11008x4096 projection and a 4096 norm vector of the list ({total} params) per step; the "
                f"reference's own Python (lpmm.optim.AdamW, qconfig=None, fused=False) on CPU tensors, torch with {threads} "
                f"threads, its CUDA pack/unpack extension replaced by a C restatement of those two functions")
        kind = "reference-python"
    else:
        value, sec, threads, total = time_cpu_oracle(steps, warmup, cpu_sample_shapes())
        desc = f"one transformer layer of the list ({total} params) per step, C restatement of the reference kernel, OpenMP"
        kind = "port"
    return value, sec, {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": desc}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, sec, cpu = reference_measurement(args.steps, args.warmup)
    if cpu["kind"] == "reference-python" and not args.no_port:
        # the faster C port of the fused kernel beside it, for scale
        v2, _, th2, tot2 = time_cpu_oracle(2, 1, cpu_sample_shapes())
        cpu["c_port_of_the_fused_kernel"] = {"value": v2, "unit": UNIT, "cores": th2, "kind": "port",
                                             "sample": f"one transformer layer ({tot2} params), OpenMP"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "llama7b_shaped_fp32_list_fused_4bit_adamw", "sample": cpu["sample"]},
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def cpu_baseline_in_subprocess(steps=2, warmup=1):
    """The ``cpu_baseline`` leg of the own arm: the reference's package has the same name as this repository's, so
    it is timed in a child process (``bench.py --impl reference``) and its JSON line is read back."""
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    env.pop("OMP_NUM_THREADS", None)
    res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", str(steps), "--warmup",
                          str(warmup)], capture_output=True, text=True, env=env, timeout=900)
    for line in reversed(res.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)["cpu_baseline"]
    raise RuntimeError("the reference arm printed no JSON line: " + res.stderr[-500:])


# --------------------------------------------------------------------------------------------------
# own arm
# --------------------------------------------------------------------------------------------------
CHECK_SHAPES = [(300, 128), (4096,), (5000,), (77, 129), (128,), (64, 64, 3), (2048, 1024)]


def zero1_check(opt, world, rank, dev, gather):
    """Is the sharded step right?  (1) After the timed steps every rank's copy of the whole parameter buffer has the
    same 64-bit checksum.  (2) A small list (4-bit tensors, fp32-state tensors, ragged sizes) is stepped three times
    both ZeRO-1 sharded over all ranks (same gather mode) and unsharded by ``lpmm.optim.AdamW(fused=True)`` on every
    rank, on the same seeded gradients: the parameters must be equal bit for bit on every rank."""
    import torch
    import torch.distributed as dist
    import lpmm
    from lpmm.zero import Zero1FusedAdamW
    c = opt.flat_checksum().reshape(1)
    lo, hi = c.clone(), c.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    same_sum = bool((lo == hi).item())
    z = Zero1FusedAdamW(CHECK_SHAPES, dev, gather=gather, **HYPER)
    z.init_params_normal_(0.02, seed=0)
    plain = [torch.nn.Parameter(v.detach().clone()) for v in z.params]
    po = lpmm.optim.AdamW(plain, fused=True, **HYPER)
    for step in range(1, 4):
        grads = []
        for i, sh in enumerate(CHECK_SHAPES):
            g = torch.empty(sh, device=dev)
            student_t_(g, step * 100003 + i)
            grads.append(g)
        z.set_grad_shard_from_full(grads)
        z.step()
        for p, g in zip(plain, grads):
            p.grad = g
        po.step()
    torch.cuda.synchronize()
    equal = all(bool(torch.equal(v.view(torch.int32), p.detach().view(torch.int32))) for v, p in zip(z.params, plain))
    flag = torch.tensor([1 if equal else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if same_sum and int(flag.item()) == 1:
        return "ok"
    return ("MISMATCH:" + ("" if same_sum else " the ranks' parameter buffers differ after the timed steps;")
            + ("" if int(flag.item()) == 1 else " sharded != unsharded on the small list"))


def local_update_rate(opt, iters, peak, world):
    """The update alone on each GPU's own shard, without the stores into the peers (what scales with the number of
    GPUs; it leaves the replicas inconsistent, so it runs after the check).  Max over ranks."""
    import torch
    import torch.distributed as dist
    ms, nbytes = opt.time_update_only(iters, peers=False)
    t = torch.tensor([ms], device=opt.device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    n_own = (opt.hi - opt.lo) * 128
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"ms": ms, "params_per_s_per_gpu": n_own / (ms * 1e-3), "aggregate_params_per_s": n_own * world / (ms * 1e-3),
            "hbm_gb_per_s_per_gpu": gbs, "frac_of_measured_hbm_peak": gbs / peak}


def sharded_step_line(shapes, dev, gather, dtype, iters, world, replica_dtype=None):
    """Whole sharded step (update + exchange) of another list / element type, timed like the headline: max over ranks.
    ``replica_dtype``: fp32 master parameters kept per shard, 16-bit replicas published to the peers."""
    import torch
    import torch.distributed as dist
    from lpmm.zero import Zero1FusedAdamW
    z = Zero1FusedAdamW(shapes, dev, gather=gather, dtype=dtype, replica_dtype=replica_dtype, **HYPER)
    z.init_params_normal_(0.02, seed=0)
    tmp = torch.empty(min(z.grad_shard.numel(), 1 << 26), device=dev)
    student_t_(tmp, 100003 + dist.get_rank(), rows_outliers=False)
    for lo in range(0, z.grad_shard.numel(), tmp.numel()):
        hi = min(lo + tmp.numel(), z.grad_shard.numel())
        z.grad_shard[lo:hi].copy_(tmp[: hi - lo])
    del tmp
    for _ in range(3):
        z.step()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        z.step()
    b.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    total = sum(numel(s) for s in shapes)
    sent = float(z.xsize) * z.shard_groups * 128 * (world - 1)
    out = {"params": total, "dtype": str(dtype).replace("torch.", "") + (
               "" if replica_dtype is None else " master, " + str(replica_dtype).replace("torch.", "") + " replicas"),
           "ms_per_step": ms, "value": total / (ms * 1e-3), "unit": UNIT,
           "steps": iters, "nvlink_bytes_sent_per_rank_per_step": sent, "nvlink_gb_per_s_per_rank": sent / (ms * 1e-3) / 1e9}
    del z
    torch.cuda.empty_cache()
    return out


def run_own(args):
    import torch
    import torch.distributed as dist
    import lpmm
    from lpmm import _kernels

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU implementation of the step")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_layers = args.layers
    if args.model == "13b":  # the ZeRO-1 configuration of the benchmark description: 40 layers, hidden 5120, inter 13824
        n_layers = 40 if args.layers == 32 else args.layers
        shapes = llama7b_shapes(layers=n_layers, hidden=5120, inter=13824)
    else:
        shapes = llama7b_shapes(layers=args.layers)
    total = sum(numel(s) for s in shapes)
    alg_bytes, nq, nf = algorithmic_bytes(shapes)
    launches = [0]
    real_multi = _kernels.adamw4bit_multi_tensor

    def counting_multi(tl, *a, **k):
        launches[0] += (tl.n + 399) // 400
        return real_multi(tl, *a, **k)

    _kernels.adamw4bit_multi_tensor = counting_multi

    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    sampler = ClockSampler(visible.split(",")[local_rank] if visible else local_rank)
    extra = {}
    if world == 1:
        torch.manual_seed(0)
        params = [torch.nn.Parameter(torch.empty(s, device=dev).normal_(0, 0.02)) for s in shapes]
        gflat = torch.empty(total, device=dev)  # the gradients are views of one buffer (the e2e copies are few and large)
        off = 0
        for i, p in enumerate(params):
            p.grad = gflat[off:off + p.numel()].view(p.shape)
            off += p.numel()
            student_t_(p.grad, 100003 + i)
        opt = lpmm.optim.AdamW(params, fused=True, **HYPER)

        def step():
            opt.step()
    else:
        from lpmm.zero import Zero1FusedAdamW
        torch.manual_seed(0)
        opt = Zero1FusedAdamW(shapes, dev, gather=args.gather, reduce_grads=args.reduce_grads, **HYPER)
        opt.init_params_normal_(0.02, seed=0)
        if args.reduce_grads:  # every rank's own full gradients; the step sums them over the ranks
            chunk = 1 << 26
            for lo_ in range(0, opt.grad_flat.numel(), chunk):
                student_t_(opt.grad_flat[lo_: lo_ + chunk], 100003 + 977 * rank + lo_ // chunk, rows_outliers=False)
        else:
            student_t_(opt.grad_shard.view(-1), 100003 + rank, rows_outliers=False)

        from lpmm.zero import copy_chunk_bytes
        shard_bytes, chunk_bytes = 4 * (opt.hi - opt.lo) * 128, copy_chunk_bytes(world)
        # gather="copy": a first range of an eighth of the chunk, then full ones
        ranges_per_step = (1 + -(-max(shard_bytes - chunk_bytes // 8, 0) // chunk_bytes)) if args.gather == "copy" else 1

        def step():
            opt.step()
            launches[0] += ranges_per_step * ((len(shapes) + 399) // 400)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    sampler.mark()
    launches[0] = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = []  # one event after every step: a step is one launch of the multi-tensor kernel (N = 1)
    e0.record()
    for _ in range(args.steps):
        step()
        if world == 1:
            marks.append(torch.cuda.Event(enable_timing=True))
            marks[-1].record()
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    n_launch = launches[0]
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = total / (ms_per_step * 1e-3)

    # dominant kernel: the launches of the timed region itself, each measured from the end of the launch before it
    # to its own end (the queue never runs dry, so that is the launch's duration)
    if world == 1:
        ks = [a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks)]
        k_ms = sum(ks) / len(ks)
        k_bytes = alg_bytes
    else:
        k_ms, k_bytes = opt.time_update_only(max(3, min(args.steps, 10)), peers=args.gather != "copy")
        extra.update(opt.breakdown(max(3, min(args.steps, 10))))
    peak, peak_kind = measured_peak()
    if world > 1:
        extra["zero1_check"] = zero1_check(opt, world, rank, dev, args.gather)
        extra["local_update"] = local_update_rate(opt, max(3, min(args.steps, 10)), peak, world)
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_PER_PARAM * (k_bytes / BYTES_Q4),
                "traffic_source": "ncu capture of this kernel on a 667 M-parameter list (14.23 B per 4-bit parameter), "
                                  "scaled by the parameters of this launch",
                "peak_kind": f"of {peak_kind}",
                "kernel": "adamw4bit_multi_kernel", "algorithmic_bytes_per_launch": k_bytes, "launch_ms": k_ms}
    if world == 1:
        roofline["launch_ms_min_max"] = [min(ks), max(ks)]
        # the tolerance mode of the same step (moments, scales and codes bit-identical; parameters within 1e-6
        # relative): same list, same states continued, timed the same way
        opt._exact_params = False
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        tm = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        tm[0].record()
        for i in range(args.steps):
            step()
            tm[i + 1].record()
        torch.cuda.synchronize()
        opt._exact_params = True
        tks = [a.elapsed_time(b) for a, b in zip(tm[:-1], tm[1:])]
        t_ms = sum(tks) / len(tks)
        t_ach = alg_bytes / (t_ms * 1e-3) / 1e9
        extra["tolerance_mode"] = {
            "what": "AdamW(fused=True, exact_params=False): codes and scales bit-identical, parameters within 1e-6 relative",
            "ms_per_step": t_ms, "value": total / (t_ms * 1e-3), "unit": UNIT,
            "roofline": {"bound": "hbm", "achieved": t_ach, "peak": peak, "unit": "GB/s", "frac": t_ach / peak,
                         "peak_kind": f"of {peak_kind}", "launch_ms": t_ms, "launch_ms_min_max": [min(tks), max(tks)],
                         "frac_of_nominal_8000": t_ach / 8000.0}}
        roofline["frac_of_nominal_8000"] = achieved / 8000.0
    if world > 1 and args.gather == "copy":
        # update kernel on ranges of the shard, each range then copied to every peer by the copy engines while the next
        # is updated: the step is bound by the bytes a rank must receive over NVLink; the kernel itself is `local_update`
        link_bytes = 4.0 * opt.shard_groups * 128 * (world - 1)
        link_peak = 770.0
        t_hbm, t_link = k_bytes / (peak * 1e9), link_bytes / (link_peak * 1e9)
        roofline = {"bound": "nvlink" if t_link >= t_hbm else "hbm", "achieved": link_bytes / (ms_per_step * 1e-3) / 1e9,
                    "peak": link_peak, "unit": "GB/s", "frac": max(t_hbm, t_link) / (ms_per_step * 1e-3), "traffic": None,
                    "peak_kind": "measured peer-copy rate of this pool (770 GB/s per direction); HBM side of measured",
                    "kernel": "adamw4bit_multi_kernel on 1-2 GB ranges + copy-engine peer copies of each finished range",
                    "launch_ms": k_ms, "step_ms": ms_per_step, "algorithmic_bytes_per_launch": k_bytes,
                    "nvlink_bytes_sent_per_rank_per_step": link_bytes,
                    "nvlink_bytes_received_per_rank_per_step": link_bytes, "target_ms": max(t_hbm, t_link) * 1e3}
    if world > 1 and args.gather == "fused":
        # fused update + peer stores: the target time is the slower of HBM and NVLink; this kernel is NVLink-bound
        link_bytes = 4.0 * opt.shard_groups * 128 * (world - 1)      # sent (and received) per rank per launch
        link_peak = 770.0                                            # GB/s per direction, measured peer copy on this pool
        # with the gradient reduction in the kernel a rank also RECEIVES its shard's gradients from every peer, on
        # the same direction of its links as the peers' parameter stores: that direction carries twice the bytes
        link_busiest = link_bytes * (2.0 if args.reduce_grads else 1.0)
        t_hbm, t_link = k_bytes / (peak * 1e9), link_busiest / (link_peak * 1e9)
        roofline = {"bound": "nvlink" if t_link >= t_hbm else "hbm", "achieved": link_busiest / (k_ms * 1e-3) / 1e9,
                    "peak": link_peak, "unit": "GB/s", "frac": max(t_hbm, t_link) / (k_ms * 1e-3), "traffic": None,
                    "peak_kind": "measured peer-copy rate of this pool (770 GB/s per direction); HBM side of measured",
                    "kernel": "adamw4bit_multi_kernel (update + stores to all peers)", "launch_ms": k_ms,
                    "algorithmic_bytes_per_launch": k_bytes, "nvlink_bytes_sent_per_rank_per_launch": link_bytes,
                    "nvlink_bytes_received_per_rank_per_launch": link_busiest, "target_ms": max(t_hbm, t_link) * 1e3}

    # end to end through the public API with the gradients coming from pinned host memory
    e2e = None
    if world == 1:
        pool_n = min(1 << 29, max(numel(s) for s in shapes) * 2)
        pool = torch.empty(pool_n, dtype=torch.float32, pin_memory=True)
        tmp = torch.empty(min(pool_n, 1 << 26), device=dev)
        student_t_(tmp, 7, rows_outliers=False)
        for lo in range(0, pool_n, tmp.numel()):
            hi = min(lo + tmp.numel(), pool_n)
            pool[lo:hi].copy_(tmp[: hi - lo])
        del tmp
        result = torch.empty(1024, dtype=torch.float32, pin_memory=True)

        # the step's gradients arrive from pinned host memory, 4 * total bytes per step (the pinned pool is the source
        # of every tensor's copy).  ``AdamW.step_from_host`` copies them on a copy stream and updates every 256 MB that
        # has landed while the rest is still on its way; the plain way (copy everything, then step) is timed beside it.
        host_grads = [pool[: numel(s)] for s in shapes]

        def e2e_step():
            opt.step_from_host(host_grads)
            result.copy_(params[-1].detach().view(-1)[:1024], non_blocking=True)

        def e2e_plain_step():
            for lo in range(0, total, pool_n):
                hi = min(lo + pool_n, total)
                gflat[lo:hi].copy_(pool[: hi - lo], non_blocking=True)
            opt.step()
            result.copy_(params[-1].detach().view(-1)[:1024], non_blocking=True)

        def time_e2e(fn, n):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n

        n_e2e = max(2, min(args.steps, 5))
        plain_ms = time_e2e(e2e_plain_step, 2)
        e_ms = time_e2e(e2e_step, n_e2e)
        e2e = {"value": total / (e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 4 * total, "d2h_bytes_per_step": 4096,
               "ms_per_step": e_ms, "steps": n_e2e, "call": "AdamW.step_from_host (copies and update overlapped)",
               "copy_then_step_ms": plain_ms}
    elif args.reduce_grads:
        e2e = None  # the gradients are produced on each GPU (data-parallel backward); no host copy belongs to this mode
    else:
        # each rank's gradient shard arrives from pinned host memory every step
        n_sh = opt.grad_shard.numel()
        pool = torch.empty(n_sh, dtype=torch.float32, pin_memory=True)
        pool.copy_(opt.grad_shard)
        result = torch.empty(1024, dtype=torch.float32, pin_memory=True)

        def e2e_step():
            opt.step_from_host(pool)
            result.copy_(opt.flat[:1024], non_blocking=True)

        def e2e_plain_step():
            opt.grad_shard.copy_(pool, non_blocking=True)
            opt.step()
            result.copy_(opt.flat[:1024], non_blocking=True)

        def time_e2e(fn, n):
            for _ in range(2):
                fn()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record()
            barrier()
            t = torch.tensor([a.elapsed_time(b) / n], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        n_e2e = max(2, min(args.steps, 5))
        plain_ms = time_e2e(e2e_plain_step, 2)
        e_ms = time_e2e(e2e_step, n_e2e)
        owned = torch.tensor([(opt.hi - opt.lo) * 128 * 4], device=dev, dtype=torch.float64)
        dist.all_reduce(owned)
        e2e = {"value": total / (e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(owned.item()),
               "d2h_bytes_per_step": 4096 * world, "ms_per_step": e_ms, "steps": n_e2e,
               "call": "Zero1FusedAdamW.step_from_host (copies and update overlapped)", "copy_then_step_ms": plain_ms}

    if world > 1 and not args.no_extras and not args.reduce_grads:
        del opt
        torch.cuda.empty_cache()
        n_x = max(3, min(args.steps, 10))
        try:
            extra["params_bf16"] = sharded_step_line(shapes, dev, args.gather, torch.bfloat16, n_x, world)
        except Exception as e:  # an extra must not cost the headline line
            extra["params_bf16"] = {"error": repr(e)[:200]}
        if args.gather == "copy":
            try:  # fp32 master parameters per shard, bf16 replicas for the model: the exchange carries 2 B per parameter
                extra["fp32_master_bf16_replicas"] = sharded_step_line(shapes, dev, "copy", torch.float32, n_x, world,
                                                                       replica_dtype=torch.bfloat16)
            except Exception as e:
                extra["fp32_master_bf16_replicas"] = {"error": repr(e)[:200]}
        other = "fused" if args.gather == "copy" else "copy"
        try:  # the same list with the other in-process exchange (stores inside the update kernel / copy engines)
            extra[f"gather_{other}"] = sharded_step_line(shapes, dev, other, torch.float32, n_x, world)
        except Exception as e:
            extra[f"gather_{other}"] = {"error": repr(e)[:200]}
        if args.model == "7b":
            try:
                s13 = llama7b_shapes(layers=40, hidden=5120, inter=13824)
                extra["llama13b"] = sharded_step_line(s13, dev, args.gather, torch.float32, n_x, world)
            except Exception as e:
                extra["llama13b"] = {"error": repr(e)[:200]}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu = cpu_baseline_in_subprocess(2, 1)
        except Exception as e:  # the child could not run the reference's Python: the C port, in this process
            v, sec, threads, tot = time_cpu_oracle(2, 1, cpu_sample_shapes())
            cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"one transformer layer of the list ({tot} params), C restatement of the reference kernel, OpenMP "
                             f"(the reference's Python could not be timed: {repr(e)[:120]})"}
        cpu["sample"] += "; 2 timed steps after 1 warm-up"
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded N(0,0.02) params, Student-t(3)*1e-3 grads with 1% outlier rows; one gradient set reused every step)",
            "config": {"workload": f"llama{args.model}_shaped_fp32_list_fused_4bit_adamw", "params": total, "tensors": len(shapes),
                       "params_4bit": nq, "params_fp32_state": nf, "layers": n_layers,
                       "parallelism": "single GPU" if world == 1 else (
                           f"ZeRO-1 over {world} GPUs, group-aligned shards, fp32 params reach the peers by "
                           + {"fused": "NVLink stores inside the update kernel",
                              "copy": "copy-engine peer copies of each updated 1-2 GB range, overlapped with the update of the next",
                              "nccl": "an NCCL all-gather after the update"}[args.gather]
                           + ("; gradients of all ranks summed by NVLink loads inside the same kernel" if args.reduce_grads else "")),
                       "l2": "inputs (>= 90 GB touched per step) exceed the 126 MB L2; no explicit flush"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": n_launch, "roofline": roofline, "cpu_baseline": cpu,
        }
        out.update(extra)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--layers", type=int, default=32, help="transformer layers of the list (32 = the 7B workload)")
    ap.add_argument("--model", default="7b", choices=["7b", "13b"],
                    help="7b: the headline list; 13b: the LLaMA-13B-shaped list (52 GB of fp32 parameters per GPU)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="N > 1: skip the bf16 and 13B-shaped extra measurements")
    ap.add_argument("--no-port", action="store_true", help="reference arm: skip the extra timing of the C port")
    ap.add_argument("--reduce-grads", action="store_true",
                    help="N > 1, --gather fused: every rank holds full local gradients and the update kernel also sums "
                         "them over the ranks (reduce-scatter inside the step); no e2e figure in this mode")
    ap.add_argument("--gather", default="copy", choices=["copy", "fused", "nccl"],
                    help="N > 1: parameters reach the peers by copy-engine peer copies of every updated range (overlapped "
                         "with the update of the next), by stores inside the update kernel, or by an NCCL all-gather after it")
    args = ap.parse_args()
    if args.reduce_grads:
        args.gather = "fused"  # the gradient reduction lives in the update kernel
    if args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
