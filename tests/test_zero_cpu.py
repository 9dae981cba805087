"""ZeRO-1 plumbing without a GPU: partition arithmetic, and two gloo ranks whose sharded steps
(the C oracle standing in for the CUDA launch on each rank's group range) followed by the
all-gather reproduce the unsharded result bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

SHAPES = [(40, 128), (4096,), (5000,), (77, 129), (100,), (64, 64, 3)]
HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


def test_partition_covers_every_group_once():
    from lpmm.zero import owned_pieces, owned_range, partition
    numels = [int(np.prod(s)) for s in SHAPES]
    for world in (1, 2, 3, 4, 8, 64):
        gstart, total, shard = partition(numels, world)
        assert total == sum((n + 127) // 128 for n in numels) and shard * world >= total
        seen = np.zeros(total, np.int32)
        for r in range(world):
            lo, hi = owned_range(r, total, shard)
            assert 0 <= lo <= hi <= total
            for i, a, b in owned_pieces(numels, gstart, lo, hi):
                assert 0 <= a < b <= (numels[i] + 127) // 128
                seen[gstart[i] + a: gstart[i] + b] += 1
        assert (seen == 1).all(), f"world {world}: groups not covered exactly once"


def _grads(step):
    out = []
    for i, s in enumerate(SHAPES):
        g = torch.Generator()
        g.manual_seed(step * 100003 + i)
        out.append(torch.randn(s, generator=g) * 1e-3)
    return out


def _oracle_update(opt, lo, hi, qm, qv, hyper=None):
    """What the CUDA launch does for global groups [lo, hi), done by the C oracle on numpy views."""
    from oracle import cpu as O
    from lpmm.zero import GROUP, THRESHOLD, owned_pieces
    hp = hyper if hyper is not None else opt.hyper
    b1, b2 = hp["betas"]
    for i, a, b in owned_pieces(opt.numels, opt.gstart, lo, hi):
        n = opt.numels[i]
        e0, e1 = a * GROUP, min(b * GROUP, n)
        cnt = e1 - e0
        d = opt.gstart[i] + a - opt.lo
        p = opt.params[i].reshape(-1)[e0:e1].numpy()
        if opt._full_grads is not None:  # whole gradient tensors (the optimizer wrapper)
            g = opt._full_grad_tensors[i].reshape(-1)[e0:e1].numpy()
        else:
            g = opt.grad_shard[d * GROUP: d * GROUP + cnt].numpy()
        if n > THRESHOLD:
            nb, ng = (cnt + 1) // 2, b - a
            O.adamw4bit(p, g, opt.m_codes[d * 64: d * 64 + nb].numpy().view(np.uint8),
                        opt.v_codes[d * 64: d * 64 + nb].numpy().view(np.uint8), opt.m_scale[d: d + ng].numpy(),
                        opt.v_scale[d: d + ng].numpy(), qm, qv, b1, b2, hp["lr"], hp["weight_decay"],
                        hp["eps"], float(opt.step_count))
        else:
            df = opt.fstart[i] + a - opt.f_lo
            O.adamw_fp32(p, g, opt.m32[df * GROUP: df * GROUP + cnt].numpy(), opt.v32[df * GROUP: df * GROUP + cnt].numpy(),
                         b1, b2, hp["lr"], hp["weight_decay"], hp["eps"], float(opt.step_count))


def _oracle_engine(qm, qv):
    from lpmm.zero import Zero1FusedAdamW

    class OracleZero(Zero1FusedAdamW):
        def _update(self, lo, hi, hyper=None, peers=True):
            _oracle_update(self, lo, hi, qm, qv, hyper)

    return OracleZero


def _make(world, rank, qm, qv):
    OracleZero = _oracle_engine(qm, qv)

    opt = OracleZero(SHAPES, "cpu", rank=rank, world=world, **HYPER)
    opt.init_params_normal_(0.02, seed=0)
    return opt


def _worker(rank, world, port, golden_dir, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    opt = _make(world, rank, z["m"], z["v"])
    for step in range(1, 4):
        opt.set_grad_shard_from_full(_grads(step))
        opt.step()
    np.save(os.path.join(out_dir, f"flat_{rank}.npy"), opt.flat.numpy())
    # ordering of the peer-store mode: the ranks meet before the launch (nobody overwrites parameters a slower rank
    # still reads) and after it (nobody reads parameters a peer still writes).  The mode itself needs peer-mapped GPU
    # memory; its host logic runs here with the oracle as the launch.
    calls = []
    real_update, real_all_reduce = opt._update, dist.all_reduce
    opt._update = lambda lo, hi, **kw: (calls.append("update"), real_update(lo, hi, **kw))[1]
    dist.all_reduce = lambda t, *a, **k: (calls.append("all_reduce"), real_all_reduce(t, *a, **k))[1]
    opt.gather, opt._flag = "fused", torch.zeros(1)
    opt.set_grad_shard_from_full(_grads(4))
    opt.step()
    dist.all_reduce = real_all_reduce
    with open(os.path.join(out_dir, f"order_{rank}.txt"), "w") as fh:
        fh.write(",".join(calls))
    dist.destroy_process_group()


def test_two_gloo_ranks_equal_the_unsharded_step(golden_dir, tmp_path):
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    single = _make(1, 0, z["m"], z["v"])
    for step in range(1, 4):
        single.set_grad_shard_from_full(_grads(step))
        single.step()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, golden_dir, str(tmp_path)), nprocs=2, join=True)
    flats = [np.load(tmp_path / f"flat_{r}.npy") for r in range(2)]
    for r in range(2):
        assert (tmp_path / f"order_{r}.txt").read_text() == "all_reduce,update,all_reduce", "barrier / launch / barrier"
    assert np.array_equal(flats[0].view(np.int32), flats[1].view(np.int32)), "ranks disagree after the all-gather"
    for i, p in enumerate(single.params):
        lo = single.gstart[i] * 128
        got = flats[0][lo: lo + p.numel()]
        assert np.array_equal(got.view(np.int32), p.reshape(-1).numpy().view(np.int32)), f"tensor {i} differs from unsharded"


# ---- failures, made on the host among gloo ranks (no GPU involved) ------------------------------
def _mismatch_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lpmm.zero import Zero1FusedAdamW
    shapes = SHAPES if rank == 0 else SHAPES[:-1] + [(64, 64, 4)]
    try:
        Zero1FusedAdamW(shapes, "cpu", **HYPER)
        verdict = "constructed"
    except ValueError as e:
        verdict = "ValueError: " + str(e)[:40]
    with open(os.path.join(out_dir, f"verdict_{rank}.txt"), "w") as fh:
        fh.write(verdict)
    dist.destroy_process_group()


def test_ranks_with_different_lists_are_refused(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_mismatch_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"verdict_{r}.txt").read_text().startswith("ValueError"), f"rank {r} accepted a mismatched list"


def _dropout_worker(rank, world, port, golden_dir, out_dir):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    opt = _make(world, rank, z["m"], z["v"])
    opt.set_grad_shard_from_full(_grads(1))
    opt.step()                                    # a healthy step first
    if rank == 1:
        os._exit(0)                               # rank 1 leaves between steps, nothing of its in flight
    opt.set_grad_shard_from_full(_grads(2))
    try:
        opt.step()                                # the all-gather cannot complete
        verdict = "completed"
    except Exception as e:  # gloo reports the lost peer or the timeout as a RuntimeError
        verdict = "error: " + type(e).__name__
    with open(os.path.join(out_dir, "verdict_0.txt"), "w") as fh:
        fh.write(verdict)
    os._exit(0)


def test_a_rank_leaving_between_steps_surfaces_as_an_error(golden_dir, tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_dropout_worker, args=(2, port, golden_dir, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "verdict_0.txt").read_text().startswith("error"), "the surviving rank did not notice"


# ---- sharded checkpoints -------------------------------------------------------------------------
def _state_worker(rank, world, port, golden_dir, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    opt = _make(world, rank, z["m"], z["v"])
    for step in range(1, 3):
        opt.set_grad_shard_from_full(_grads(step))
        opt.step()
    full = opt.gather_state()
    # a fresh sharded optimizer resumed from the gathered state continues identically
    opt2 = _make(world, rank, z["m"], z["v"])
    opt2.flat.copy_(opt.flat)
    opt2.load_full_state(full)
    for o in (opt, opt2):
        o.set_grad_shard_from_full(_grads(3))
        o.step()
    same = bool(torch.equal(opt.flat.view(torch.int32), opt2.flat.view(torch.int32)))
    if rank == 0:
        torch.save({"full": full, "same": same}, os.path.join(out_dir, "state.pt"))
    dist.destroy_process_group()


def test_sharded_state_gathers_to_the_unsharded_layout_and_reloads(golden_dir, tmp_path):
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    single = _make(1, 0, z["m"], z["v"])
    for step in range(1, 3):
        single.set_grad_shard_from_full(_grads(step))
        single.step()
    ref = single.gather_state()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_state_worker, args=(2, port, golden_dir, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / "state.pt", weights_only=False)
    assert got["same"], "resuming from the gathered state changed the next step"
    assert len(got["full"]) == len(ref) == len(SHAPES)
    for i, (a, b) in enumerate(zip(got["full"], ref)):
        assert a.keys() == b.keys() and a["step"] == b["step"] == 2.0
        for k in a:
            if k != "step":
                assert a[k].dtype == b[k].dtype and a[k].shape == b[k].shape, (i, k)
                assert torch.equal(a[k].view(torch.uint8), b[k].view(torch.uint8)), f"tensor {i} {k}"


# ---- the optimizer wrapper: parameters adopted into the flat buffer, parameter groups, state_dict ------------------
def _wrapper_run(qm, qv, steps=3, resume_from=None, from_host=False):
    """A small model stepped by ``lpmm.optim.ZeroAdamW`` (engine = the C oracle): two parameter groups with different
    weight decay, the learning rate of the second halved at step 2.  ``from_host``: the gradients are handed to
    ``step_from_host`` (tiny chunks: several launches per parameter group) instead of being put into ``p.grad``.
    Returns (optimizer, parameters)."""
    import lpmm
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(s) * 0.02) for s in SHAPES]
    groups = [dict(params=params[:3], weight_decay=0.01), dict(params=params[3:], weight_decay=0.1, lr=2e-3)]
    opt = lpmm.optim.ZeroAdamW(groups, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, engine_cls=_oracle_engine(qm, qv))
    first = 1
    if resume_from is not None:
        sd, pvals, first = resume_from
        opt.load_state_dict(sd)
        for p, v in zip(params, pvals):
            p.data.copy_(v)
    for step in range(first, steps + 1):
        if step == 2:
            opt.param_groups[1]["lr"] = 1e-3
        if from_host:
            opt.step_from_host(_grads(step), chunk_bytes=4096)
            continue
        for p, g in zip(params, _grads(step)):
            p.grad = g
        opt.step()
    return opt, params


def _wrapper_worker(rank, world, port, golden_dir, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    opt, params = _wrapper_run(z["m"], z["v"], steps=2)
    sd = opt.state_dict()                                   # collective
    pvals = [p.detach().clone() for p in params]
    # resume in a fresh wrapper from the gathered dict and take step 3 (gradients through step_from_host); and take
    # step 3 directly
    opt2, params2 = _wrapper_run(z["m"], z["v"], steps=3, resume_from=(sd, pvals, 3), from_host=True)
    for p, g in zip(params, _grads(3)):
        p.grad = g
    opt.step()
    same = all(torch.equal(a.detach().view(torch.int32), b.detach().view(torch.int32)) for a, b in zip(params, params2))
    final = opt.state_dict()
    if rank == 0:
        torch.save({"sd": final, "params": [p.detach().clone() for p in params], "resumed_same": same},
                   os.path.join(out_dir, "wrapper.pt"))
    dist.destroy_process_group()


def _assert_same_tree(a, b, path="sd"):
    assert type(a) is type(b) or (isinstance(a, (int, float)) and isinstance(b, (int, float))), (path, type(a), type(b))
    if isinstance(a, torch.Tensor):
        assert a.dtype == b.dtype and a.shape == b.shape, (path, a.dtype, b.dtype, a.shape, b.shape)
        assert torch.equal(a.contiguous().reshape(-1).view(torch.uint8), b.contiguous().reshape(-1).view(torch.uint8)), path
    elif isinstance(a, dict):
        assert list(a.keys()) == list(b.keys()), (path, list(a.keys()), list(b.keys()))
        for k in a:
            _assert_same_tree(a[k], b[k], f"{path}[{k!r}]")
    elif isinstance(a, (list, tuple)):
        assert len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            _assert_same_tree(x, y, f"{path}[{i}]")
    elif path.endswith("['qconfig']"):
        assert str(a) == str(b), path
    else:
        assert a == b, (path, a, b)


def test_zero_optimizer_wrapper_two_ranks_equal_one_rank(golden_dir, tmp_path):
    """Two gloo ranks of ``lpmm.optim.ZeroAdamW`` against the same wrapper on one rank: equal parameters and equal
    ``state_dict()`` (the unsharded fused layout) after 3 steps with two parameter groups and a changed learning
    rate; a wrapper resumed from the gathered dict continues identically."""
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    single, sparams = _wrapper_run(z["m"], z["v"], steps=3)
    ref = single.state_dict()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_wrapper_worker, args=(2, port, golden_dir, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / "wrapper.pt", weights_only=False)
    assert got["resumed_same"], "a wrapper resumed from the gathered state_dict diverged"
    for i, (a, b) in enumerate(zip(got["params"], sparams)):
        assert torch.equal(a.view(torch.int32), b.detach().view(torch.int32)), f"tensor {i}"
    _assert_same_tree(got["sd"], ref)
    # the layout of the reference's fused state (lpmm/optim/adamw.py:508-523)
    st = ref["state"][0]
    n = int(np.prod(SHAPES[0]))
    assert list(st.keys()) == ["step", "exp_avg", "exp_avg_qstate", "exp_avg_sq", "exp_avg_sq_qstate"]
    assert st["exp_avg"].dtype == torch.int8 and st["exp_avg"].numel() == (n + 1) // 2
    assert st["exp_avg_qstate"]["overhead"]["max1"].numel() == (n + 127) // 128 and st["exp_avg_qstate"]["enable"]
    small = ref["state"][1]  # 4096 elements: fp32 moments shaped like the parameter
    assert small["exp_avg"].dtype == torch.float32 and tuple(small["exp_avg"].shape) == SHAPES[1]
    assert ref["param_groups"][1]["weight_decay"] == 0.1 and ref["param_groups"][1]["lr"] == 1e-3
    assert "qconfig" in ref


def test_step_from_host_without_a_gpu_is_copy_then_step(golden_dir):
    """On a CPU engine (the oracle as the launch) ``step_from_host`` has nothing to overlap: it must equal
    ``grad_shard.copy_(host); step()`` and refuse a shard of the wrong size."""
    z = np.load(os.path.join(golden_dir, "qmaps.npz"))
    a, b = _make(1, 0, z["m"], z["v"]), _make(1, 0, z["m"], z["v"])
    for step in range(1, 3):
        b.set_grad_shard_from_full(_grads(step))
        host = b.grad_shard.clone()
        b.step()
        a.step_from_host(host)
    assert a.step_count == b.step_count == 2
    assert np.array_equal(a.flat.numpy().view(np.int32), b.flat.numpy().view(np.int32))
    with pytest.raises(RuntimeError):
        a.step_from_host(host[:-1])


def test_copy_exchange_cuts_the_owned_range_into_a_short_first_range_and_full_ones():
    """gather="copy": ``_update_in_chunks`` must cover ``[lo, hi)`` exactly once, in order, with a first range of an
    eighth of ``copy_chunk_bytes(world)`` (the copy engines start early) and full ranges after it; other modes take
    one launch.  The launches are recorded instead of run."""
    from lpmm import zero as Z

    class Recorder(Z.Zero1FusedAdamW):
        def __init__(self):  # no buffers: only the fields the chunking reads
            self.calls, self.esize = [], 4

        def _update(self, lo, hi, hyper=None, peers=True):
            self.calls.append((lo, hi))

    assert Z.copy_chunk_bytes(2) == 1 << 30 and Z.copy_chunk_bytes(4) == Z.copy_chunk_bytes(8) == 2 << 30
    for world in (2, 4, 8):
        per = Z.copy_chunk_bytes(world) // (Z.GROUP * 4)
        for lo, hi in ((0, 1), (5, 5 + per // 8), (7, 7 + per // 8 + 1), (100, 100 + 3 * per + 17)):
            r = Recorder()
            r.gather, r.world = "copy", world
            r._update_in_chunks(lo, hi)
            assert r.calls[0][0] == lo and r.calls[-1][1] == hi
            assert all(a[1] == b[0] for a, b in zip(r.calls, r.calls[1:])), "ranges must follow each other"
            assert r.calls[0][1] - r.calls[0][0] <= max(1, per // 8)
            assert all(b - a <= per for a, b in r.calls[1:])
            assert len(r.calls) == 1 + max(0, -(-(hi - lo - max(1, per // 8)) // per))
    r = Recorder()
    r.gather, r.world = "fused", 8
    r._update_in_chunks(3, 10 ** 9)
    assert r.calls == [(3, 10 ** 9)]
