"""ZeRO-1 sharding of the fused 4-bit AdamW step (no counterpart in the reference, which has no
distributed code beyond a seed broadcast, lpmm/optim/optimizer.py:19-22).

The parameter list defines a global sequence of 128-element groups (tensor t contributes
ceil(numel_t / 128) groups, in list order).  Every group is independent in the fused step -- its
codes, its two scales, its slice of p and g -- so the sequence is cut into ``world`` contiguous
ranges of equal length S = ceil(G / world) and rank r

* keeps 4-bit codes, scales, fp32 moments of small tensors and gradients ONLY for its range,
* updates its range of the (replicated, flat) fp32 parameter buffer with the same multi-tensor
  launch as the unsharded step, restricted to ``[r*S, (r+1)*S)``,
* makes the updated range visible to all ranks: either one NCCL ``all_gather_into_tensor`` of the
  flat parameter buffer after the launch (``gather="nccl"``), or -- ``gather="fused"`` -- the launch
  itself stores every updated parameter into all peers' buffers through peer-mapped symmetric
  memory (plain vectorised stores over NVLink, no multicast), so transfer and update overlap group
  by group and only a barrier follows.

With ``reduce_grads=True`` the gradient reduce-scatter moves into the launch as well: every rank keeps
its full local gradients in a peer-mapped buffer and the update kernel sums, for each element of the
rank's own range, the values of all ranks (fixed rank order) before the update -- reads of the peers'
gradients and stores into the peers' parameters travel over NVLink in opposite directions while the
kernel computes.  The whole ZeRO-1 step (reduce-scatter, update, all-gather) is then one kernel.

The result is bit-identical to the unsharded step.  A shard may cut a tensor but never a group.
"""
import ctypes

import torch
import torch.distributed as dist

GROUP = 128
THRESHOLD = 4096


def groups_of(numel):
    return (numel + GROUP - 1) // GROUP


def partition(numels, world):
    """Group layout of a parameter list.

    Returns ``(gstart, total_groups, shard_groups)``: first global group of every tensor, the
    number of groups, and S = ceil(total / world).  Rank r owns ``[r*S, min((r+1)*S, total))``."""
    gstart, g = [], 0
    for n in numels:
        gstart.append(g)
        g += groups_of(n)
    shard = (g + world - 1) // world if world > 0 else g
    return gstart, g, shard


def owned_range(rank, total_groups, shard_groups):
    lo = min(rank * shard_groups, total_groups)
    return lo, min(lo + shard_groups, total_groups)


def owned_pieces(numels, gstart, lo, hi):
    """``(tensor index, first local group, one-past-last local group)`` for every tensor that
    intersects the global group range ``[lo, hi)``."""
    out = []
    for i, (n, gs) in enumerate(zip(numels, gstart)):
        a, b = max(lo, gs), min(hi, gs + groups_of(n))
        if a < b:
            out.append((i, a - gs, b - gs))
    return out


class Zero1FusedAdamW:
    """Fused 4-bit AdamW over a flat, replicated fp32 parameter buffer with ZeRO-1 sharded states.

    ``shapes``: shapes of the parameter list.  ``self.params[i]`` is a view of the flat buffer
    (tensor i starts on a group boundary).  ``self.grad_shard`` is this rank's slice of the flat
    gradient (what a reduce-scatter of gradients would deliver), ``shard_groups * 128`` floats.
    """

    def __init__(self, shapes, device, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, process_group=None,
                 rank=None, world=None, gather="nccl", reduce_grads=False, grad_scale=None):
        from .functional import create_general_qmap
        self.shapes = [tuple(s) for s in shapes]
        self.numels = [int(torch.Size(s).numel()) for s in self.shapes]
        self.device = torch.device(device)
        self.pg = process_group
        self.world = world if world is not None else (dist.get_world_size(process_group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(process_group) if dist.is_initialized() else 0)
        self.hyper = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.step_count = 0
        self.gstart, self.total_groups, self.shard_groups = partition(self.numels, self.world)
        self.lo, self.hi = owned_range(self.rank, self.total_groups, self.shard_groups)
        S = self.shard_groups
        self._check_same_layout_everywhere()
        if gather not in ("nccl", "fused"):
            raise ValueError("gather must be 'nccl' or 'fused'")
        self.gather = gather if self.world > 1 else "nccl"
        self.peer_offsets = None
        if self.gather == "fused":
            import torch.distributed._symmetric_memory as symm_mem
            self.flat = symm_mem.empty(self.world * S * GROUP, dtype=torch.float32, device=self.device)
            self.flat.zero_()
            self._symm = symm_mem.rendezvous(self.flat, process_group if process_group is not None else dist.group.WORLD)
            ptrs = list(self._symm.buffer_ptrs)
            mine = self.flat.data_ptr()
            self.peer_offsets = [int(ptrs[r]) - mine for r in range(self.world) if r != self.rank]
            self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        else:
            self.flat = torch.zeros(self.world * S * GROUP, dtype=torch.float32, device=self.device)
        self.params = [self.flat[gs * GROUP: gs * GROUP + n].view(s)
                       for s, n, gs in zip(self.shapes, self.numels, self.gstart)]
        self.grad_shard = torch.zeros(S * GROUP, dtype=torch.float32, device=self.device)
        # reduce_grads: every rank holds a FULL flat gradient buffer (its local gradients, as data-parallel
        # backward leaves them) in symmetric memory, ``self.grads[i]`` its views; the update kernel of a rank
        # sums the gradients of its own group range over all ranks (rank order 0 .. world-1) and multiplies
        # by ``grad_scale`` (default 1/world): the reduce-scatter happens inside the step.
        self.reduce_grads = bool(reduce_grads) and self.world > 1
        self.grad_offsets = None
        if self.reduce_grads:
            if self.gather != "fused":
                raise ValueError("reduce_grads needs gather='fused' (peer-mapped buffers)")
            import torch.distributed._symmetric_memory as symm_mem
            self.grad_flat = symm_mem.empty(self.world * S * GROUP, dtype=torch.float32, device=self.device)
            self.grad_flat.zero_()
            self._gsymm = symm_mem.rendezvous(self.grad_flat, process_group if process_group is not None else dist.group.WORLD)
            gptrs = list(self._gsymm.buffer_ptrs)
            gmine = self.grad_flat.data_ptr()
            self.grad_offsets = [int(gptrs[r]) - gmine for r in range(self.world)]
            self.grad_scale = float(grad_scale) if grad_scale is not None else 1.0 / self.world
            self.grads = [self.grad_flat[gs * GROUP: gs * GROUP + n].view(s)
                          for s, n, gs in zip(self.shapes, self.numels, self.gstart)]
        # states of the owned range only
        self.m_codes = torch.zeros(S * (GROUP // 2), dtype=torch.int8, device=self.device)
        self.v_codes = torch.zeros(S * (GROUP // 2), dtype=torch.int8, device=self.device)
        self.m_scale = torch.zeros(S, dtype=torch.float32, device=self.device)
        self.v_scale = torch.zeros(S, dtype=torch.float32, device=self.device)
        # fp32 moments of the tensors at or below the threshold: own "small-tensor group" index space
        self.fstart, f = [], 0
        for n in self.numels:
            self.fstart.append(f)
            if n <= THRESHOLD:
                f += groups_of(n)
        pieces = owned_pieces(self.numels, self.gstart, self.lo, self.hi)
        small = [(i, a, b) for (i, a, b) in pieces if self.numels[i] <= THRESHOLD]
        self.f_lo = self.fstart[small[0][0]] + small[0][1] if small else 0
        f_cnt = sum(b - a for (_, a, b) in small)
        self.m32 = torch.zeros(max(f_cnt, 1) * GROUP, dtype=torch.float32, device=self.device)
        self.v32 = torch.zeros(max(f_cnt, 1) * GROUP, dtype=torch.float32, device=self.device)
        self.qmap_m = create_general_qmap("nonlinear", 4, True).to(self.device)
        self.qmap_v = create_general_qmap("power-1", 4, False).to(self.device)
        self._tl = None

    def _check_same_layout_everywhere(self):
        """All ranks must cut the same list the same way; a rank built from a different list would
        update the wrong ranges silently.  Compares (tensor count, group count, a hash of the sizes)."""
        if self.world == 1 or not dist.is_initialized():
            return
        h = 0
        for n in self.numels:
            h = (h * 1000003 + n) % 2147483629
        mine = torch.tensor([len(self.numels), self.total_groups, h], dtype=torch.int64)
        backend = dist.get_backend(self.pg)
        dev = self.device if backend == "nccl" else torch.device("cpu")
        lo, hi = mine.to(dev).clone(), mine.to(dev).clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.pg)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.pg)
        if not torch.equal(lo, hi):
            raise ValueError("ZeRO-1: the ranks were given different parameter lists "
                             f"(this rank: {len(self.numels)} tensors, {self.total_groups} groups)")

    # ---- data ---------------------------------------------------------------------------------
    def init_params_normal_(self, std, seed=0):
        """Same values on every rank (seeded), like replicated model parameters."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        chunk = 1 << 26
        for lo in range(0, self.flat.numel(), chunk):
            hi = min(lo + chunk, self.flat.numel())
            self.flat[lo:hi].normal_(0, std, generator=g)

    def set_grad_shard_from_full(self, grads):
        """Copy this rank's slice out of a full gradient list (tests / single-process use)."""
        self.grad_shard.zero_()
        for i, a, b in owned_pieces(self.numels, self.gstart, self.lo, self.hi):
            n = self.numels[i]
            e0, e1 = a * GROUP, min(b * GROUP, n)
            off = (self.gstart[i] + a - self.lo) * GROUP
            self.grad_shard[off: off + (e1 - e0)].copy_(grads[i].reshape(-1)[e0:e1])

    # ---- the step -----------------------------------------------------------------------------
    def descriptors(self):
        """Descriptor entries (p, g, m, v, m_scale, v_scale, numel, kind) with *virtual* base addresses:
        states and gradients exist only for the owned range, so their pointers are offset such that
        indexing by a tensor-local group lands inside the shard buffers for owned groups.  Groups
        outside ``[lo, hi)`` are never touched by the launch."""
        out = []
        for n, gs, fs in zip(self.numels, self.gstart, self.fstart):
            d = gs - self.lo  # may be negative
            p = self.flat.data_ptr() + gs * GROUP * 4
            if self.reduce_grads:
                g = self.grad_flat.data_ptr() + gs * GROUP * 4
            else:
                g = self.grad_shard.data_ptr() + d * GROUP * 4
            if n > THRESHOLD:
                out.append((p, g, self.m_codes.data_ptr() + d * (GROUP // 2), self.v_codes.data_ptr() + d * (GROUP // 2),
                            self.m_scale.data_ptr() + d * 4, self.v_scale.data_ptr() + d * 4, n, 0))
            else:
                df = fs - self.f_lo
                out.append((p, g, self.m32.data_ptr() + df * GROUP * 4, self.v32.data_ptr() + df * GROUP * 4, 0, 0, n, 1))
        return out

    def _update(self, lo, hi):
        """Update global groups ``[lo, hi)`` (a sub-range of the owned range) on the current stream."""
        from . import _native as N
        if self._tl is None:
            desc = self.descriptors()
            arr = (N.Tensor * len(desc))()
            for i, (p, g, m, v, sm, sv, n, kind) in enumerate(desc):
                arr[i] = N.Tensor(p, g, m, v, sm or None, sv or None, n, kind, 0)
            self._tl = arr
        b1, b2 = self.hyper["betas"]
        h = N.Hyper(b1, b2, self.hyper["lr"], self.hyper["weight_decay"], self.hyper["eps"], float(self.step_count))
        with torch.cuda.device(self.device):
            qm, qv = ctypes.c_void_p(self.qmap_m.data_ptr()), ctypes.c_void_p(self.qmap_v.data_ptr())
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            if self.reduce_grads:
                offs = (ctypes.c_int64 * len(self.peer_offsets))(*self.peer_offsets)
                goffs = (ctypes.c_int64 * len(self.grad_offsets))(*self.grad_offsets)
                N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_zero1(self._tl, len(self.numels), qm, qv, h, lo, hi, offs,
                                                                     len(self.peer_offsets), goffs, len(self.grad_offsets),
                                                                     self.grad_scale, st))
            elif self.peer_offsets:
                offs = (ctypes.c_int64 * len(self.peer_offsets))(*self.peer_offsets)
                N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_peers(self._tl, len(self.numels), qm, qv, h, lo, hi, offs,
                                                                     len(self.peer_offsets), st))
            else:
                N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor(self._tl, len(self.numels), qm, qv, h, lo, hi, st))

    def _gather(self):
        if self.world == 1:
            return
        if self.gather == "fused":
            # the launch already wrote every peer's copy; order the ranks on the stream
            dist.all_reduce(self._flag, group=self.pg)
            return
        S = self.shard_groups * GROUP
        dist.all_gather_into_tensor(self.flat, self.flat[self.rank * S:(self.rank + 1) * S], group=self.pg)

    def step(self):
        self.step_count += 1
        if self.gather == "fused":
            # The launch stores into every peer's parameter buffer: no rank may start it while another still reads
            # its parameters (forward / backward of a slower rank), and with reduce_grads every rank's gradients must
            # be complete before any rank reads them.  One tiny all-reduce on the stream orders the ranks; the one
            # after the update (in _gather) keeps parameters and gradients from being touched while a peer still
            # writes or reads them.
            dist.all_reduce(self._flag, group=self.pg)
        if self.hi > self.lo:
            self._update(self.lo, self.hi)
        self._gather()

    # ---- checkpoints --------------------------------------------------------------------------
    def gather_state(self):
        """Reassemble, on every rank, the optimizer state of the whole list in the layout of the
        unsharded fused optimizer: per tensor ``exp_avg`` / ``exp_avg_sq`` as ``int8[(numel+1)//2]``
        codes with ``float32[groups]`` scales, or fp32 moments for the small tensors; plus ``step``.
        Collective: every rank must call it."""
        S = self.shard_groups

        def gathered(x):
            if self.world == 1:
                return x.clone()
            out = torch.empty(self.world * x.numel(), dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(out, x.contiguous(), group=self.pg)
            return out

        mc, vc = gathered(self.m_codes), gathered(self.v_codes)
        ms, vs = gathered(self.m_scale), gathered(self.v_scale)
        # small-tensor fp32 moments: every rank contributes (first small-group index, data)
        small = [None] * self.world
        mine = (self.f_lo, self.m32.cpu(), self.v32.cpu())
        if self.world == 1:
            small = [mine]
        else:
            dist.all_gather_object(small, mine, group=self.pg)
        f_total = self.fstart[-1] + (groups_of(self.numels[-1]) if self.numels[-1] <= THRESHOLD else 0) if self.numels else 0
        m32 = torch.zeros(max(f_total, 1) * GROUP, dtype=torch.float32)
        v32 = torch.zeros(max(f_total, 1) * GROUP, dtype=torch.float32)
        for r, (f_lo, a, b) in enumerate(small):
            lo, hi = owned_range(r, self.total_groups, S)
            cnt = sum(y - x for (i, x, y) in owned_pieces(self.numels, self.gstart, lo, hi) if self.numels[i] <= THRESHOLD)
            m32[f_lo * GROUP:(f_lo + cnt) * GROUP] = a[:cnt * GROUP]
            v32[f_lo * GROUP:(f_lo + cnt) * GROUP] = b[:cnt * GROUP]
        out = []
        for n, gs, fs in zip(self.numels, self.gstart, self.fstart):
            if n > THRESHOLD:
                nb, ng = (n + 1) // 2, groups_of(n)
                out.append({"step": float(self.step_count), "exp_avg": mc[gs * 64: gs * 64 + nb].clone(),
                            "exp_avg_sq": vc[gs * 64: gs * 64 + nb].clone(), "exp_avg_scale": ms[gs: gs + ng].clone(),
                            "exp_avg_sq_scale": vs[gs: gs + ng].clone()})
            else:
                out.append({"step": float(self.step_count), "exp_avg": m32[fs * GROUP: fs * GROUP + n].to(self.device),
                            "exp_avg_sq": v32[fs * GROUP: fs * GROUP + n].to(self.device)})
        return out

    def load_full_state(self, states):
        """Inverse of ``gather_state``: every rank keeps its own range of a full (unsharded-layout)
        state list, e.g. one taken from ``lpmm.optim.AdamW(fused=True)``."""
        self.step_count = int(states[0]["step"]) if states else 0
        for buf in (self.m_codes, self.v_codes, self.m_scale, self.v_scale, self.m32, self.v32):
            buf.zero_()
        for i, a, b in owned_pieces(self.numels, self.gstart, self.lo, self.hi):
            n, st = self.numels[i], states[i]
            d = self.gstart[i] + a - self.lo
            if n > THRESHOLD:
                b0, b1 = a * 64, min(b * 64, (n + 1) // 2)
                self.m_codes[d * 64: d * 64 + (b1 - b0)].copy_(st["exp_avg"].reshape(-1)[b0:b1])
                self.v_codes[d * 64: d * 64 + (b1 - b0)].copy_(st["exp_avg_sq"].reshape(-1)[b0:b1])
                self.m_scale[d: d + (b - a)].copy_(st["exp_avg_scale"].reshape(-1)[a:b])
                self.v_scale[d: d + (b - a)].copy_(st["exp_avg_sq_scale"].reshape(-1)[a:b])
            else:
                e0, e1 = a * GROUP, min(b * GROUP, n)
                df = self.fstart[i] + a - self.f_lo
                self.m32[df * GROUP: df * GROUP + (e1 - e0)].copy_(st["exp_avg"].reshape(-1)[e0:e1])
                self.v32[df * GROUP: df * GROUP + (e1 - e0)].copy_(st["exp_avg_sq"].reshape(-1)[e0:e1])

    # ---- measurement helpers (bench) -------------------------------------------------------------
    def time_update_only(self, iters):
        """Mean duration (ms) of the sharded update launch alone and its algorithmic bytes."""
        ms = []
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.step_count += 1
            a.record()
            self._update(self.lo, self.hi)
            b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        nbytes = 0.0
        for i, a_, b_ in owned_pieces(self.numels, self.gstart, self.lo, self.hi):
            cnt = min(b_ * GROUP, self.numels[i]) - a_ * GROUP
            nbytes += cnt * (14.125 if self.numels[i] > THRESHOLD else 28.0)
        return sum(ms) / len(ms), nbytes

    def breakdown(self, iters):
        """Update-only and all-gather-only timings, max over ranks."""
        upd, _ = self.time_update_only(iters)
        ms = []
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier(group=self.pg)
            a.record()
            self._gather()
            b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        t = torch.tensor([upd, sum(ms) / len(ms)], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.pg)
        upd_ms, ag_ms = float(t[0]), float(t[1])
        total = sum(self.numels)
        recv = 4.0 * self.shard_groups * GROUP * (self.world - 1)
        if self.gather == "fused":
            return {"update_with_peer_stores": {"ms": upd_ms, "aggregate_params_per_s": total / (upd_ms * 1e-3),
                                                "nvlink_bytes_sent_per_rank": recv,
                                                "nvlink_gb_per_s_per_rank": recv / (upd_ms * 1e-3) / 1e9},
                    "rank_barrier": {"ms": ag_ms}}
        return {"update_only": {"ms": upd_ms, "aggregate_params_per_s": total / (upd_ms * 1e-3)},
                "all_gather": {"ms": ag_ms, "bytes_received_per_rank": recv, "gb_per_s_per_rank": recv / (ag_ms * 1e-3) / 1e9}}
