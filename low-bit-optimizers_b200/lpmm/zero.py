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
  by group and only a barrier follows; or -- ``gather="copy"`` -- the range is updated in pieces of 1-2 GB and the
  copy engines write every finished piece into the peers' buffers while the next piece is updated (on this
  hardware the copy engines move 770 GB/s per direction where stores from the SMs reach 660-690, so this is the
  fastest of the three; measured 18.2 / 27.5 / 31.2 ms per step of the 7B list on 2 / 4 / 8 GPUs against 20.0 / 30.2 / 35.4).

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


def copy_chunk_bytes(world):
    """gather="copy": bytes of parameters per update launch / round of peer copies.  Large rounds keep the ranks in
    step (one sender per receiver at a time); with a single peer shorter rounds fill the pipeline sooner.  Measured on
    the 7B list: 2 GPUs 18.2 / 18.7 / 19.8 ms with 1 / 2 / 4 GB, 4 GPUs 33.3 / 28.6 / 27.4 / 27.4 ms with 0.5 / 1 / 2 GB /
    the whole shard."""
    return (1 << 30) if world <= 2 else (2 << 30)


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
                 rank=None, world=None, gather="nccl", reduce_grads=False, grad_scale=None, dtype=torch.float32,
                 exact_params=True, replica_dtype=None):
        """``dtype``: element type of parameters and gradients, fp32 or bf16 / fp16 (the 16-bit fused step; half the
        bytes over NVLink).  ``exact_params=False``: the tolerance mode of the fused step (codes and scales as
        always, parameters within 1e-6 relative).  ``replica_dtype`` (bf16 / fp16; fp32 parameters, gather="copy"): fp32
        MASTER parameters with 16-bit replicas -- a rank keeps fp32 parameters only for its own range (the rest of
        ``flat`` is never refreshed), narrows every updated range into ``replica`` and the copy engines publish that
        to the peers: the exchange carries 2 bytes per parameter and the model computes on ``replica_params``."""
        from .functional import create_general_qmap
        if dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise ValueError("dtype must be float32, bfloat16 or float16")
        self.dtype = dtype
        self.esize = 4 if dtype == torch.float32 else 2
        self.exact_params = bool(exact_params)
        self._full_grads = None  # data pointers of whole gradient tensors (use_full_grads) instead of grad_shard
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
        if gather not in ("nccl", "fused", "copy"):
            raise ValueError("gather must be 'nccl', 'fused' or 'copy'")
        self.gather = gather if self.world > 1 else "nccl"
        self.peer_offsets = None
        if self.gather in ("fused", "copy"):
            import torch.distributed._symmetric_memory as symm_mem
            self.flat = symm_mem.empty(self.world * S * GROUP, dtype=self.dtype, device=self.device)
            self.flat.zero_()
            self._symm = symm_mem.rendezvous(self.flat, process_group if process_group is not None else dist.group.WORLD)
            ptrs = list(self._symm.buffer_ptrs)
            mine = self.flat.data_ptr()
            if self.gather == "fused":
                self.peer_offsets = [int(ptrs[r]) - mine for r in range(self.world) if r != self.rank]
            else:
                # the peers' copies of the flat buffer as tensors, nearest rank first (every rank starts with another peer)
                order = [(self.rank + k) % self.world for k in range(1, self.world)]
                self._peer_flats = [self._symm.get_buffer(r, (self.world * S * GROUP,), self.dtype) for r in order]
                self._peer_stream = torch.cuda.Stream(device=self.device)
            self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        else:
            self.flat = torch.zeros(self.world * S * GROUP, dtype=self.dtype, device=self.device)
        self.params = [self.flat[gs * GROUP: gs * GROUP + n].view(s)
                       for s, n, gs in zip(self.shapes, self.numels, self.gstart)]
        self.replica = None
        if replica_dtype is not None:
            if self.dtype != torch.float32 or replica_dtype not in (torch.bfloat16, torch.float16):
                raise ValueError("replica_dtype is bfloat16 or float16, next to float32 parameters")
            if self.world > 1 and self.gather != "copy":
                raise ValueError("replica_dtype needs gather='copy'")
            if self.world > 1:
                import torch.distributed._symmetric_memory as symm_mem
                self.replica = symm_mem.empty(self.world * S * GROUP, dtype=replica_dtype, device=self.device)
                self.replica.zero_()
                self._rsymm = symm_mem.rendezvous(self.replica, process_group if process_group is not None else dist.group.WORLD)
                order = [(self.rank + k) % self.world for k in range(1, self.world)]
                self._peer_replicas = [self._rsymm.get_buffer(r, (self.world * S * GROUP,), replica_dtype) for r in order]
            else:
                self.replica = torch.zeros(self.world * S * GROUP, dtype=replica_dtype, device=self.device)
            self.replica_params = [self.replica[gs * GROUP: gs * GROUP + n].view(s)
                                   for s, n, gs in zip(self.shapes, self.numels, self.gstart)]
        self.xsize = 2 if self.replica is not None else self.esize  # bytes per parameter that reach the peers
        self.grad_shard = torch.zeros(S * GROUP, dtype=self.dtype, device=self.device)
        # reduce_grads: every rank holds a FULL flat gradient buffer (its local gradients, as data-parallel
        # backward leaves them) in symmetric memory, ``self.grads[i]`` its views; the update kernel of a rank
        # sums the gradients of its own group range over all ranks (rank order 0 .. world-1) and multiplies
        # by ``grad_scale`` (default 1/world): the reduce-scatter happens inside the step.
        self.reduce_grads = bool(reduce_grads) and self.world > 1
        self.grad_offsets = None
        if self.reduce_grads:
            if self.gather != "fused":
                raise ValueError("reduce_grads needs gather='fused' (peer-mapped buffers)")
            if self.dtype != torch.float32:
                raise NotImplementedError("reduce_grads is built for fp32 parameters and gradients")
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
            if self.replica is not None:
                self.replica[lo:hi].copy_(self.flat[lo:hi])

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
        es = self.esize
        for i, (n, gs, fs) in enumerate(zip(self.numels, self.gstart, self.fstart)):
            d = gs - self.lo  # may be negative
            p = self.flat.data_ptr() + gs * GROUP * es
            if self._full_grads is not None:
                g = self._full_grads[i]  # a whole gradient tensor: indexed by the tensor's own groups
            elif self.reduce_grads:
                g = self.grad_flat.data_ptr() + gs * GROUP * es
            else:
                g = self.grad_shard.data_ptr() + d * GROUP * es
            if n > THRESHOLD:
                out.append((p, g, self.m_codes.data_ptr() + d * (GROUP // 2), self.v_codes.data_ptr() + d * (GROUP // 2),
                            self.m_scale.data_ptr() + d * 4, self.v_scale.data_ptr() + d * 4, n, 0))
            else:
                df = fs - self.f_lo
                out.append((p, g, self.m32.data_ptr() + df * GROUP * 4, self.v32.data_ptr() + df * GROUP * 4, 0, 0, n, 1))
        return out

    def use_full_grads(self, grads):
        """Take the gradients from whole per-tensor gradient tensors (already reduced over the ranks, as data-parallel
        backward with an all-reduce leaves them) instead of ``grad_shard``: nothing is copied, the launch reads this
        rank's groups out of them.  Call before every step; descriptors are patched only when a pointer changed."""
        ptrs = []
        for g, n in zip(grads, self.numels):
            if g.dtype != self.dtype or not g.is_contiguous() or g.numel() != n or g.device != self.device:
                raise RuntimeError("gradients must be contiguous tensors of the parameters' dtype, size and device")
            ptrs.append(g.data_ptr())
        if self._tl is not None and self._full_grads is not None:
            for i, (a, b) in enumerate(zip(ptrs, self._full_grads)):
                if a != b:
                    self._tl[i].g = a
        else:
            self._tl = None
        self._full_grads = ptrs
        self._full_grad_tensors = list(grads)  # kept alive until the next step replaces them

    def _update(self, lo, hi, hyper=None, peers=True):
        """Update global groups ``[lo, hi)`` (a sub-range of the owned range) on the current stream.  ``hyper``:
        a dict with lr / betas / eps / weight_decay for this launch (a parameter group's), default the
        constructor's.  ``peers=False``: no stores into the peers' buffers (measurement of the local update)."""
        from . import _native as N
        if self._tl is None:
            desc = self.descriptors()
            arr = (N.Tensor * len(desc))()
            for i, (p, g, m, v, sm, sv, n, kind) in enumerate(desc):
                arr[i] = N.Tensor(p, g, m, v, sm or None, sv or None, n, kind, 0)
            self._tl = arr
        hp = hyper if hyper is not None else self.hyper
        b1, b2 = hp["betas"]
        h = N.Hyper(b1, b2, hp["lr"], hp["weight_decay"], hp["eps"], float(self.step_count))
        flags = 0 if self.exact_params else N.FLAG_PARAMS_WITHIN_TOLERANCE
        nt = len(self.numels)
        with torch.cuda.device(self.device):
            qm, qv = ctypes.c_void_p(self.qmap_m.data_ptr()), ctypes.c_void_p(self.qmap_v.data_ptr())
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            offs = n_offs = None
            if peers and self.peer_offsets:
                offs = (ctypes.c_int64 * len(self.peer_offsets))(*self.peer_offsets)
                n_offs = len(self.peer_offsets)
            if self.dtype != torch.float32:
                dt = N.DTYPE_BF16 if self.dtype == torch.bfloat16 else N.DTYPE_FP16
                if offs is not None:
                    N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_peers(self._tl, nt, dt, qm, qv, h, lo, hi, offs,
                                                                               n_offs, flags, st))
                else:
                    N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_16bit_flags(self._tl, nt, dt, qm, qv, h, lo, hi, flags, st))
            elif self.reduce_grads and peers:
                goffs = (ctypes.c_int64 * len(self.grad_offsets))(*self.grad_offsets)
                N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_zero1(self._tl, nt, qm, qv, h, lo, hi, offs, n_offs, goffs,
                                                                     len(self.grad_offsets), self.grad_scale, st))
            elif offs is not None:
                N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_peers_flags(self._tl, nt, qm, qv, h, lo, hi, offs, n_offs,
                                                                           flags, st))
            else:
                N.check(N.lib.lpmm_b200_adamw4bit_multi_tensor_flags(self._tl, nt, qm, qv, h, lo, hi, flags, st))
        if peers and self.gather == "copy":
            self._push_to_peers(lo, hi)
        elif peers and self.replica is not None:
            self._narrow(lo, hi)

    def _narrow(self, lo, hi):
        """The 16-bit replica of groups ``[lo, hi)`` from the fp32 master parameters, on the current stream."""
        from . import _native as N
        e0, n = lo * GROUP, (hi - lo) * GROUP
        dt = N.DTYPE_BF16 if self.replica.dtype == torch.bfloat16 else N.DTYPE_FP16
        with torch.cuda.device(self.device):
            N.check(N.lib.lpmm_b200_narrow_fp32(ctypes.c_void_p(self.flat.data_ptr() + 4 * e0),
                                                ctypes.c_void_p(self.replica.data_ptr() + 2 * e0), n, dt,
                                                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def _push_to_peers(self, lo, hi):
        """gather="copy": once the launches enqueued so far have finished, the copy engines write groups ``[lo, hi)``
        of the flat buffer into every peer's copy (one stream, peers in rank order starting after this rank, so that
        ranks in step send to different peers); the caller's stream goes on with the next range meanwhile."""
        main = torch.cuda.current_stream(self.device)
        src, peers = self.flat, self._peer_flats
        if self.replica is not None:  # fp32 master parameters stay here; the peers get the 16-bit replica of the range
            self._narrow(lo, hi)
            src, peers = self.replica, self._peer_replicas
        ev = torch.cuda.Event()
        ev.record(main)
        self._peer_stream.wait_event(ev)
        e0, e1 = lo * GROUP, hi * GROUP
        with torch.cuda.stream(self._peer_stream):
            for peer in peers:
                peer[e0:e1].copy_(src[e0:e1], non_blocking=True)

    def _update_in_chunks(self, lo, hi, hyper=None):
        """``_update`` of ``[lo, hi)``; with gather="copy" in ranges of ``copy_chunk_bytes(world)`` so that the copies of
        one range run while the next is being updated."""
        if self.gather != "copy":
            return self._update(lo, hi, hyper=hyper)
        per = max(1, copy_chunk_bytes(self.world) // (GROUP * self.esize))
        a, n = lo, max(1, per // 8)  # a short first range: the copy engines start early
        while a < hi:
            b = min(a + n, hi)
            self._update(a, b, hyper=hyper)
            a, n = b, per

    def _pre_step_barrier(self):
        """gather="fused": the launch stores into every peer's parameter buffer, so no rank may start it while another
        still reads its parameters (forward / backward of a slower rank), and with reduce_grads every rank's gradients
        must be complete before any rank reads them.  One tiny all-reduce on the stream orders the ranks; the one
        after the update (in _gather) keeps parameters and gradients from being touched while a peer still writes or
        reads them."""
        if self.gather in ("fused", "copy"):
            dist.all_reduce(self._flag, group=self.pg)

    def _gather(self):
        if self.world == 1:
            return
        if self.gather == "copy":
            torch.cuda.current_stream(self.device).wait_stream(self._peer_stream)
        if self.gather in ("fused", "copy"):
            # every peer's copy has been written (by the launch, or by the copies just waited for); order the ranks
            dist.all_reduce(self._flag, group=self.pg)
            return
        S = self.shard_groups * GROUP
        dist.all_gather_into_tensor(self.flat, self.flat[self.rank * S:(self.rank + 1) * S], group=self.pg)

    def step(self):
        self.step_count += 1
        self._pre_step_barrier()
        if self.hi > self.lo:
            self._update_in_chunks(self.lo, self.hi)
        self._gather()

    def step_from_host(self, host_shard, chunk_bytes=256 << 20):
        """One step whose gradient shard arrives from (pinned) host memory: ``host_shard`` holds what ``grad_shard``
        would, ``shard_groups * 128`` elements.  It is copied chunk by chunk on a copy stream, and every chunk that has
        landed is followed by a launch over just its groups, so the update and its stores to the peers overlap the
        remaining copies; the step ends one chunk's update after the last byte arrives.  Results are those of
        ``grad_shard.copy_(host_shard); step()``."""
        if self._full_grads is not None or self.reduce_grads:
            raise RuntimeError("step_from_host feeds grad_shard; it does not combine with use_full_grads / reduce_grads")
        if host_shard.numel() != self.grad_shard.numel() or host_shard.dtype != self.dtype:
            raise RuntimeError("host_shard must have the size and dtype of grad_shard")
        if self.device.type != "cuda":  # nothing to overlap
            self.grad_shard.copy_(host_shard.view(-1))
            return self.step()
        self.step_count += 1
        self._pre_step_barrier()
        main = torch.cuda.current_stream(self.device)
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        cs = self._copy_stream
        cs.wait_stream(main)  # launches already enqueued may still read grad_shard
        per = max(1, int(chunk_bytes) // (GROUP * self.esize))  # groups per chunk
        src = host_shard.view(-1)
        for a in range(self.lo, self.hi, per):
            b = min(a + per, self.hi)
            e0, e1 = (a - self.lo) * GROUP, (b - self.lo) * GROUP
            with torch.cuda.stream(cs):
                self.grad_shard[e0:e1].copy_(src[e0:e1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(cs)
            main.wait_event(ev)
            self._update(a, b)
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
    def bytes_per_param(self, small=False):
        """Algorithmic bytes per parameter of the update: p read + write, g read, for 4-bit tensors two codes read +
        write and two fp32 scales per 128 elements, for small tensors two fp32 moments read + write."""
        return (2 * self.esize + self.esize + 16.0) if small else (3 * self.esize + 2.0 + 0.125)

    def time_update_only(self, iters, peers=True):
        """Mean duration (ms) of the sharded update launch alone and its algorithmic bytes.  ``peers=False``: without
        the stores into the peers' buffers (the local update: leaves the replicas inconsistent; measurement only)."""
        ms = []
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.step_count += 1
            a.record()
            self._update(self.lo, self.hi, peers=peers)
            b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        nbytes = 0.0
        for i, a_, b_ in owned_pieces(self.numels, self.gstart, self.lo, self.hi):
            cnt = min(b_ * GROUP, self.numels[i]) - a_ * GROUP
            nbytes += cnt * self.bytes_per_param(self.numels[i] <= THRESHOLD)
        return sum(ms) / len(ms), nbytes

    def breakdown(self, iters):
        """Update-only and all-gather-only timings, max over ranks."""
        upd, _ = self.time_update_only(iters, peers=self.gather != "copy")
        ms = []
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier(group=self.pg)
            a.record()
            if self.gather == "copy" and self.hi > self.lo:
                self._push_to_peers(self.lo, self.hi)  # the whole shard to every peer, nothing to overlap with
            self._gather()
            b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        t = torch.tensor([upd, sum(ms) / len(ms)], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.pg)
        upd_ms, ag_ms = float(t[0]), float(t[1])
        total = sum(self.numels)
        recv = float(self.xsize) * self.shard_groups * GROUP * (self.world - 1)
        if self.gather == "fused":
            return {"update_with_peer_stores": {"ms": upd_ms, "aggregate_params_per_s": total / (upd_ms * 1e-3),
                                                "nvlink_bytes_sent_per_rank": recv,
                                                "nvlink_gb_per_s_per_rank": recv / (upd_ms * 1e-3) / 1e9},
                    "rank_barrier": {"ms": ag_ms}}
        if self.gather == "copy":
            return {"update_only": {"ms": upd_ms, "aggregate_params_per_s": total / (upd_ms * 1e-3)},
                    "peer_copies_of_the_shard": {"ms": ag_ms, "bytes_received_per_rank": recv,
                                                 "gb_per_s_per_rank": recv / (ag_ms * 1e-3) / 1e9}}
        return {"update_only": {"ms": upd_ms, "aggregate_params_per_s": total / (upd_ms * 1e-3)},
                "all_gather": {"ms": ag_ms, "bytes_received_per_rank": recv, "gb_per_s_per_rank": recv / (ag_ms * 1e-3) / 1e9}}

    def flat_checksum(self):
        """A 64-bit checksum of the whole parameter buffer (sum of its 32-bit words as integers, in chunks)."""
        words = self.flat.view(torch.int32)
        total = torch.zeros((), dtype=torch.int64, device=self.device)
        chunk = 1 << 27
        for lo in range(0, words.numel(), chunk):
            total += words[lo:lo + chunk].sum(dtype=torch.int64)
        return total


class ZeroAdamW(torch.optim.Optimizer):
    """``lpmm.optim.AdamW(params, fused=True)`` with its states ZeRO-1 sharded over the ranks of a process group.

    The model's parameters are adopted into one flat buffer (``p.data`` becomes a view that starts on a
    128-element group boundary; with ``gather="fused"`` the buffer lives in symmetric memory and the update kernel
    writes every rank's copy, with ``gather="copy"`` the copy engines do while the next range is updated).  Every rank must construct it from identical parameters (a replicated model) and must
    call ``step()`` with identical, already reduced gradients in ``p.grad`` (what data-parallel backward with an
    all-reduce leaves): each rank reads only its own groups out of them, nothing is copied.  Parameter groups keep
    their own ``lr`` / ``betas`` / ``eps`` / ``weight_decay``, read at every step (schedulers work), one launch per
    group (per 1-2 GB range of a group with ``gather="copy"``).  ``state_dict()`` gathers the shards into exactly what the unsharded optimizer's ``state_dict()`` holds
    (the reference's fused layout, lpmm/optim/adamw.py:508-523: ``int8[(numel + 1) // 2]`` codes, fp32 group
    maxima in ``overhead['max1']``, fp32 moments for tensors of at most 4096 elements) and ``load_state_dict`` takes
    such a dict, so checkpoints move freely between the two.  Both are collective calls.
    Not covered: sparse or missing gradients (every parameter needs one), parameter groups added later,
    configurations other than the fused step's (4-bit group-128 states)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, *, process_group=None,
                 gather="nccl", exact_params=True, engine_cls=None):
        from .config import get_config
        hyper = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        # the same group keys as lpmm.optim.AdamW(fused=True), so that state dicts are interchangeable
        defaults = dict(hyper, fused=True, use_first_moment=True, factor_second_moment=False)
        super().__init__(params, defaults)
        plist = [p for g in self.param_groups for p in g["params"]]
        if not plist:
            raise ValueError("ZeroAdamW got an empty parameter list")
        dev, dt = plist[0].device, plist[0].dtype
        if any(p.device != dev or p.dtype != dt for p in plist):
            raise ValueError("all parameters must share one device and one dtype")
        self._plist = plist
        self.qconfig = get_config(None)
        self.engine = (engine_cls or Zero1FusedAdamW)([tuple(p.shape) for p in plist], dev, process_group=process_group,
                                                      gather=gather, dtype=dt, exact_params=exact_params, **hyper)
        with torch.no_grad():
            for p, view in zip(plist, self.engine.params):
                view.copy_(p.detach())
                p.data = view
        # global group range of every parameter group (its tensors are consecutive in the flat buffer)
        self._ranges, i = [], 0
        eng = self.engine
        for g in self.param_groups:
            k = len(g["params"])
            beg = eng.gstart[i] if k else 0
            end = (eng.gstart[i + k] if i + k < len(plist) else eng.total_groups) if k else 0
            self._ranges.append((beg, end))
            i += k

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        eng = self.engine
        grads = []
        for p in self._plist:
            if p.grad is None:
                raise RuntimeError("ZeroAdamW needs a gradient for every parameter")
            if p.grad.is_sparse:
                raise RuntimeError("AdamW does not support sparse gradients")
            grads.append(p.grad)
        eng.use_full_grads(grads)
        eng.step_count += 1
        eng._pre_step_barrier()
        for (beg, end), group in zip(self._ranges, self.param_groups):
            lo, hi = max(eng.lo, beg), min(eng.hi, end)
            if lo < hi:
                eng._update_in_chunks(lo, hi, hyper=group)
        eng._gather()
        return loss

    @torch.no_grad()
    def step_from_host(self, host_grads, chunk_bytes=256 << 20):
        """One step whose (already reduced) gradients arrive from host memory: ``host_grads`` holds one CPU tensor per
        parameter (pinned, for the copies to be asynchronous), in the order of ``param_groups``.  Only this rank's
        slices are copied into ``p.grad`` (allocated here if missing; the rest of a ``p.grad`` is left as it is), on a
        copy stream, and every ``chunk_bytes`` that have landed are followed by a launch over just those groups, so
        update and peer stores overlap the remaining copies.  Results are those of ``step()`` on the same gradients."""
        eng = self.engine
        host = list(host_grads)
        if len(host) != len(self._plist):
            raise ValueError(f"expected {len(self._plist)} host gradients, got {len(host)}")
        grads = []
        for p, h in zip(self._plist, host):
            if h is None:
                raise RuntimeError("ZeroAdamW needs a gradient for every parameter")
            if h.numel() != p.numel() or h.dtype != p.dtype:
                raise RuntimeError("a host gradient must have its parameter's size and dtype")
            if p.grad is None:
                p.grad = torch.empty_like(p, memory_format=torch.contiguous_format)
            grads.append(p.grad)
        eng.use_full_grads(grads)
        owner = [gi for gi, g in enumerate(self.param_groups) for _ in g["params"]]
        pieces = owned_pieces(eng.numels, eng.gstart, eng.lo, eng.hi)
        cuda = eng.device.type == "cuda"
        eng.step_count += 1
        eng._pre_step_barrier()
        if cuda:
            main = torch.cuda.current_stream(eng.device)
            if getattr(eng, "_copy_stream", None) is None:
                eng._copy_stream = torch.cuda.Stream(device=eng.device)
            cs = eng._copy_stream
            cs.wait_stream(main)  # launches already enqueued may still read the gradients
        run_lo, run_hi, pending = None, None, 0
        for k, (i, a, b) in enumerate(pieces):
            e0, e1 = a * GROUP, min(b * GROUP, eng.numels[i])
            dst, src = grads[i].view(-1)[e0:e1], host[i].view(-1)[e0:e1]
            if cuda:
                with torch.cuda.stream(cs):
                    dst.copy_(src, non_blocking=True)
            else:
                dst.copy_(src)
            if run_lo is None:
                run_lo = eng.gstart[i] + a
            run_hi = eng.gstart[i] + b
            pending += (e1 - e0) * eng.esize
            last = k + 1 == len(pieces)
            if last or pending >= chunk_bytes or owner[pieces[k + 1][0]] != owner[i]:  # a launch stays inside one group
                if cuda:
                    ev = torch.cuda.Event()
                    ev.record(cs)
                    main.wait_event(ev)
                eng._update(run_lo, run_hi, hyper=self.param_groups[owner[i]])
                run_lo, pending = None, 0
        eng._gather()

    def state_dict(self):
        """Collective.  The unsharded optimizer's ``state_dict()``: every rank returns the full state."""
        eng = self.engine
        full = eng.gather_state()
        self.state.clear()
        for p, st in zip(self._plist, full):
            quant = p.numel() > THRESHOLD
            oh_m, oh_v = {}, {}
            m, v = st["exp_avg"], st["exp_avg_sq"]
            if quant:
                oh_m["max1"], oh_v["max1"] = st["exp_avg_scale"], st["exp_avg_sq_scale"]
            else:
                m, v = m.view(p.shape), v.view(p.shape)
            self.state[p] = {
                "step": torch.tensor(float(st["step"])),
                "exp_avg": m,
                "exp_avg_qstate": {"enable": quant, "overhead": oh_m, "qmap": eng.qmap_m},
                "exp_avg_sq": v,
                "exp_avg_sq_qstate": {"enable": quant, "overhead": oh_v, "qmap": eng.qmap_v},
            }
        sd = super().state_dict()
        self.state.clear()  # the live state is the engine's shards
        sd["qconfig"] = self.qconfig
        return sd

    def load_state_dict(self, state_dict):
        """Collective in the sense that every rank must load the same dict; each keeps its own range."""
        groups, saved = self.param_groups, state_dict["param_groups"]
        if len(groups) != len(saved) or any(len(g["params"]) != len(s["params"]) for g, s in zip(groups, saved)):
            raise ValueError("loaded state dict does not match the optimizer's parameter groups")
        for g, s in zip(groups, saved):
            for k, val in s.items():
                if k != "params":
                    g[k] = val
        ids = [i for s in saved for i in s["params"]]
        states = []
        for idx, p in zip(ids, self._plist):
            st = state_dict["state"].get(idx)
            if st is None:
                raise ValueError("ZeroAdamW needs the state of every parameter")
            entry = {"step": float(st["step"]), "exp_avg": st["exp_avg"], "exp_avg_sq": st["exp_avg_sq"]}
            if p.numel() > THRESHOLD:
                entry["exp_avg_scale"] = st["exp_avg_qstate"]["overhead"]["max1"]
                entry["exp_avg_sq_scale"] = st["exp_avg_sq_qstate"]["overhead"]["max1"]
            states.append(entry)
        self.engine.load_full_state(states)
        if "qconfig" in state_dict:
            self.qconfig = state_dict["qconfig"]
