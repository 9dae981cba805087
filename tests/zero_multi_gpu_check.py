"""Run under torch.distributed.run on 2 or more GPUs (tests/test_gpu_zero_multi.py does): the ZeRO-1 step
with parameters pushed to the peers by stores inside the update kernel, or by copy-engine peer copies of the updated
ranges, equals the ZeRO-1 step followed by an NCCL all-gather, bit for bit, and every rank ends with the same parameter buffer; and the step that also
reduces the gradients of all ranks inside the update kernel equals the step on gradients summed beforehand;
16-bit parameters, the optimizer wrapper and the step fed from pinned host memory likewise.
Prints one OK line per rank."""
import os, sys, torch, torch.distributed as dist
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "low-bit-optimizers_b200"))
from lpmm.zero import Zero1FusedAdamW
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); lr_ = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(lr_); dev = torch.device("cuda", lr_)
dist.init_process_group("nccl", device_id=dev)
shapes = [(300, 128), (4096,), (5000,), (77, 129), (128,), (64, 64, 3), (2048, 1024)]
H = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
opts = {g: Zero1FusedAdamW(shapes, dev, gather=g, **H) for g in ("nccl", "fused", "copy")}
for o in opts.values(): o.init_params_normal_(0.02, seed=0)
for step in range(1, 5):
    grads = []
    for i, s in enumerate(shapes):
        g = torch.Generator(device=dev); g.manual_seed(step * 100003 + i)
        grads.append(torch.randn(s, generator=g, device=dev) * 1e-3)
    for o in opts.values():
        o.set_grad_shard_from_full(grads); o.step()
torch.cuda.synchronize(); dist.barrier()
a, b = opts["nccl"].flat, opts["fused"].flat
same = bool(torch.equal(a.view(torch.int32), b.view(torch.int32)))
same = same and bool(torch.equal(a.view(torch.int32), opts["copy"].flat.view(torch.int32)))  # copy-engine peer copies
chk = torch.tensor([float(b.double().sum())], device=dev, dtype=torch.float64); lst = [torch.zeros_like(chk) for _ in range(world)]
dist.all_gather(lst, chk)
ok = same and all(float(x) == float(lst[0]) for x in lst)
# ---- gradient reduce-scatter inside the update kernel: every rank contributes its own gradients; the result
# must equal the step on gradients summed in rank order and scaled by 1/world with torch ops
red = Zero1FusedAdamW(shapes, dev, gather="fused", reduce_grads=True, **H)
ref = Zero1FusedAdamW(shapes, dev, gather="nccl", **H)
red.init_params_normal_(0.02, seed=0); ref.init_params_normal_(0.02, seed=0)
for step in range(1, 4):
    per_rank = []
    for r in range(world):
        gs = []
        for i, s in enumerate(shapes):
            g = torch.Generator(device=dev); g.manual_seed(step * 100003 + 1000 * r + i)
            gs.append(torch.randn(s, generator=g, device=dev) * 1e-3)
        per_rank.append(gs)
    for i in range(len(shapes)):
        red.grads[i].copy_(per_rank[rank][i])
    summed = []
    for i in range(len(shapes)):
        acc = per_rank[0][i].clone()
        for r in range(1, world):
            acc = acc + per_rank[r][i]
        summed.append(acc * (1.0 / world))
    ref.set_grad_shard_from_full(summed)
    red.step(); ref.step()
torch.cuda.synchronize(); dist.barrier()
same2 = bool(torch.equal(red.flat.view(torch.int32), ref.flat.view(torch.int32)))
ok = ok and same2
# ---- 16-bit parameters: the sharded step with peer stores == the sharded step with an NCCL all-gather == the
# unsharded 16-bit fused step on one GPU (same list, same gradients)
import lpmm
from lpmm import _kernels as K
same3 = True
for dt in (torch.bfloat16, torch.float16):
    zs = {g: Zero1FusedAdamW(shapes, dev, gather=g, dtype=dt, **H) for g in ("nccl", "fused", "copy")}
    for o in zs.values(): o.init_params_normal_(0.02, seed=0)
    torch.manual_seed(0)
    plain = [torch.nn.Parameter(v.detach().clone()) for v in zs["nccl"].params]
    po = lpmm.optim.AdamW(plain, fused=True, **H)
    for step in range(1, 4):
        grads = []
        for i, s in enumerate(shapes):
            g = torch.Generator(device=dev); g.manual_seed(step * 100003 + i)
            grads.append((torch.randn(s, generator=g, device=dev) * 1e-3).to(dt))
        for o in zs.values():
            o.set_grad_shard_from_full(grads); o.step()
        for p, g in zip(plain, grads): p.grad = g
        po.step()
    torch.cuda.synchronize(); dist.barrier()
    a, b = zs["nccl"].flat.view(torch.int16), zs["fused"].flat.view(torch.int16)
    same3 = same3 and bool(torch.equal(a, b)) and bool(torch.equal(a, zs["copy"].flat.view(torch.int16)))
    for v, p in zip(zs["fused"].params, plain):
        same3 = same3 and bool(torch.equal(v.view(-1).view(torch.int16), p.detach().view(-1).view(torch.int16)))
    del zs
# ---- the optimizer wrapper over real parameters: ZeroAdamW (peer stores) == AdamW(fused=True) unsharded
torch.manual_seed(1)
wa = [torch.nn.Parameter(torch.randn(s, device=dev) * 0.02) for s in shapes]
wb = [torch.nn.Parameter(p.detach().clone()) for p in wa]
grp = lambda ps: [dict(params=ps[:3], weight_decay=0.01), dict(params=ps[3:], weight_decay=0.1, lr=2e-3)]
za = lpmm.optim.ZeroAdamW(grp(wa), lr=1e-3, gather="fused")
ob = lpmm.optim.AdamW(grp(wb), lr=1e-3, fused=True)
for step in range(1, 5):
    for i, (x, y) in enumerate(zip(wa, wb)):
        g = torch.Generator(device=dev); g.manual_seed(step * 100003 + 7 * i)
        x.grad = torch.randn(x.shape, generator=g, device=dev) * 1e-3
        y.grad = x.grad.clone()
    if step == 3: za.param_groups[1]["lr"] = ob.param_groups[1]["lr"] = 1e-3
    za.step(); ob.step()
torch.cuda.synchronize(); dist.barrier()
same4 = all(bool(torch.equal(x.detach().view(torch.int32), y.detach().view(torch.int32))) for x, y in zip(wa, wb))
sd_a, sd_b = za.state_dict(), ob.state_dict()
for k in sd_b["state"]:
    for name in ("exp_avg", "exp_avg_sq"):
        same4 = same4 and bool(torch.equal(sd_a["state"][k][name].view(-1).view(torch.uint8), sd_b["state"][k][name].view(-1).view(torch.uint8)))
# ---- gradient shards arriving from pinned host memory, updated chunk by chunk while the copies run (peer stores
# from several launches per step) == the step on a shard copied beforehand
sa = Zero1FusedAdamW(shapes, dev, gather="fused", **H)
sb = Zero1FusedAdamW(shapes, dev, gather="nccl", **H)
sa.init_params_normal_(0.02, seed=0); sb.init_params_normal_(0.02, seed=0)
for step in range(1, 4):
    grads = []
    for i, s in enumerate(shapes):
        g = torch.Generator(device=dev); g.manual_seed(step * 100003 + 13 * i)
        grads.append(torch.randn(s, generator=g, device=dev) * 1e-3)
    sb.set_grad_shard_from_full(grads)
    host = sb.grad_shard.cpu().pin_memory()
    sb.step()
    sa.step_from_host(host, chunk_bytes=1 << 16)
torch.cuda.synchronize(); dist.barrier()
same5 = bool(torch.equal(sa.flat.view(torch.int32), sb.flat.view(torch.int32)))
# the same through the optimizer wrapper: every rank copies only its own slices of the host gradients
wc = [torch.nn.Parameter(p.detach().clone()) for p in wa]
wd = [torch.nn.Parameter(p.detach().clone()) for p in wa]
zc = lpmm.optim.ZeroAdamW(grp(wc), lr=1e-3, gather="copy")
zd = lpmm.optim.ZeroAdamW(grp(wd), lr=1e-3, gather="nccl")
for step in range(1, 4):
    hg = []
    for i, x in enumerate(wc):
        g = torch.Generator(device=dev); g.manual_seed(step * 100003 + 17 * i)
        hg.append((torch.randn(x.shape, generator=g, device=dev) * 1e-3).cpu().pin_memory())
    for y, h in zip(wd, hg): y.grad = h.to(dev)
    zc.step_from_host(hg, chunk_bytes=1 << 16); zd.step()
torch.cuda.synchronize(); dist.barrier()
same5 = same5 and all(bool(torch.equal(x.detach().view(torch.int32), y.detach().view(torch.int32))) for x, y in zip(wc, wd))
# ---- fp32 master parameters per shard with bf16 replicas: the replica equals the narrowed parameters of the plain
# sharded step on every rank, and a rank's own range of master parameters equals that step's fp32 parameters
ma = Zero1FusedAdamW(shapes, dev, gather="copy", replica_dtype=torch.bfloat16, **H)
mb = Zero1FusedAdamW(shapes, dev, gather="nccl", **H)
ma.init_params_normal_(0.02, seed=0); mb.init_params_normal_(0.02, seed=0)
for step in range(1, 4):
    grads = []
    for i, s in enumerate(shapes):
        g = torch.Generator(device=dev); g.manual_seed(step * 100003 + 19 * i)
        grads.append(torch.randn(s, generator=g, device=dev) * 1e-3)
    for o in (ma, mb):
        o.set_grad_shard_from_full(grads); o.step()
torch.cuda.synchronize(); dist.barrier()
own = slice(ma.lo * 128, ma.hi * 128)
same6 = bool(torch.equal(ma.replica.view(torch.int16), mb.flat.to(torch.bfloat16).view(torch.int16)))
same6 = same6 and bool(torch.equal(ma.flat[own].view(torch.int32), mb.flat[own].view(torch.int32)))
ok = ok and same3 and same4 and same5 and same6
print(f"rank {rank}: {'OK' if ok else 'MISMATCH'} (fused == nccl: {same}, in-kernel gradient reduction == summed gradients: {same2}, "
      f"16-bit sharded == unsharded: {same3}, optimizer wrapper == unsharded optimizer: {same4}, "
      f"step_from_host == copy then step: {same5}, fp32 master + bf16 replicas == narrowed parameters: {same6})", flush=True)
dist.destroy_process_group()
