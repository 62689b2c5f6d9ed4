"""Worker for the multi-GPU tests (one process per GPU, launched by torch.distributed.run)."""
import json
import os
import sys

import torch
import torch.distributed as dist

from chronicals_b200.ops import _ext
from chronicals_b200.optimizers.fused_adamw import FusedAdamW
from chronicals_b200.parallel.bootstrap import init_distributed, shutdown


def main():
    out = sys.argv[1]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, local, world = init_distributed("nccl", timeout_s=60)
    dev = torch.device("cuda", local)
    from chronicals_b200.parallel import symm
    from chronicals_b200.parallel.zero import ShardedFusedAdamW
    res = {"world": world}

    # ---- barrier with payload
    ctx = symm.SymmetricContext()
    pay = torch.tensor([float(rank + 1), 0, 0, 0], device=dev)
    got = ctx.barrier(pay).clone()
    torch.cuda.synchronize()
    res["payload_ok"] = [got[r * 4].item() for r in range(world)] == [float(r + 1) for r in range(world)]
    for _ in range(5):
        ctx.barrier()
    torch.cuda.synchronize()
    _ext.check_status(dev)

    # ---- sharded fused AdamW against the single-GPU optimizer on the averaged gradients
    torch.manual_seed(0)
    shapes = [(300, 64), (1000,), (513, 129), (7,)]
    ref_p = [torch.nn.Parameter(torch.randn(*s, device=dev).to(torch.bfloat16)) for s in shapes]
    my_p = [torch.nn.Parameter(p.detach().clone()) for p in ref_p]
    o_ref = FusedAdamW(ref_p, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1.0)
    o_my = ShardedFusedAdamW(my_p, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1.0)
    for step in range(4):
        gens = [torch.Generator(device="cpu").manual_seed(100 * step + r) for r in range(world)]
        all_g = [[torch.randn(*s, generator=gens[r]).to(torch.bfloat16) for s in shapes] for r in range(world)]
        for i, (p, q) in enumerate(zip(ref_p, my_p)):
            avg = sum(all_g[r][i].float() for r in range(world)) / world
            p.grad = avg.to(torch.bfloat16).to(dev)
            q.grad = all_g[rank][i].to(dev)
        o_ref.step()
        o_my.step()
    torch.cuda.synchronize()
    _ext.check_status(dev)
    err = max((p.float() - q.float()).abs().max().item() for p, q in zip(ref_p, my_p))
    res["adamw_max_err"] = err
    res["norm"] = [o_ref.last_grad_norm.item(), o_my.last_grad_norm.item()]
    # every rank must hold identical parameters
    flat = torch.cat([q.detach().float().reshape(-1) for q in my_p])
    lo, hi = flat.clone(), flat.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    res["ranks_identical"] = bool(torch.equal(lo, hi))
    # canary words behind every symmetric buffer are intact and the barrier epochs only ever grew
    res["canaries_ok"] = all(b.canary_ok() for b in (o_my.param_buf, o_my.grad_buf, o_my.ctx.pad, ctx.pad))
    res["epochs"] = [int(ctx.epoch_ctr.item()), int(o_my.ctx.epoch_ctr.item())]
    res["buckets"] = len(o_my.buckets)

    # ---- the same optimizer fed by a backward pass: several buckets, each reduce-scattered on the side stream from
    # the gradient hooks while the backward pass continues; eager steps, then the step replayed from a CUDA graph
    torch.manual_seed(1)
    dims = [(256, 384), (384,), (384, 256), (256,), (512, 256)]
    ref_q = [torch.nn.Parameter((torch.randn(*s2, device=dev) * 0.1).to(torch.bfloat16)) for s2 in dims]
    my_q = [torch.nn.Parameter(p.detach().clone()) for p in ref_q]
    o_ref2 = FusedAdamW(ref_q, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1.0)
    o_my2 = ShardedFusedAdamW(my_q, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1.0, bucket_mb=0.1,
                              overlap=True, rs_grid=64)
    res["hook_buckets"] = len(o_my2.buckets)

    def loss_fn(ps, x):
        h = torch.tanh(x @ ps[0] + ps[1]) @ ps[2] + ps[3]
        return (h @ ps[4].t()).float().pow(2).mean()

    def batches(step):
        return [torch.randn(64, 256, generator=torch.Generator().manual_seed(1000 * step + r)).to(torch.bfloat16).to(dev)
                for r in range(world)]

    def ref_step(step):
        per_rank = []
        for x in batches(step):
            for p in ref_q:
                p.grad = None
            loss_fn(ref_q, x).backward()
            per_rank.append([p.grad.float() for p in ref_q])       # each rank contributes its bf16 gradient
        for i, p in enumerate(ref_q):
            p.grad = (sum(g[i] for g in per_rank) / world).to(torch.bfloat16)
        o_ref2.step()

    for step in range(3):
        ref_step(step)
        loss_fn(my_q, batches(step)[rank]).backward()
        o_my2.step()
    torch.cuda.synchronize()
    _ext.check_status(dev)
    res["hook_max_err"] = max((p.float() - q.float()).abs().max().item() for p, q in zip(ref_q, my_q))
    res["hook_norm"] = [o_ref2.last_grad_norm.item(), o_my2.last_grad_norm.item()]
    # whole step (backward with hooks, side-stream reduce-scatters, update, all-gather) as one CUDA graph
    static_x = batches(3)[rank].clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        loss_fn(my_q, static_x).backward()                          # warm-up backward that is not followed by a step
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        loss_fn(my_q, static_x).backward()
        o_my2.launch_step()
    for step in range(3, 6):
        ref_step(step)
        static_x.copy_(batches(step)[rank])
        o_my2.prepare_step()
        graph.replay()
    torch.cuda.synchronize()
    _ext.check_status(dev)
    res["graph_max_err"] = max((p.float() - q.float()).abs().max().item() for p, q in zip(ref_q, my_q))
    flat2 = torch.cat([q.detach().float().reshape(-1) for q in my_q])
    lo2, hi2 = flat2.clone(), flat2.clone()
    dist.all_reduce(lo2, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi2, op=dist.ReduceOp.MAX)
    res["hook_ranks_identical"] = bool(torch.equal(lo2, hi2))
    del graph

    # ---- bounded wait: a barrier nobody else joins gives up with an error status instead of hanging
    if os.environ.get("CB_TEST_TIMEOUT", "1") == "1":
        lone = symm.SymmetricContext(wait_budget_us=2000)
        dist.barrier()
        if rank == 0:
            lone.barrier()                      # rank 1.. never call it
            torch.cuda.synchronize()
            try:
                _ext.check_status(dev)
                res["timeout_detected"] = False
            except _ext.KernelError as e:
                res["timeout_detected"] = "201" in str(e)
        dist.barrier()
    if rank == 0:
        with open(out, "w") as f:
            json.dump(res, f)
    shutdown()


if __name__ == "__main__":
    main()
