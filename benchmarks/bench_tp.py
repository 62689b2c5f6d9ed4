"""Tensor + sequence parallel training step: fused peer-memory kernels against the NCCL baseline.

No counterpart in the reference (single GPU).  Launch with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29561 benchmarks/bench_tp.py --model qwen2.5-14b --comm fused --steps 5 --warmup 3

Every rank holds 1/W of each projection and of the vocabulary; the step is forward + backward +
replicated-gradient sync + fused AdamW on the local shards, on the same global batch of
``batch x seq`` tokens.  Device-timed with CUDA events, maximum over ranks, one JSON line from rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def micro(tp, cfg, tokens: int, dev, iters: int = 20):
    """All-gather→GEMM and GEMM→reduce-scatter in isolation, fused kernels against NCCL + the same GEMM."""
    import torch.distributed as dist
    from chronicals_b200 import ops
    from chronicals_b200.parallel.bootstrap import max_over_ranks
    W = tp.world
    H, I = cfg.hidden_size, cfg.intermediate_size
    Tl = tokens // W
    g = torch.Generator().manual_seed(tp.rank)
    x = torch.randn(Tl, H, generator=g).to(dev, torch.bfloat16)
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    w_col = (0.02 * torch.randn(2 * I // W, H, generator=g)).to(dev, torch.bfloat16)      # gate_up shard
    w_row = (0.02 * torch.randn(H, I // W, generator=g)).to(dev, torch.bfloat16)          # down shard
    act = torch.randn(tokens, I // W, generator=g).to(dev, torch.bfloat16)
    ft = tp.fused_ops(tokens, H, dev)
    full = torch.empty(tokens, H, device=dev, dtype=torch.bfloat16)
    part_out = torch.empty(Tl, H, device=dev, dtype=torch.bfloat16)

    def nccl_ag_gemm():
        h = ops.rmsnorm(x, nw, 1e-6)
        dist.all_gather_into_tensor(full, h)
        return ops.gemm(full, w_col)

    def fused_ag_gemm():
        hf, _ = ft.push(x, nw, 1e-6, 0.0, 0)
        y = ft.gemm_wait(hf, w_col, None, 0)
        ft.ctx.barrier()            # stands in for the reduce-scatter barrier that separates two pushes in a layer
        return y

    def nccl_gemm_rs():
        p = ops.gemm(act, w_row)
        dist.reduce_scatter_tensor(part_out, p)
        return part_out + x

    def fused_gemm_rs():
        return ft.gemm_push_reduce(act, w_row, x)

    res = {}
    for name, fn in (("ag_gemm_nccl", nccl_ag_gemm), ("ag_gemm_fused", fused_ag_gemm), ("gemm_rs_nccl", nccl_gemm_rs),
                     ("gemm_rs_fused", fused_gemm_rs)):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        res[name + "_us"] = 1e3 * max_over_ranks(e0.elapsed_time(e1), dev) / iters
    res["shapes"] = {"tokens": tokens, "hidden": H, "col_n_per_rank": 2 * I // W, "row_k_per_rank": I // W,
                     "gathered_bytes": tokens * H * 2}
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", action="store_true", help="time AG->GEMM and GEMM->RS in isolation instead of a step")
    ap.add_argument("--model", default="qwen2.5-14b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0: the model's own)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--single-cta", action="store_true", help="keep the fused GEMMs on the single-CTA kernel (no CTA pairs)")
    a = ap.parse_args()
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from chronicals_b200 import ChronicalsConfig
    from chronicals_b200.ops import _ext
    from chronicals_b200.optimizers import FusedAdamW
    from chronicals_b200.parallel.bootstrap import init_distributed, max_over_ranks, shutdown
    from chronicals_b200.parallel.tensor_parallel import TensorParallelCausalLM, TPState
    rank, local, world = init_distributed("nccl", timeout_s=180)
    if world < 2:
        print(json.dumps({"unavailable": "bench_tp needs at least 2 ranks"}))
        return 0
    dev = torch.device("cuda", local)
    cfg = ChronicalsConfig.from_model_name(a.model)
    if a.layers:
        cfg.num_hidden_layers = a.layers
    tp = TPState(backend=a.comm)
    tp.pair_gemm = not a.single_cta
    if a.micro:
        res = micro(tp, cfg, a.batch * a.seq, dev)
        _ext.check_status(dev)
        if rank == 0:
            print(json.dumps({"bench": "tensor_parallel_micro", "model": a.model, "tp": world, "pair_gemm": not a.single_cta,
                              **res}), flush=True)
        shutdown()
        return 0
    model = TensorParallelCausalLM.from_config(cfg, tp, dtype=torch.bfloat16, device=dev, seed=0)
    n_local = sum(p.numel() for p in model.parameters())
    opt = FusedAdamW(model.parameters(), lr=1e-5, weight_decay=0.01, max_grad_norm=1.0)
    g = torch.Generator().manual_seed(0)
    batches = [torch.randint(0, cfg.vocab_size, (a.batch, a.seq), generator=g).to(dev) for _ in range(4)]

    def step(i):
        ids = batches[i % len(batches)]
        loss = model(ids, labels=ids).loss
        loss.backward()
        model.sync_replicated_grads()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    torch.distributed.barrier()
    l0 = _ext.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(i)
    e1.record()
    torch.cuda.synchronize()
    torch.distributed.barrier()
    ms = max_over_ranks(e0.elapsed_time(e1), dev) / a.steps
    _ext.check_status(dev)
    tokens = a.batch * a.seq
    mem = torch.cuda.max_memory_allocated() / 2 ** 30
    if rank == 0:
        print(json.dumps({"bench": "tensor_parallel_step", "model": a.model, "layers": cfg.num_hidden_layers, "tp": world,
                          "comm": a.comm, "pair_gemm": not a.single_cta, "tokens_per_step": tokens, "ms_per_step": ms, "tokens_per_sec": tokens / (ms / 1e3),
                          "params_per_rank": n_local, "peak_mem_gb": mem, "loss": float(loss),
                          "kernel_launches_per_step": (_ext.launches() - l0) // a.steps, "dtype": "bf16",
                          "data": "synthetic token ids, random-init shards"}), flush=True)
    shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
