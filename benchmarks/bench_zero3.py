"""ZeRO-3 training step (parameters, gradients and AdamW state sharded over the ranks).

No counterpart in the reference (single GPU).  Launch with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29562 benchmarks/bench_zero3.py --model qwen2.5-7b --steps 5 --warmup 3

Every rank processes its own ``batch x seq`` tokens (weak scaling); the step is forward + backward with
per-layer parameter all-gather / gradient reduce-scatter by peer loads, and the sharded AdamW update.
Device-timed with CUDA events, maximum over ranks, one JSON line from rank 0.
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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-prefetch", action="store_true")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="fused: gathers / reduce-scatters by peer-memory kernels; nccl: all_gather_into_tensor and "
                         "reduce_scatter_tensor on the same schedule (comparison arm)")
    ap.add_argument("--fp8", default="none", choices=["none", "rowwise", "mxfp8"],
                    help="forward projections on FP8 operands (rowwise: e4m3 tensor-core GEMM; mxfp8: MX block scales applied by the block-scaled tensor-core GEMM, also in backward)")
    a = ap.parse_args()
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from chronicals_b200 import ChronicalsConfig, build_model
    from chronicals_b200.ops import _ext
    from chronicals_b200.parallel.bootstrap import init_distributed, max_over_ranks, shutdown
    from chronicals_b200.parallel.zero3 import Zero3Engine
    rank, local, world = init_distributed("nccl", timeout_s=180)
    if world < 2:
        print(json.dumps({"unavailable": "bench_zero3 needs at least 2 ranks"}))
        return 0
    dev = torch.device("cuda", local)
    cfg = ChronicalsConfig.from_model_name(a.model)
    if a.layers:
        cfg.num_hidden_layers = a.layers
    model = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=None)
    n_params = sum(p.numel() for p in model.parameters())
    if a.fp8 != "none":
        from chronicals_b200.utils.fp8_deepseek import convert_model_to_fp8
        convert_model_to_fp8(model, exclude_patterns=[], mode=a.fp8)
    eng = Zero3Engine(model, lr=1e-5, weight_decay=0.01, max_grad_norm=1.0, prefetch=not a.no_prefetch, backend=a.comm)
    torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(100 + rank)
    batches = [torch.randint(0, cfg.vocab_size, (a.batch, a.seq), generator=g).to(dev) for _ in range(4)]

    def step(i):
        ids = batches[i % len(batches)]
        loss = eng.forward_backward(ids, labels=ids)
        eng.step()
        return loss

    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    torch.distributed.barrier()
    torch.cuda.reset_peak_memory_stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(i)
    e1.record()
    torch.cuda.synchronize()
    torch.distributed.barrier()
    ms = max_over_ranks(e0.elapsed_time(e1), dev) / a.steps
    _ext.check_status(dev)
    tokens = a.batch * a.seq * world
    if rank == 0:
        print(json.dumps({"bench": "zero3_step", "model": a.model, "layers": cfg.num_hidden_layers, "n_gpus": world,
                          "tokens_per_step": tokens, "ms_per_step": ms, "tokens_per_sec": tokens / (ms / 1e3),
                          "n_params": n_params, "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
                          "mfu_6N_vs_2250TF": 6.0 * n_params * tokens / (ms / 1e3) / (2250e12 * world),
                          "prefetch": not a.no_prefetch, "fp8": a.fp8, "comm": a.comm, "batch": a.batch, "seq": a.seq, "loss": float(loss), "dtype": "bf16",
                          "data": "synthetic token ids, random-init weights"}), flush=True)
    shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
