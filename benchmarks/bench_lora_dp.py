"""LoRA+ fine-tune on packed variable-length documents, data-parallel over N GPUs.

Configuration: Qwen2.5-0.5B architecture, frozen bf16 base, LoRA rank 16 / alpha 32 / dropout 0 on
q, k, v, o, gate, up, down, LoRA+ with the B matrices at 16x the A learning rate; documents with lengths
drawn lognormal(mu 5.5, sigma 1.0) clipped to [32, 2048], seeded uniform token ids, greedy-packed into
4096-token rows with ``cu_seqlens`` for varlen attention; ``--rows`` rows per GPU per step.  Only the
adapter gradients are reduced across ranks (small buckets: all-reduce by peer loads, or NCCL with
``--comm nccl``).  The reference's LoRA numbers are single-GPU (benchmarks/run_benchmark.py:1878-2228).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29563 benchmarks/bench_lora_dp.py --steps 10 --warmup 3

Runs on one GPU without a launcher too.  Device-timed with CUDA events, maximum over ranks; tokens/s
counts every token of the packed rows (padding included, as the reference's methodology does).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def lognormal_documents(n: int, vocab: int, seed: int, mu: float = 5.5, sigma: float = 1.0, lo: int = 32, hi: int = 2048):
    g = torch.Generator().manual_seed(seed)
    lens = torch.exp(torch.randn(n, generator=g) * sigma + mu).clamp(lo, hi).long().tolist()
    return [{"input_ids": torch.randint(0, vocab, (L,), generator=g), "labels": None} for L in lens]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--rows", type=int, default=2, help="packed rows of --row-len tokens per GPU per step")
    ap.add_argument("--row-len", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rank-r", type=int, default=16)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--no-graph", action="store_true", help="launch the step kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--max-docs", type=int, default=0, help="documents per batch the captured graph is sized for "
                                                            "(0: the largest count among the generated batches)")
    a = ap.parse_args()
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
    from chronicals_b200.data.data_loader import create_packed_dataloader
    from chronicals_b200.lora import apply_lora_to_model, count_lora_params
    from chronicals_b200.ops import _ext
    from chronicals_b200.parallel.bootstrap import init_distributed, max_over_ranks, shutdown
    cuda = torch.cuda.is_available()
    rank, local, world = init_distributed("nccl" if cuda else "gloo", timeout_s=180)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    cfg = ChronicalsConfig.from_model_name(a.model)
    model = build_model(cfg, dtype=torch.bfloat16 if cuda else torch.float32, device=dev, seed=1234)
    apply_lora_to_model(model, rank=a.rank_r, alpha=2.0 * a.rank_r)
    trainable, total = count_lora_params(model)
    targs = TrainingConfig(output_dir=os.path.join("/tmp", f"cb_lora_{os.getpid()}"), per_device_train_batch_size=a.rows,
                           max_seq_length=a.row_len, gradient_accumulation_steps=1, learning_rate=2e-4, weight_decay=0.0,
                           max_grad_norm=1.0, lr_scheduler_type="constant", warmup_ratio=0.0, bf16=cuda, fp8=False,
                           use_gradient_checkpointing=False, use_sequence_packing=True, logging_steps=10 ** 9, save_steps=0,
                           visual_reporting=False, optimizer_type="lora_plus", seed=1234,
                           use_cuda_graphs=cuda and not a.no_graph and a.comm == "fused")
    targs.lora_plus_ratio = 16.0
    targs.save_final = False
    targs.log_jsonl = False
    targs.parallel.dp = world
    targs.parallel.comm_backend = a.comm
    n_steps = a.warmup + a.steps
    docs = lognormal_documents(int(n_steps * a.rows * world * a.row_len / 350) + 64, cfg.vocab_size, 99)
    for d in docs:
        d["labels"] = d["input_ids"]
    loader = create_packed_dataloader(docs, batch_size=a.rows, max_length=a.row_len, strategy="greedy", rank=rank,
                                      world_size=world, pin_memory=True)
    batches = [b for _, b in zip(range(n_steps), loader)]
    if len(batches) < n_steps:
        batches = (batches * (n_steps // max(1, len(batches)) + 1))[:n_steps]
    targs.cuda_graph_max_documents = a.max_docs or max(int(b["cu_seqlens"].numel()) - 1 for b in batches)
    if world > 1:
        t = torch.tensor([targs.cuda_graph_max_documents], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        targs.cuda_graph_max_documents = int(t.item())
    trainer = ChronicalsTrainer(model, targs, None)
    real = sum(int((b["labels"] != -100).sum()) for b in batches[a.warmup:])
    for b in batches[: a.warmup]:
        trainer.training_step(b)
    if cuda:
        torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    l0 = _ext.launches()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    else:
        import time
        t0 = time.perf_counter()
    for b in batches[a.warmup:]:
        loss = trainer.training_step(b)
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        elapsed = e0.elapsed_time(e1)
    else:
        elapsed = 1e3 * (time.perf_counter() - t0)
    if world > 1:
        torch.distributed.barrier()
    ms = max_over_ranks(elapsed, dev) / a.steps
    if cuda:
        _ext.check_status(dev)
    tokens = a.rows * a.row_len * world
    if rank == 0:
        print(json.dumps({"bench": "lora_plus_packed_dp", "model": a.model, "n_gpus": world, "lora_rank": a.rank_r,
                          "trainable_params": trainable, "total_params": total, "tokens_per_step": tokens,
                          "ms_per_step": ms, "tokens_per_sec": tokens / (ms / 1e3),
                          "non_masked_token_fraction_rank0": real / (a.steps * a.rows * a.row_len),
                          "vs_published_lora_a100": tokens / (ms / 1e3) / 11699.0, "comm": a.comm if world > 1 else "none",
                          "cuda_graph": bool(trainer.use_cuda_graphs),
                          "kernel_launches_per_step": (trainer.graph_kernel_launches if trainer.use_cuda_graphs
                                                       else (_ext.launches() - l0) // a.steps),
                          "documents_per_batch_max": int(targs.cuda_graph_max_documents),
                          "loss": float(loss), "dtype": "bf16", "data": "synthetic lognormal-length documents, random-init weights"}),
              flush=True)
    shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
