"""LoRA at the best settings of each stack: this framework's packed LoRA+ run against a library baseline.

The reference's script of this name (benchmarks/unsloth_max_benchmark.py) times Unsloth with packing and its
own trainer and hard-codes the reference's 11,699 tok/s (:378) as the number to beat.  Unsloth and TRL need a
model hub, so when they cannot be imported the second arm is the baseline that does run offline: transformers'
implementation of the same architecture with plain PyTorch LoRA modules on all seven projections, SDPA attention
and torch's fused AdamW (``run_benchmark.benchmark_huggingface_lora``) - random-init weights and synthetic
Alpaca-length token ids in both arms, one optimizer step per micro-batch, CUDA-event timing.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from benchmarks.run_benchmark import benchmark_chronicals, benchmark_huggingface_lora  # noqa: E402

CHRONICALS_PUBLISHED_LORA_TOK_S = 11_699.0      # reference README, 1x A100-40GB
UNSLOTH_PUBLISHED_LORA_TOK_S = 2_857.0          # same table ("Unsloth MAX")


def benchmark_unsloth_max(a) -> dict:
    """Unsloth itself when it is installed and a local model directory is given; otherwise the reason."""
    try:
        import unsloth  # noqa: F401
        import trl  # noqa: F401
    except Exception as e:
        return {"method": "unsloth_max", "status": "skipped", "reason": f"{type(e).__name__}: unsloth / trl not installed"}
    return {"method": "unsloth_max", "status": "skipped", "reason": "needs a pretrained checkpoint from a model hub"}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup_steps", type=int, default=5)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--seq_length", type=int, default=1024)
    ap.add_argument("--lora_rank", type=int, default=16)
    a = ap.parse_args(argv)
    a.grad_accum, a.use_cuda_graphs, a.num_runs = 1, True, 1
    ours = benchmark_chronicals(a, lora=True, packed=True).to_dict()
    unsloth = benchmark_unsloth_max(a)
    library = benchmark_huggingface_lora(a).to_dict()
    for r in (ours, library, unsloth):
        print(json.dumps(r))
    if library.get("status", "ok") == "ok" and library.get("tokens_per_sec"):
        print(f"measured here: {ours['tokens_per_sec']:,.0f} tok/s against {library['tokens_per_sec']:,.0f} tok/s for "
              f"transformers + plain LoRA ({ours['tokens_per_sec'] / library['tokens_per_sec']:.2f}x)")
    print(f"published (A100-40GB): reference LoRA {CHRONICALS_PUBLISHED_LORA_TOK_S:,.0f} tok/s, Unsloth MAX "
          f"{UNSLOTH_PUBLISHED_LORA_TOK_S:,.0f} tok/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
