"""Unsloth at its best settings (packing + its trainer) against this framework's packed LoRA run.

Reference: benchmarks/unsloth_max_benchmark.py (hard-codes the reference's own 11,699 tok/s at :378 as
the number to compare with).  Unsloth and TRL are not installed here and need a model hub, so the
Unsloth arm reports why it was skipped; the comparison constant is kept, labelled as published.
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

from benchmarks.run_benchmark import benchmark_chronicals  # noqa: E402

CHRONICALS_PUBLISHED_LORA_TOK_S = 11_699.0      # reference README, 1x A100-40GB
UNSLOTH_PUBLISHED_LORA_TOK_S = 2_857.0          # same table ("Unsloth MAX")


def benchmark_unsloth_max(a) -> dict:
    try:
        import unsloth  # noqa: F401
        import trl  # noqa: F401
    except Exception as e:
        return {"method": "unsloth_max", "status": "skipped", "reason": f"{type(e).__name__}: unsloth/trl not installed"}
    return {"method": "unsloth_max", "status": "skipped", "reason": "needs network access for its model hub"}


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
    theirs = benchmark_unsloth_max(a)
    print(json.dumps(ours))
    print(json.dumps(theirs))
    print(f"published (A100-40GB): reference LoRA {CHRONICALS_PUBLISHED_LORA_TOK_S:,.0f} tok/s, Unsloth MAX "
          f"{UNSLOTH_PUBLISHED_LORA_TOK_S:,.0f} tok/s; measured here: {ours['tokens_per_sec']:,.0f} tok/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
