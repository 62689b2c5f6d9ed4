"""LoRA head-to-head: this framework's LoRA fine-tune against Unsloth and HuggingFace PEFT-style LoRA.

Reference: benchmarks/benchmark_vs_unsloth.py (``TARGET_THROUGHPUTS`` :51-56,
``benchmark_chronicals_lora`` :279-536, ``benchmark_unsloth_lora`` :543-777,
``benchmark_huggingface_lora`` :784-941, table :948-1031, ``run_full_benchmark`` :1038-1129, CLI :1132-1177).

All arms use rank 16, alpha 32, the seven projection targets and LoRA+ (B matrices at 16x the learning
rate).  The HuggingFace arm is the transformers model with this framework-independent, plain-PyTorch
LoRA wrapper (``PlainLoRALinear`` below: two extra matmuls per projection, autograd backward) and torch's
fused AdamW.  Unsloth needs its package and a model hub; without them the arm reports ``skipped``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from benchmarks.run_benchmark import (BenchmarkResult, _device, _finish, _skipped, _time_steps,  # noqa: E402
                                      benchmark_chronicals_lora, load_alpaca_dataloader, print_comparison)

TARGET_THROUGHPUTS = {"chronicals_lora_a100_published": 11_699.0, "unsloth_lora_a100_published": 2_857.0,
                      "hf_peft_lora_a100_published": 3_420.0}
LORA_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


class PlainLoRALinear(nn.Module):
    """``y = W x + (alpha / r) B A x`` with a frozen ``W`` — the textbook formulation."""

    def __init__(self, base: nn.Linear, rank: int, alpha: float):
        super().__init__()
        self.base = base
        for p in self.base.parameters():
            p.requires_grad_(False)
        self.lora_A = nn.Parameter(torch.empty(rank, base.in_features, dtype=base.weight.dtype, device=base.weight.device))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, rank, dtype=base.weight.dtype, device=base.weight.device))
        nn.init.kaiming_uniform_(self.lora_A, a=5 ** 0.5)
        self.scaling = alpha / rank

    def forward(self, x):
        return self.base(x) + self.scaling * ((x @ self.lora_A.t()) @ self.lora_B.t())


def wrap_with_plain_lora(model: nn.Module, rank: int = 16, alpha: float = 32.0) -> int:
    n = 0
    for p in model.parameters():
        p.requires_grad_(False)
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear) and name in LORA_TARGETS:
                setattr(parent, name, PlainLoRALinear(child, rank, alpha))
                n += 1
    return n


def benchmark_huggingface_lora(a) -> BenchmarkResult:
    try:
        import transformers
    except Exception as e:                               # pragma: no cover
        return BenchmarkResult("huggingface_lora", status="skipped", reason=f"transformers not importable: {e}")
    from chronicals_b200 import ChronicalsConfig
    dev = _device()
    cfg = ChronicalsConfig.from_model_name(a.model)
    hf_cfg = transformers.Qwen2Config(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads, rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
        tie_word_embeddings=cfg.tie_word_embeddings, attn_implementation="sdpa")
    torch.manual_seed(0)
    model = transformers.AutoModelForCausalLM.from_config(hf_cfg).to(dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    wrap_with_plain_lora(model, a.lora_rank, 2.0 * a.lora_rank)
    model.enable_input_require_grads()
    groups = [{"params": [p for n, p in model.named_parameters() if n.endswith("lora_A")], "lr": 2e-4},
              {"params": [p for n, p in model.named_parameters() if n.endswith("lora_B")], "lr": 2e-4 * 16.0}]
    opt = torch.optim.AdamW(groups, weight_decay=0.0, fused=dev.type == "cuda")
    n_params = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for g in groups for p in g["params"])
    data = [{k: v.to(dev) for k, v in b.items()}
            for b in load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 4, seed=0)]

    def step(i):
        loss = model(**data[i % len(data)]).loss
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss
    return _finish("huggingface_lora", a, n_params, trainable, _time_steps(step, a, a.batch_size * a.seq_length))


def run_full_benchmark(a) -> List[BenchmarkResult]:
    arms = [benchmark_chronicals_lora, benchmark_huggingface_lora, _skipped("unsloth_lora", "unsloth")]
    out = []
    for fn in arms:
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats()
        try:
            out.append(fn(a))
        except Exception as e:
            out.append(BenchmarkResult(getattr(fn, "__name__", "arm"), status="failed", reason=f"{type(e).__name__}: {e}"[:300]))
        print(json.dumps(out[-1].to_dict()), flush=True)
    return out


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="LoRA throughput: chronicals_b200 vs HuggingFace-style LoRA vs Unsloth")
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup_steps", type=int, default=5)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--seq_length", type=int, default=1024)
    ap.add_argument("--lora_rank", type=int, default=16)
    ap.add_argument("--num_runs", type=int, default=1)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    a.grad_accum, a.use_cuda_graphs = 1, True
    results = run_full_benchmark(a)
    print_comparison(results)
    print("published on 1x A100-40GB (reference README): " + ", ".join(f"{k} {v:,.0f} tok/s" for k, v in TARGET_THROUGHPUTS.items()))
    if a.output:
        with open(a.output, "w") as f:
            json.dump({"results": [r.to_dict() for r in results], "targets": TARGET_THROUGHPUTS}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
