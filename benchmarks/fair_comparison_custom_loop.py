"""One hand-written training loop shared by every arm, so only the model/kernels/optimizer differ.

Reference: benchmarks/fair_comparison_custom_loop.py (``custom_loop_benchmark`` :153-213, the two
framework set-ups :216-435).  The loop is: forward → loss → backward → optimizer step → zero grads,
device-timed with CUDA events, identical batches for all arms, losses compared at the end.
Arms: this framework's LoRA model with LoRA+ on the fused AdamW; the transformers model with a plain
LoRA wrapper on torch AdamW; Unsloth + 8-bit AdamW when those packages exist (otherwise skipped).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Callable, Dict, List, Optional

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from benchmarks.run_benchmark import CUDATimer, _device, compute_mfu, load_alpaca_dataloader  # noqa: E402


def custom_loop_benchmark(name: str, model, optimizer, batches: List[Dict[str, torch.Tensor]], steps: int, warmup: int,
                          forward: Callable) -> Dict[str, float]:
    """The shared loop.  ``forward(model, batch)`` returns the scalar loss."""
    def one(i):
        loss = forward(model, batches[i % len(batches)])
        loss.backward()
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss
    for i in range(warmup):
        one(i)
    with CUDATimer() as t:
        for i in range(steps):
            loss = one(i)
    tokens = sum(batches[i % len(batches)]["input_ids"].numel() for i in range(steps))
    n_params = sum(p.numel() for p in model.parameters())
    tok_s = tokens / (t.ms / 1e3)
    return {"name": name, "tokens_per_sec": tok_s, "ms_per_step": t.ms / steps, "final_loss": float(loss.item()),
            "mfu": compute_mfu(n_params, tok_s), "trainable": sum(p.numel() for p in model.parameters() if p.requires_grad)}


def setup_chronicals(model_name: str, rank: int, dev):
    from chronicals_b200 import ChronicalsConfig, build_model
    from chronicals_b200.lora import apply_lora_to_model
    from chronicals_b200.optimizers.lora_plus_optimizer import create_lora_plus_optimizer
    cfg = ChronicalsConfig.from_model_name(model_name)
    model = build_model(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev, seed=0)
    apply_lora_to_model(model, rank=rank, alpha=float(rank))          # alpha = r, as in the reference's fair setup
    opt = create_lora_plus_optimizer(model, base_lr=2e-4, lr_ratio=16.0) if dev.type == "cuda" else \
        torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=2e-4)
    return cfg, model, opt, (lambda m, b: m(b["input_ids"], labels=b["labels"]).loss)


def setup_huggingface(model_name: str, rank: int, dev):
    import transformers
    from chronicals_b200 import ChronicalsConfig
    from benchmarks.benchmark_vs_unsloth import wrap_with_plain_lora
    cfg = ChronicalsConfig.from_model_name(model_name)
    hf_cfg = transformers.Qwen2Config(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads, rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
        tie_word_embeddings=cfg.tie_word_embeddings, attn_implementation="sdpa")
    torch.manual_seed(0)
    model = transformers.AutoModelForCausalLM.from_config(hf_cfg).to(dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    wrap_with_plain_lora(model, rank, float(rank))
    model.enable_input_require_grads()
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=2e-4, fused=dev.type == "cuda")
    return cfg, model, opt, (lambda m, b: m(**b).loss)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="same custom loop for every framework")
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--seq_length", type=int, default=1024)
    ap.add_argument("--lora_rank", type=int, default=32)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    dev = _device()
    rows = []
    for name, setup in (("chronicals_b200", setup_chronicals), ("huggingface+plain-lora", setup_huggingface)):
        try:
            cfg, model, opt, fwd = setup(a.model, a.lora_rank, dev)
            batches = [{k: v.to(dev) for k, v in b.items()}
                       for b in load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 4, seed=0)]
            rows.append(custom_loop_benchmark(name, model, opt, batches, a.steps, a.warmup, fwd))
            del model, opt
            if dev.type == "cuda":
                torch.cuda.empty_cache()
        except Exception as e:
            rows.append({"name": name, "error": f"{type(e).__name__}: {e}"[:300]})
        print(json.dumps(rows[-1]), flush=True)
    try:
        import unsloth  # noqa: F401
        rows.append({"name": "unsloth", "error": "needs network access for its model hub"})
    except Exception:
        rows.append({"name": "unsloth", "error": "unsloth is not installed"})
    ok = [r for r in rows if "error" not in r]
    if len(ok) == 2:
        print(f"speed-up {ok[0]['name']} vs {ok[1]['name']}: {ok[0]['tokens_per_sec'] / ok[1]['tokens_per_sec']:.2f}x; "
              f"loss difference {abs(ok[0]['final_loss'] - ok[1]['final_loss']):.3f}")
    if a.output:
        with open(a.output, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
