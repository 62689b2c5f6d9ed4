"""Training-step time of the same model with bf16, row-wise FP8 and MXFP8 projections (1 GPU).

    python benchmarks/bench_fp8_modes.py --model qwen2.5-7b --layers 4 --steps 10 --warmup 3

Each mode builds the model afresh (same seed), runs ``ChronicalsTrainer.training_step`` (forward, backward,
clipping, fused AdamW; eager launches) on synthetic batches resident on the device, and times ``--steps``
steps with CUDA events after ``--warmup`` untimed ones.  One JSON line per mode.

  bf16     every projection on the bf16 tcgen05 GEMMs
  rowwise  forward projections on the e4m3 tensor-core GEMM (per-token x per-channel scales), backward in bf16
  mxfp8    forward, dX and dW on the block-scaled tensor-core GEMM (32-element blocks, e8m0 scales; gradients
           of the output in e5m2), operands quantised on the fly from the bf16 master copies

The reference only simulates FP8 (quantise, dequantise, bf16 matmul: chronicals/utils/fp8_deepseek.py:612-760),
so it has no counterpart of these timings.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_mode(mode: str, a) -> dict:
    from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
    from chronicals_b200.ops import _ext
    on_gpu = torch.cuda.is_available()
    dev = torch.device("cuda", 0) if on_gpu else torch.device("cpu")
    cfg = ChronicalsConfig.from_model_name(a.model)
    if a.layers:
        cfg.num_hidden_layers = a.layers
    model = build_model(cfg, dtype=torch.bfloat16 if on_gpu else torch.float32, device=dev, seed=1234)
    n_params = sum(p.numel() for p in model.parameters())
    if mode != "bf16":
        from chronicals_b200.utils.fp8_deepseek import convert_model_to_fp8
        convert_model_to_fp8(model, exclude_patterns=[], mode=mode)
    targs = TrainingConfig(
        output_dir=os.path.join("/tmp", f"cb_fp8_modes_{os.getpid()}"), num_train_epochs=1,
        per_device_train_batch_size=a.batch, max_seq_length=a.seq, gradient_accumulation_steps=1, learning_rate=1e-5,
        weight_decay=0.01, max_grad_norm=1.0, lr_scheduler_type="constant", warmup_ratio=0.0, bf16=on_gpu, fp8=False,
        use_gradient_checkpointing=False, use_sequence_packing=False, z_loss_weight=0.0, logging_steps=1, save_steps=0,
        visual_reporting=False, use_cuda_graphs=False, seed=1234)
    targs.save_final = False
    targs.log_jsonl = False
    trainer = ChronicalsTrainer(model, targs, train_dataloader=None)
    g = torch.Generator().manual_seed(7)
    batches = []
    for _ in range(4):
        ids = torch.randint(0, cfg.vocab_size, (a.batch, a.seq), generator=g).to(dev)
        batches.append({"input_ids": ids, "labels": ids.clone()})
    for i in range(a.warmup):
        loss = trainer.training_step(batches[i % 4])
    if on_gpu:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.steps):
            loss = trainer.training_step(batches[i % 4])
        e1.record()
        torch.cuda.synchronize()
        _ext.check_status(dev)
        ms = e0.elapsed_time(e1) / a.steps
    else:                                     # functional check of the three modes on a CPU (host clock)
        t0 = time.perf_counter()
        for i in range(a.steps):
            loss = trainer.training_step(batches[i % 4])
        ms = (time.perf_counter() - t0) * 1e3 / a.steps
    out = {"mode": mode, "model": a.model, "layers": cfg.num_hidden_layers, "params": n_params, "tokens_per_step": a.batch * a.seq,
           "ms_per_step": ms, "tokens_per_s": a.batch * a.seq / ms * 1e3, "loss": float(loss.item())}
    out["device"] = "cuda" if on_gpu else "cpu"
    del trainer, model
    if on_gpu:
        torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--modes", default="bf16,rowwise,mxfp8")
    a = ap.parse_args()
    for mode in a.modes.split(","):
        print(json.dumps(run_mode(mode, a)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
