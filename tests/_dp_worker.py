"""Worker for the gloo data-parallel test (launched by torch.distributed.run, CPU only)."""
import json
import sys

import torch
import torch.distributed as dist

from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
from chronicals_b200.parallel.bootstrap import init_distributed, shutdown


def make_args(out):
    a = TrainingConfig(output_dir=out, num_train_epochs=1, gradient_accumulation_steps=1, learning_rate=1e-3,
                       lr_scheduler_type="constant", warmup_ratio=0.0, logging_steps=1, save_steps=0, bf16=False,
                       fp8=False, use_gradient_checkpointing=False, visual_reporting=False, z_loss_weight=0.0)
    a.shift_labels = False
    a.save_final = False
    a.log_jsonl = False
    a.parallel.comm_backend = "gloo"
    return a


def main():
    out = sys.argv[1]
    zero3 = len(sys.argv) > 2 and sys.argv[2] == "zero3"
    zero1 = len(sys.argv) > 2 and sys.argv[2] == "zero1"
    rank, _, world = init_distributed("gloo")
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers, cfg.vocab_size, cfg.dtype = 2, 2048, "float32"
    g = torch.Generator().manual_seed(0)
    steps, per = 5, 2
    ids = torch.randint(0, cfg.vocab_size, (steps, per * world, 65), generator=g)
    mine = [{"input_ids": ids[s, rank * per:(rank + 1) * per, :-1].contiguous(),
             "labels": ids[s, rank * per:(rank + 1) * per, 1:].contiguous()} for s in range(steps)]
    model = build_model(cfg, dtype=torch.float32, seed=0)
    a1 = make_args(out + f".r{rank}")
    if zero3:
        a1.parallel.zero_stage = 3
        a1.max_grad_norm = 0.5
    if zero1:
        a1.parallel.zero_stage = 1
        a1.parallel.shard_bucket_mb = 0.25           # several buckets, so bucket completion and slicing are exercised
        a1.max_grad_norm = 0.5
    tr = ChronicalsTrainer(model, a1, mine)
    st = tr.train()
    trained = tr.zero3.gather_full_state_dict() if zero3 else None
    dp_losses = [h["loss"] for h in st.log_history if "lr" in h]
    if rank == 0:
        # single-process oracle on the concatenated batch (no process group used by this trainer)
        full = [{"input_ids": ids[s, :, :-1].contiguous(), "labels": ids[s, :, 1:].contiguous()} for s in range(steps)]
        m2 = build_model(cfg, dtype=torch.float32, seed=0)
        a2 = make_args(out + ".single")
        a2.use_distributed = False
        if zero3 or zero1:
            a2.max_grad_norm = 0.5
        t2 = ChronicalsTrainer(m2, a2, full)
        single = [h["loss"] for h in t2.train().log_history if "lr" in h]
        if zero3:
            want = m2.hf_state_dict()
            diff = max((trained[k] - want[k]).abs().max().item() for k in want)
        else:
            diff = max((p - q).abs().max().item() for p, q in zip(model.parameters(), m2.parameters()))
        with open(out, "w") as f:
            json.dump({"dp_losses": dp_losses, "single_losses": single, "max_param_diff": diff,
                       "optimizer": type(tr.optimizer).__name__,
                       "buckets": len(getattr(tr.optimizer, "buckets", []))}, f)
    dist.barrier()
    shutdown()


if __name__ == "__main__":
    main()
