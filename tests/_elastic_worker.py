"""Worker for the elastic-restart test (gloo ranks on CPU).

    _elastic_worker.py <dir> <mode> save      trains 2 steps, writes a checkpoint, trains 2 more and records their losses
    _elastic_worker.py <dir> <mode> resume    loads that checkpoint at THIS world size and records the same 2 losses

``mode`` picks the optimizer layout: ``dp`` (replicated AdamW state), ``zero1`` (sharded state), ``zero3`` (sharded
parameters and state).  The global batch is fixed (4 rows), so every world size sees the same data."""
import json
import os
import sys

import torch
import torch.distributed as dist

from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
from chronicals_b200.parallel.bootstrap import init_distributed, shutdown

GLOBAL_ROWS, STEPS, SAVE_AT = 4, 4, 2


def make_args(out, mode, world):
    a = TrainingConfig(output_dir=out, num_train_epochs=1, gradient_accumulation_steps=1, learning_rate=2e-3,
                       lr_scheduler_type="constant", warmup_ratio=0.0, logging_steps=1, save_steps=0, bf16=False,
                       fp8=False, use_gradient_checkpointing=False, visual_reporting=False, z_loss_weight=0.0,
                       max_grad_norm=0.5)
    a.shift_labels = False
    a.save_final = False
    a.log_jsonl = False
    a.parallel.comm_backend = "gloo"
    if world > 1:
        a.parallel.zero_stage = {"dp": 0, "zero1": 1, "zero3": 3}[mode]
        a.parallel.shard_bucket_mb = 0.25
    return a


def main():
    root, mode, phase = sys.argv[1], sys.argv[2], sys.argv[3]
    rank, _, world = init_distributed("gloo")
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers, cfg.vocab_size, cfg.dtype = 2, 1024, "float32"
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (STEPS, GLOBAL_ROWS, 49), generator=g)
    per = GLOBAL_ROWS // world
    mine = [{"input_ids": ids[s, rank * per:(rank + 1) * per, :-1].contiguous(),
             "labels": ids[s, rank * per:(rank + 1) * per, 1:].contiguous()} for s in range(STEPS)]
    model = build_model(cfg, dtype=torch.float32, seed=0 if phase == "save" else 99)
    tr = ChronicalsTrainer(model, make_args(os.path.join(root, f"run_{phase}_{world}"), mode, world), mine)
    ck = os.path.join(root, "ckpt")

    def global_loss(step):
        t = tr.training_step(mine[step]).detach().float().reshape(1).clone()
        if world > 1:
            dist.all_reduce(t)
        return float(t) / world

    losses = []
    if phase == "save":
        for s in range(SAVE_AT):
            global_loss(s)
            tr.state.global_step += 1
        tr.args.output_dir = root
        tr.save_checkpoint("ckpt")
    else:
        tr.load_checkpoint(ck)
    for s in range(SAVE_AT, STEPS):
        losses.append(global_loss(s))
    if rank == 0:
        with open(os.path.join(root, f"{phase}_{world}.json"), "w") as f:
            json.dump({"losses": losses, "world": world, "step_count": int(getattr(tr.optimizer, "step_count", 0) or
                                                                           getattr(getattr(tr.optimizer, "engine", None),
                                                                                   "step_count", 0))}, f)
    if world > 1:
        dist.barrier()
    shutdown()


if __name__ == "__main__":
    main()
