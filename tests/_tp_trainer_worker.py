"""Worker: ChronicalsTrainer with parallel.tp = world over gloo against a single-process trainer."""
import json
import sys

import torch
import torch.distributed as dist

from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
from chronicals_b200.parallel.bootstrap import init_distributed, shutdown


def make_args(out, tp):
    a = TrainingConfig(output_dir=out, num_train_epochs=1, gradient_accumulation_steps=1, learning_rate=1e-3,
                       lr_scheduler_type="constant", warmup_ratio=0.0, logging_steps=1, save_steps=0, bf16=False, fp8=False,
                       use_gradient_checkpointing=False, visual_reporting=False, z_loss_weight=0.0, max_grad_norm=0.5)
    a.log_jsonl = False
    a.save_final = tp > 1
    a.parallel.tp = tp
    a.parallel.comm_backend = "gloo"
    return a


def main():
    out = sys.argv[1]
    rank, _, world = init_distributed("gloo", timeout_s=120)
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers, cfg.vocab_size, cfg.dtype = 2, 2048, "float32"
    g = torch.Generator().manual_seed(0)
    steps = 4
    ids = torch.randint(0, cfg.vocab_size, (steps, 2, 32), generator=g)
    data = [{"input_ids": ids[s], "labels": ids[s]} for s in range(steps)]
    model = build_model(cfg, dtype=torch.float32, seed=0)
    tr = ChronicalsTrainer(model, make_args(out + ".tp", world), data)
    st = tr.train()
    tp_losses = [h["loss"] for h in st.log_history if "lr" in h]
    full_sd = tr.model.gather_full_state_dict()
    if rank == 0:
        m2 = build_model(cfg, dtype=torch.float32, seed=0)
        a2 = make_args(out + ".single", 1)
        a2.use_distributed = False
        t2 = ChronicalsTrainer(m2, a2, data)
        single = [h["loss"] for h in t2.train().log_history if "lr" in h]
        ref = m2.hf_state_dict()
        diff = max((full_sd[k] - ref[k]).abs().max().item() for k in ref)
        from chronicals_b200.checkpoint.io import read_weights
        import os
        saved = read_weights(os.path.join(out + ".tp", "final"))
        saved_diff = max((saved[k].float() - full_sd[k].float()).abs().max().item() for k in full_sd)
        with open(out, "w") as f:
            json.dump({"tp_losses": tp_losses, "single_losses": single, "max_param_diff": diff, "saved_diff": saved_diff}, f)
    dist.barrier()
    shutdown()


if __name__ == "__main__":
    main()
