"""Worker: rank 1 fails between steps; rank 0 must notice before its next launch and keep its state."""
import json
import os
import sys
import time

import torch

from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
from chronicals_b200.parallel.bootstrap import init_distributed
from chronicals_b200.parallel.watchdog import PeerFailure


def main():
    out = sys.argv[1]
    rank, _, world = init_distributed("gloo", timeout_s=30)
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers, cfg.vocab_size = 1, 512
    model = build_model(cfg, dtype=torch.float32, seed=0)
    a = TrainingConfig(output_dir=out + f".r{rank}", max_steps=10, gradient_accumulation_steps=1, logging_steps=100, save_steps=0,
                       visual_reporting=False, fp8=False, use_gradient_checkpointing=False, bf16=False)
    a.save_final = False
    a.log_jsonl = False
    a.parallel.comm_backend = "gloo"
    a.watchdog_interval_s = 0.2
    ids = torch.randint(0, cfg.vocab_size, (12, 2, 16), generator=torch.Generator().manual_seed(rank))
    data = [{"input_ids": ids[i], "labels": ids[i]} for i in range(12)]

    def cb(trainer, state):
        if rank == 1 and state.global_step == 2:
            raise RuntimeError("injected host-side failure on rank 1")
        if rank == 0:
            time.sleep(0.5)                       # rank 1's report is published before rank 0's next check

    tr = ChronicalsTrainer(model, a, data, callbacks=[cb])
    res = {"rank": rank}
    try:
        tr.train()
        res["outcome"] = "finished"
    except PeerFailure as e:
        res["outcome"] = "peer_failure"
        res["failed_rank"] = e.rank
        res["step"] = tr.state.global_step
        res["emergency"] = sorted(os.listdir(a.output_dir)) if os.path.isdir(a.output_dir) else []
    except RuntimeError as e:
        res["outcome"] = "raised:" + str(e)[:40]
    with open(out + f".{rank}.json", "w") as f:
        json.dump(res, f)
    os._exit(0)                                   # no collective shutdown: the peer is gone


if __name__ == "__main__":
    main()
