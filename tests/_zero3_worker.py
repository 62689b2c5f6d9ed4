"""Worker: ZeRO-3 engine (gloo on CPU / fused kernels on GPUs) against single-process AdamW on the joint batch."""
import json
import os
import sys

import torch
import torch.distributed as dist

from chronicals_b200 import ChronicalsConfig, build_model
from chronicals_b200.parallel.bootstrap import init_distributed, shutdown
from chronicals_b200.parallel.zero3 import Zero3Engine


def main():
    out, backend = sys.argv[1], sys.argv[2]
    use_cuda = backend != "gloo"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, local, world = init_distributed("nccl" if use_cuda else "gloo", timeout_s=60)
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    dtype = torch.bfloat16 if use_cuda else torch.float32
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers, cfg.vocab_size = 3, 2048
    steps, per, S = 3, 2, 64
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (steps, per * world, S), generator=g)
    model = build_model(cfg, dtype=dtype, device=dev, seed=0)
    ref = build_model(cfg, dtype=dtype, device=dev, seed=0)
    hyper = dict(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    eng = Zero3Engine(model, max_grad_norm=1.0, backend="nccl" if backend == "nccl" else "fused", **hyper)
    if use_cuda:
        from chronicals_b200.optimizers import FusedAdamW
        opt = FusedAdamW(ref.parameters(), max_grad_norm=1.0, **hyper)
    else:
        opt = torch.optim.AdamW(ref.parameters(), **hyper)
    z_losses, r_losses = [], []
    for s in range(steps):
        mine = ids[s, rank * per:(rank + 1) * per].to(dev)
        z_losses.append(float(eng.forward_backward(mine, labels=mine)))
        eng.step()
        # reference: gradients averaged over the per-rank micro-batches, as data parallelism defines them
        for r in range(world):
            b = ids[s, r * per:(r + 1) * per].to(dev)
            loss = ref(b, labels=b).loss
            (loss / world).backward()
            if r == rank:
                r_losses.append(float(loss))
        if not use_cuda:
            torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
    if use_cuda:
        torch.cuda.synchronize()
        from chronicals_b200.ops import _ext
        _ext.check_status(dev)
    full = eng.gather_full_state_dict()
    want = ref.hf_state_dict()
    diff = max((full[k].float() - want[k].float()).abs().max().item() for k in want)
    t = torch.tensor([diff], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        with open(out, "w") as f:
            json.dump({"zero3_losses": z_losses, "ref_losses": r_losses, "max_param_diff": float(t),
                       "grad_norm": float(eng.last_grad_norm)}, f)
    shutdown()


if __name__ == "__main__":
    main()
