"""Worker for the tensor-parallel tests (gloo on CPU, NCCL on GPUs; launched by torch.distributed.run)."""
import json
import os
import sys

import torch
import torch.distributed as dist

from chronicals_b200 import ChronicalsConfig, build_model
from chronicals_b200.parallel.bootstrap import init_distributed, shutdown
from chronicals_b200.parallel.tensor_parallel import TensorParallelCausalLM, TPState


def main():
    out, backend = sys.argv[1], sys.argv[2]
    use_cuda = backend != "gloo"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, local, world = init_distributed("nccl" if use_cuda else "gloo", timeout_s=60)
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    dtype = torch.bfloat16 if use_cuda else torch.float32
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers = 2
    cfg.vocab_size = 4096
    cfg.tie_word_embeddings = sys.argv[3] == "tied"
    if use_cuda:                                   # panel = T / world rows must be a multiple of 128 for the fused path
        B, S = 2, 128 * world
    else:
        B, S = 2, 16 * world
    full = build_model(cfg, dtype=dtype, device=dev, seed=0)
    with torch.no_grad():                           # non-trivial norm weights and biases
        g = torch.Generator().manual_seed(1)
        for n, p in full.named_parameters():
            if p.dim() == 1:
                p.add_((0.1 * torch.randn(p.shape, generator=g)).to(p.dtype).to(dev))
    tp = TPState(backend="fused" if backend.startswith("fused") else "nccl")
    if backend == "fused_pair":
        tp.pair_min_dim = 0                        # the CTA-pair kernels also on these small projections
    elif backend == "fused":
        tp.pair_gemm = False
    model = TensorParallelCausalLM.from_full(full, tp)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=g).to(dev)
    labels = ids.clone()
    labels[0, :5] = -100
    res = {"world": world, "backend": backend}
    losses_tp, losses_full = [], []
    for it in range(2):
        loss = model(ids, labels=labels).loss
        loss.backward()
        ref_loss = full(ids, labels=labels).loss
        ref_loss.backward()
        losses_tp.append(float(loss))
        losses_full.append(float(ref_loss))
    model.sync_replicated_grads()                  # once, on the accumulated gradients
    if use_cuda:
        torch.cuda.synchronize()
        from chronicals_b200.ops import _ext
        _ext.check_status(dev)
    res["loss_tp"], res["loss_full"] = losses_tp, losses_full

    # gradients: re-assemble the sharded ones and compare with the full model's (two accumulated backward passes)
    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12))
    l0, f0 = model.layers[0], full.model.layers[0]
    W = world
    d = cfg.head_dim
    lq = l0.hq * d
    nq = cfg.num_attention_heads * d
    errs = {}
    errs["qkv_q"] = rel(l0.qkv_weight.grad[:lq], f0.self_attn.qkv_proj.weight.grad[rank * lq:(rank + 1) * lq])
    errs["o"] = rel(l0.o_weight.grad, f0.self_attn.o_proj.weight.grad[:, rank * lq:(rank + 1) * lq])
    li = cfg.intermediate_size // W
    errs["gate"] = rel(l0.gate_up_weight.grad[:li], f0.mlp.gate_up_proj.weight.grad[rank * li:(rank + 1) * li])
    errs["down"] = rel(l0.down_weight.grad, f0.mlp.down_proj.weight.grad[:, rank * li:(rank + 1) * li])
    errs["norm"] = rel(l0.input_norm_weight.grad, f0.input_layernorm.weight.grad)
    errs["final_norm"] = rel(model.norm_weight.grad, full.model.norm.weight.grad)
    errs["embed"] = rel(model.embed_tokens.weight.grad, full.model.embed_tokens.weight.grad)
    if l0.qkv_bias is not None:
        errs["qkv_bias"] = rel(l0.qkv_bias.grad[:lq], f0.self_attn.qkv_proj.bias.grad[rank * lq:(rank + 1) * lq])
    if not model.tied:
        errs["lm_head"] = rel(model.lm_head_weight.grad, full.lm_head.weight.grad[model.v0:model.v0 + model.vs])
    t = torch.tensor([max(errs.values())], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["grad_rel_err_max"] = float(t)
    res["grad_rel_errs_rank0"] = errs
    sd = model.gather_full_state_dict()
    full_sd = full.hf_state_dict()
    res["state_dict_ok"] = all(torch.equal(sd[k].cpu(), full_sd[k].cpu()) for k in sd)
    if rank == 0:
        with open(out, "w") as f:
            json.dump(res, f)
    shutdown()


if __name__ == "__main__":
    main()
