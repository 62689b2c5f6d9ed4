"""Tensor parallelism with sequence parallelism and a vocab-parallel fused cross-entropy.

The reference is single-GPU (no tensor, sequence or vocab parallel code anywhere); this module is new.

Layout (Megatron-style, W ranks in the group):

* QKV and gate/up projections are column-parallel (each rank owns ``1/W`` of the heads / of the
  intermediate width); o_proj and down_proj are row-parallel.
* Between those regions the residual stream, the RMSNorms and the residual adds live on ``T/W``
  tokens per rank (sequence parallel).  Entering a column-parallel GEMM the normalised activations are
  all-gathered along tokens; leaving a row-parallel GEMM the partial outputs are reduce-scattered.
* The LM head is sharded along the vocabulary; the cross-entropy runs on the local ``V/W`` columns
  without materialising logits and the per-token (log-sum-exp, target logit) pairs are combined
  across ranks.

Two communication back-ends:

* ``"nccl"`` — ``torch.distributed`` collectives wrapped in autograd functions (gloo on CPU); the
  comparison baseline and the CPU-testable reference of the data flow.
* ``"fused"`` — the kernels of ``csrc/comm.cu`` / ``csrc/gemm.cu`` over peer memory
  (``parallel.tp_fused``): the RMSNorm kernel pushes its rows into every peer's gather buffer and
  raises a per-panel flag, the consuming tcgen05 GEMM waits per token panel (own panel first) while
  it computes; the row-parallel GEMM's epilogue stores each output tile straight into the owning
  rank's staging buffer, and one kernel sums the W partials with the residual.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import _ext, ref


class TPState:
    """The tensor-parallel group of this process and its communication back-end."""

    def __init__(self, group=None, backend: str = "nccl", wait_budget_us: int = 2_000_000):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("tensor parallelism needs an initialised process group")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend = backend
        self.wait_budget_us = wait_budget_us
        self.fused = None                       # parallel.tp_fused.FusedTP, created on first use

    def fused_ops(self, tokens: int, hidden: int, device):
        if self.fused is None:
            from .tp_fused import FusedTP
            self.fused = FusedTP(self, tokens, hidden, device)
        self.fused.ensure(tokens, hidden)
        return self.fused


# ---------------------------------------------------------------------------------------------- collectives
def _all_gather_rows(x: torch.Tensor, tp: TPState) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty((x.shape[0] * tp.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    try:
        dist.all_gather_into_tensor(out, x, group=tp.group)
    except (RuntimeError, NotImplementedError):
        parts = [torch.empty_like(x) for _ in range(tp.world)]
        dist.all_gather(parts, x, group=tp.group)
        out = torch.cat(parts, dim=0)
    return out


def _reduce_scatter_rows(x: torch.Tensor, tp: TPState) -> torch.Tensor:
    x = x.contiguous()
    n = x.shape[0] // tp.world
    if x.is_cuda:
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=tp.group)
        return out
    y = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x.clone()      # gloo: all-reduce, keep my rows
    dist.all_reduce(y, group=tp.group)
    return y[tp.rank * n:(tp.rank + 1) * n].to(x.dtype).contiguous()


class _GatherTokens(torch.autograd.Function):
    """``[T/W, ...] → [T, ...]``; the backward sums the W partial gradients of my rows."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_rows(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_rows(g, ctx.tp), None


class _ScatterSumTokens(torch.autograd.Function):
    """``[T, ...]`` partial sums on every rank → my ``[T/W, ...]`` rows of the total."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _reduce_scatter_rows(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_rows(g, ctx.tp), None


def gather_tokens(x: torch.Tensor, tp: TPState) -> torch.Tensor:
    return _GatherTokens.apply(x, tp)


def scatter_sum_tokens(x: torch.Tensor, tp: TPState) -> torch.Tensor:
    return _ScatterSumTokens.apply(x, tp)


# ---------------------------------------------------------------------------------------------- vocab-parallel CE
def _exchange_lse_tgt(lse_local: torch.Tensor, tgt_local: torch.Tensor, tp: TPState) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combine per-rank (log-sum-exp over the local vocabulary shard, target logit if owned)."""
    if tp.backend == "fused" and lse_local.is_cuda:
        return tp.fused_ops(0, 0, lse_local.device).combine_lse_tgt(lse_local, tgt_local)
    both = torch.stack((lse_local, tgt_local)).contiguous()
    allv = _all_gather_rows(both.unsqueeze(0), tp)             # [W, 2, T]
    return torch.logsumexp(allv[:, 0], dim=0), allv[:, 1].sum(dim=0)


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross-entropy of ``h @ W_shardᵀ`` (columns ``[v0, v0 + Vs)`` of a ``V_total`` vocabulary)
    against global ``labels``; identical value on every rank.  Returns partial ``dh`` (to be summed over
    ranks by the caller's gather backward) and the complete ``dW_shard``."""

    @staticmethod
    def forward(ctx, h, w, labels, tp, v0, v_total, z_weight):
        T, K = h.shape
        Vs = w.shape[0]
        valid = labels != -100
        fast = h.is_cuda and h.dtype == torch.bfloat16 and not _ext.reference_forced() and K % 8 == 0
        if fast:
            L = _ext.lib()
            dev = h.device
            n_splits = L.cb_cce_num_splits(T, Vs)
            part = torch.empty(2, n_splits, T, dtype=torch.float32, device=dev)
            tgt = torch.zeros(T, dtype=torch.float32, device=dev)
            status = _ext.status_buffer(dev)
            _ext.check(L.cb_cce_forward(h.data_ptr(), w.data_ptr(), labels.data_ptr(), T, Vs, K, h.stride(0), w.stride(0),
                                        int(v0), part[0].data_ptr(), part[1].data_ptr(), None, tgt.data_ptr(),
                                        status.data_ptr(), _ext.stream_ptr()), "cce_forward")
            m = part[0].max(dim=0).values
            lse_local = m + torch.log((part[1] * torch.exp(part[0] - m)).sum(dim=0))
            tgt_local = tgt
            logits = None
        else:
            logits = h.float() @ w.float().t()
            lse_local = torch.logsumexp(logits, dim=-1)
            rel = labels - v0
            own = valid & (rel >= 0) & (rel < Vs)
            tgt_local = torch.where(own, logits.gather(1, rel.clamp(0, Vs - 1).unsqueeze(1)).squeeze(1),
                                    torch.zeros_like(lse_local))
        lse, tgt = _exchange_lse_tgt(lse_local, tgt_local, tp)
        n_valid = valid.sum().clamp(min=1).float()
        rows = (lse - tgt) * valid
        if z_weight:
            rows = rows + z_weight * lse * lse * valid
        loss = rows.sum() / n_valid
        ctx.save_for_backward(h, w, labels, lse, (valid.float() / n_valid))
        ctx.cfg = (int(v0), int(v_total), float(z_weight), fast)
        ctx.set_materialize_grads(False)
        return loss

    @staticmethod
    def backward(ctx, gout):
        h, w, labels, lse, gscale = ctx.saved_tensors
        v0, v_total, z_weight, fast = ctx.cfg
        T, K = h.shape
        Vs = w.shape[0]
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if fast:
            L = _ext.lib()
            dev = h.device
            status = _ext.status_buffer(dev)
            g1 = gout.float().reshape(1).contiguous()
            Vc = min(ops.CCE_BWD_CHUNK, (Vs + 7) // 8 * 8)
            G = torch.empty(T, Vc, dtype=torch.bfloat16, device=dev)
            dh32 = torch.empty(T, K, dtype=torch.float32, device=dev) if need_dh else None
            dw = torch.empty_like(w) if need_dw else None
            for c0 in range(0, Vs, Vc):
                vc = min(Vc, Vs - c0)
                wc = w[c0:c0 + vc]
                _ext.check(L.cb_cce_dlogits(h.data_ptr(), wc.data_ptr(), labels.data_ptr(), lse.data_ptr(),
                                            gscale.data_ptr(), g1.data_ptr(), G.data_ptr(), T, vc, K, h.stride(0),
                                            w.stride(0), G.stride(0), v0 + c0, v_total, 0.0, z_weight, status.data_ptr(),
                                            _ext.stream_ptr()), "cce_dlogits")
                Gc = G[:, :vc]
                if need_dh:
                    ops.gemm(Gc, wc, b_mn=True, out=dh32, accumulate=c0 > 0)
                if need_dw:
                    ops.gemm(Gc, h, a_mn=True, b_mn=True, out=dw[c0:c0 + vc])
            return (dh32.to(h.dtype) if need_dh else None), dw, None, None, None, None, None
        logits = h.float() @ w.float().t()
        p = torch.exp(logits - lse.unsqueeze(1)) * (1.0 + 2.0 * z_weight * lse).unsqueeze(1)
        rel = labels - v0
        own = (labels != -100) & (rel >= 0) & (rel < Vs)
        idx = rel.clamp(0, Vs - 1).unsqueeze(1)
        p.scatter_add_(1, idx, -own.float().unsqueeze(1))
        G = p * (gscale * gout.float()).unsqueeze(1)
        dh = (G @ w.float()).to(h.dtype) if need_dh else None
        dw = (G.t() @ h.float()).to(w.dtype) if need_dw else None
        return dh, dw, None, None, None, None, None


def vocab_parallel_cross_entropy(h_full: torch.Tensor, w_shard: torch.Tensor, labels: torch.Tensor, tp: TPState,
                                 v0: int, v_total: int, z_loss_weight: float = 0.0) -> torch.Tensor:
    """``labels`` are already shifted, ``-100`` ignored; ``h_full`` is the gathered ``[T, H]`` hidden state."""
    return _VocabParallelCE.apply(h_full.contiguous(), w_shard, labels.long().contiguous(), tp, v0, v_total,
                                  float(z_loss_weight))


# ---------------------------------------------------------------------------------------------- sharded model
def _rows(w: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    return w[lo:hi].detach().clone().contiguous()


class TPDecoderLayer(nn.Module):
    """One decoder layer holding this rank's shards.  ``x`` is the residual stream on ``T/W`` tokens."""

    def __init__(self, full_layer, cfg, tp: TPState):
        super().__init__()
        W, r = tp.world, tp.rank
        self.tp = tp
        hq, hk, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if hq % W or hk % W or cfg.intermediate_size % W:
            raise ValueError(f"heads ({hq}/{hk}) and intermediate size ({cfg.intermediate_size}) must divide by the "
                             f"tensor-parallel size {W}")
        self.hq, self.hk, self.d = hq // W, hk // W, d
        self.eps = cfg.rms_norm_eps
        a, m = full_layer.self_attn, full_layer.mlp
        self.norm_offset = full_layer.input_layernorm.offset
        self.gelu = m.gelu
        qw = a.qkv_proj.weight
        nq, nk = hq * d, hk * d
        lq, lk = self.hq * d, self.hk * d
        self.qkv_weight = nn.Parameter(torch.cat((_rows(qw, r * lq, (r + 1) * lq), _rows(qw, nq + r * lk, nq + (r + 1) * lk),
                                                  _rows(qw, nq + nk + r * lk, nq + nk + (r + 1) * lk))))
        if a.qkv_proj.bias is not None:
            b = a.qkv_proj.bias
            self.qkv_bias = nn.Parameter(torch.cat((_rows(b, r * lq, (r + 1) * lq), _rows(b, nq + r * lk, nq + (r + 1) * lk),
                                                    _rows(b, nq + nk + r * lk, nq + nk + (r + 1) * lk))))
        else:
            self.qkv_bias = None
        self.o_weight = nn.Parameter(a.o_proj.weight[:, r * lq:(r + 1) * lq].detach().clone().contiguous())
        I = cfg.intermediate_size
        li = I // W
        gw = m.gate_up_proj.weight
        self.gate_up_weight = nn.Parameter(torch.cat((_rows(gw, r * li, (r + 1) * li), _rows(gw, I + r * li, I + (r + 1) * li))))
        self.down_weight = nn.Parameter(m.down_proj.weight[:, r * li:(r + 1) * li].detach().clone().contiguous())
        self.input_norm_weight = nn.Parameter(full_layer.input_layernorm.weight.detach().clone())
        self.post_norm_weight = nn.Parameter(full_layer.post_attention_layernorm.weight.detach().clone())
        self.interleaved_rope = a.interleaved_rope

    def _column(self, x, norm_w, weight, bias):
        """RMSNorm on my tokens → all-gather → column-parallel GEMM."""
        tp = self.tp
        if tp.backend == "fused" and x.is_cuda:
            return tp.fused_ops(x.shape[0] * tp.world, x.shape[1], x.device).norm_gather_linear(
                x, norm_w, self.eps, self.norm_offset, weight, bias)
        h = ops.rmsnorm(x, norm_w, self.eps, self.norm_offset)
        return ops.linear(gather_tokens(h, tp), weight, bias)

    def _row(self, a, weight, x):
        """Row-parallel GEMM → reduce-scatter → residual add on my tokens."""
        tp = self.tp
        if tp.backend == "fused" and a.is_cuda:
            return tp.fused_ops(a.shape[0], weight.shape[0], a.device).linear_scatter_add(a, weight, x)
        return x + scatter_sum_tokens(ops.linear(a, weight), tp)

    def forward(self, x, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host=None):
        qkv = self._column(x, self.input_norm_weight, self.qkv_weight, self.qkv_bias)
        qkv = ops.qk_rope_(qkv, cos, sin, position_ids, self.hq, self.hk, self.d, self.interleaved_rope)
        o = ops.attention_qkv_packed(qkv, cu_seqlens, self.hq, self.hk, self.d, max_seqlen, seqlens_host)
        x = self._row(o, self.o_weight, x)
        gu = self._column(x, self.post_norm_weight, self.gate_up_weight, None)
        act = ops.geglu(gu) if self.gelu else ops.swiglu(gu)
        return self._row(act, self.down_weight, x)


REPLICATED_MARK = "_tp_replicated"


class TensorParallelCausalLM(nn.Module):
    """A ``CausalLM`` re-laid-out for tensor + sequence parallel execution on ``tp.world`` ranks.

    Build it on every rank from the same full model (``from_full``); each rank keeps its shards and the
    small replicated parameters (norm weights, embedding table).  ``forward`` takes the *global* batch
    (identical on all ranks) and returns the global mean loss.  Call :meth:`sync_replicated_grads`
    after ``backward`` and before the optimizer step.
    """

    def __init__(self, full, tp: TPState):
        super().__init__()
        cfg = full.config
        self.config, self.tp = cfg, tp
        W, r = tp.world, tp.rank
        if cfg.vocab_size % W:
            raise ValueError(f"vocabulary size {cfg.vocab_size} must divide by the tensor-parallel size {W}")
        self.embed_tokens = nn.Embedding.from_pretrained(full.model.embed_tokens.weight.detach().clone(), freeze=False)
        self.layers = nn.ModuleList([TPDecoderLayer(l, cfg, tp) for l in full.model.layers])
        self.norm_weight = nn.Parameter(full.model.norm.weight.detach().clone())
        self.norm_offset = full.model.norm.offset
        self.eps = cfg.rms_norm_eps
        self.vs = cfg.vocab_size // W
        self.v0 = r * self.vs
        self.tied = full.lm_head is None
        if not self.tied:
            self.lm_head_weight = nn.Parameter(_rows(full.lm_head.weight, self.v0, self.v0 + self.vs))
        self.embed_scale = full.embed_scale
        self.z_loss_weight = full.z_loss_weight
        self._rope_len = 0
        self._rope_cache: Tuple[Optional[torch.Tensor], Optional[torch.Tensor]] = (None, None)
        for name, p in self.named_parameters():
            # norm weights and the embedding table are replicated: every rank applies them to its own tokens
            if name.endswith("norm_weight") or name.startswith("embed_tokens"):
                setattr(p, REPLICATED_MARK, True)

    @classmethod
    def from_full(cls, full, tp: TPState) -> "TensorParallelCausalLM":
        return cls(full, tp)

    @classmethod
    def from_config(cls, cfg, tp: TPState, dtype=torch.bfloat16, device=None, seed: int = 0, std: float = 0.02
                    ) -> "TensorParallelCausalLM":
        """Random-initialised shards built without ever holding the full model (the full layout exists only
        on the meta device).  Replicated parameters get the same values on every rank; shards differ."""
        from ..models.decoder import CausalLM
        with torch.device("meta"):
            full = CausalLM(cfg, dtype=dtype)
        model = cls(full, tp).to_empty(device=device)
        gdev = torch.device(device) if device is not None else torch.device("cpu")
        shared = torch.Generator(device=gdev).manual_seed(seed)
        own = torch.Generator(device=gdev).manual_seed(seed * 1000 + 17 + tp.rank)
        with torch.no_grad():
            for name, p in model.named_parameters():
                replicated = getattr(p, REPLICATED_MARK, False) or name.endswith("norm_weight") or name.startswith("embed_tokens")
                if name.endswith("norm_weight"):
                    p.fill_(1.0 if model.norm_offset == 0.0 else 0.0)
                elif name.endswith("bias"):
                    p.zero_()
                else:
                    g = shared if replicated else own
                    p.copy_(torch.empty(p.shape, dtype=torch.float32, device=gdev).normal_(0.0, std, generator=g).to(p.dtype))
                if replicated:
                    setattr(p, REPLICATED_MARK, True)
        return model

    def _rope(self, need: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        cos, sin = self._rope_cache
        if cos is None or need > self._rope_len or cos.device != torch.device(device):
            n = max(need, min(self.config.max_position_embeddings, 1 << 16), 16)
            cos, sin = ref.rope_cache(n, self.config.head_dim, self.config.rope_theta, self.config.rope_scaling, device)
            self._rope_cache, self._rope_len = (cos.contiguous(), sin.contiguous()), n
        return self._rope_cache

    def replicated_parameters(self) -> List[nn.Parameter]:
        return [p for p in self.parameters() if getattr(p, REPLICATED_MARK, False)]

    @property
    def output_weight_shard(self) -> torch.Tensor:
        if self.tied:
            return self.embed_tokens.weight[self.v0:self.v0 + self.vs]
        return self.lm_head_weight

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None,
                max_seqlen: Optional[int] = None, seqlens_host: Optional[Sequence[int]] = None, shift_labels: bool = True, **_):
        from ..models.decoder import CausalLMOutput, _positions_from_cu
        tp = self.tp
        dev = input_ids.device
        B, S = input_ids.shape if input_ids.dim() == 2 else (1, input_ids.shape[0])
        T = B * S
        if T % tp.world:
            raise ValueError(f"token count {T} must divide by the tensor-parallel size {tp.world}")
        ids = input_ids.reshape(T)
        derived = cu_seqlens is None
        if derived:
            cu_seqlens = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev)
            max_seqlen = S
            seqlens_host = seqlens_host or [S] * B
        if position_ids is None:
            position_ids = torch.arange(S, device=dev).repeat(B) if derived else _positions_from_cu(cu_seqlens, T)
        pos = position_ids.reshape(T)
        cos, sin = self._rope(max(int(max_seqlen or S), 1), dev)
        Tl = T // tp.world
        mine = slice(tp.rank * Tl, (tp.rank + 1) * Tl)
        x = ops.embedding(ids[mine].contiguous(), self.embed_tokens.weight)
        if self.embed_scale != 1.0:
            x = x * self.embed_scale
        for layer in self.layers:
            x = layer(x, cos, sin, pos, cu_seqlens, max_seqlen, seqlens_host)
        out = CausalLMOutput()
        if labels is not None:
            y = labels.reshape(B, S)
            if shift_labels:
                y = torch.cat((y[:, 1:], torch.full((B, 1), -100, dtype=y.dtype, device=y.device)), dim=1)
            if tp.backend == "fused" and x.is_cuda:
                hf = tp.fused_ops(T, x.shape[1], dev).norm_gather(x, self.norm_weight, self.eps, self.norm_offset)
            else:
                hf = gather_tokens(ops.rmsnorm(x, self.norm_weight, self.eps, self.norm_offset), tp)
            out.loss = vocab_parallel_cross_entropy(hf, self.output_weight_shard, y.reshape(T), tp, self.v0,
                                                    self.config.vocab_size, self.z_loss_weight)
        else:
            out.hidden_states = x
        return out

    @torch.no_grad()
    def sync_replicated_grads(self) -> None:
        """Sum the gradients of replicated parameters over the group (each rank saw only its tokens)."""
        grads = [p.grad for p in self.replicated_parameters() if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=self.tp.group)
        o = 0
        for g in grads:
            n = g.numel()
            g.copy_(flat[o:o + n].view_as(g))
            o += n

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        """Global-norm clipping where the norm spans every rank's shards (replicated tensors counted once);
        all ranks apply the same coefficient, so replicated parameters stay identical.  Returns the norm."""
        sharded = [p.grad for p in self.parameters() if p.grad is not None and not getattr(p, REPLICATED_MARK, False)]
        repl = [p.grad for p in self.replicated_parameters() if p.grad is not None]
        dev = (sharded or repl)[0].device
        sq = torch.zeros(1, dtype=torch.float32, device=dev)
        if sharded:
            sq += torch.stack([g.float().pow(2).sum() for g in sharded]).sum()
        dist.all_reduce(sq, group=self.tp.group)
        if repl:
            sq += torch.stack([g.float().pow(2).sum() for g in repl]).sum()
        norm = sq.sqrt()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        grads = sharded + repl
        torch._foreach_mul_(grads, coef.squeeze(0))
        return norm.squeeze(0)

    @torch.no_grad()
    def gather_full_state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        """Re-assemble HuggingFace-named full tensors on every rank (checkpoint consolidation; not hot)."""
        tp, cfg = self.tp, self.config
        W = tp.world

        def cat_rows(t):
            return _all_gather_rows(t.detach().unsqueeze(0).contiguous(), tp)          # [W, ...]
        sd: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        sd["model.embed_tokens.weight"] = self.embed_tokens.weight.detach()
        d = cfg.head_dim
        for i, l in enumerate(self.layers):
            pre = f"model.layers.{i}."
            lq, lk = l.hq * d, l.hk * d
            qkv = cat_rows(l.qkv_weight)
            sd[pre + "self_attn.q_proj.weight"] = qkv[:, :lq].reshape(W * lq, -1)
            sd[pre + "self_attn.k_proj.weight"] = qkv[:, lq:lq + lk].reshape(W * lk, -1)
            sd[pre + "self_attn.v_proj.weight"] = qkv[:, lq + lk:].reshape(W * lk, -1)
            if l.qkv_bias is not None:
                b = cat_rows(l.qkv_bias)
                sd[pre + "self_attn.q_proj.bias"] = b[:, :lq].reshape(-1)
                sd[pre + "self_attn.k_proj.bias"] = b[:, lq:lq + lk].reshape(-1)
                sd[pre + "self_attn.v_proj.bias"] = b[:, lq + lk:].reshape(-1)
            sd[pre + "self_attn.o_proj.weight"] = torch.cat(list(cat_rows(l.o_weight)), dim=1)
            gu = cat_rows(l.gate_up_weight)
            li = gu.shape[1] // 2
            sd[pre + "mlp.gate_proj.weight"] = gu[:, :li].reshape(W * li, -1)
            sd[pre + "mlp.up_proj.weight"] = gu[:, li:].reshape(W * li, -1)
            sd[pre + "mlp.down_proj.weight"] = torch.cat(list(cat_rows(l.down_weight)), dim=1)
            sd[pre + "input_layernorm.weight"] = l.input_norm_weight.detach()
            sd[pre + "post_attention_layernorm.weight"] = l.post_norm_weight.detach()
        sd["model.norm.weight"] = self.norm_weight.detach()
        if not self.tied:
            sd["lm_head.weight"] = cat_rows(self.lm_head_weight).reshape(cfg.vocab_size, -1)
        return sd
