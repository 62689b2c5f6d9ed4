"""Llama-family decoder (Qwen2 / Llama / Mistral / Gemma) in packed-token layout.

The reference trains HuggingFace ``transformers`` models and monkey-patches
fused kernels into them (chronicals/training/chronicals_trainer.py:704-816).
This framework owns the model instead: activations are ``[T, hidden]`` with
``T`` the packed token count of the micro-batch, documents are described by
``cu_seqlens`` + ``position_ids``, and every block calls the fused ops in
``chronicals_b200.ops`` directly:

    embedding -> N x [ RMSNorm -> QKV GEMM(+bias) -> QK-RoPE (in place)
                       -> varlen causal GQA attention -> o_proj GEMM(+residual)
                       -> RMSNorm -> gate|up GEMM -> SwiGLU -> down GEMM(+residual) ]
              -> RMSNorm -> fused linear-cross-entropy (logits never materialised)

Projection weights are stored fused (``qkv_proj``, ``gate_up_proj``) so each is
one GEMM; :meth:`CausalLM.hf_state_dict` / :meth:`load_hf_state_dict` convert
to and from the HuggingFace parameter names, so checkpoints stay loadable by
``transformers``.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as _checkpoint

from .. import ops
from ..config.config import ChronicalsConfig
from ..ops import ref


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    z_loss: Optional[torch.Tensor] = None

    def __getitem__(self, k):
        return getattr(self, k)


class FusedLinear(nn.Module):
    """Several projections sharing one input, stored as one ``[sum(out), in]`` weight.

    ``splits`` maps the HuggingFace sub-module name (``q_proj`` …) to its output
    width.  Optional per-split LoRA adapters (PEFT convention: ``A [r, in]``,
    ``B [out, r]``, ``y += (alpha / r) * B (A x)``) are attached by
    ``chronicals_b200.lora``; their parameters are named ``lora_A.<split>`` /
    ``lora_B.<split>`` so LoRA+ grouping by name works.
    """

    def __init__(self, in_features: int, splits: "OrderedDict[str, int]", bias: bool = False,
                 dtype=torch.float32, device=None):
        super().__init__()
        self.in_features = in_features
        self.splits = OrderedDict(splits)
        self.out_features = sum(self.splits.values())
        self.weight = nn.Parameter(torch.empty(self.out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(self.out_features, dtype=dtype, device=device)) if bias else None
        self.lora_A = nn.ParameterDict()
        self.lora_B = nn.ParameterDict()
        self.lora_scaling: Dict[str, float] = {}
        self.lora_dropout_p = 0.0
        self.lora_merged = False

    def split_slices(self) -> Dict[str, slice]:
        out, o = {}, 0
        for name, n in self.splits.items():
            out[name] = slice(o, o + n)
            o += n
        return out

    # -- LoRA ---------------------------------------------------------------------------------------
    def add_lora(self, split: str, rank: int, alpha: float, dropout: float = 0.0, init: str = "kaiming") -> None:
        n_out = self.splits[split]
        dev, dt = self.weight.device, self.weight.dtype
        a = torch.empty(rank, self.in_features, device=dev, dtype=torch.float32)
        if init == "zeros":
            a.zero_()
        else:
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        self.lora_A[split] = nn.Parameter(a.to(dt))
        self.lora_B[split] = nn.Parameter(torch.zeros(n_out, rank, device=dev, dtype=dt))
        self.lora_scaling[split] = alpha / rank
        self.lora_dropout_p = dropout

    @property
    def has_lora(self) -> bool:
        return len(self.lora_A) > 0

    def lora_delta(self, split: str) -> torch.Tensor:
        return (self.lora_B[split].float() @ self.lora_A[split].float()) * self.lora_scaling[split]

    @torch.no_grad()
    def merge_lora(self) -> None:
        if self.lora_merged:
            return
        sl = self.split_slices()
        for s in self.lora_A:
            self.weight[sl[s]] += self.lora_delta(s).to(self.weight.dtype)
        self.lora_merged = True

    @torch.no_grad()
    def unmerge_lora(self) -> None:
        if not self.lora_merged:
            return
        sl = self.split_slices()
        for s in self.lora_A:
            self.weight[sl[s]] -= self.lora_delta(s).to(self.weight.dtype)
        self.lora_merged = False

    def is_plain(self) -> bool:
        """No adapter branch and no FP8 path: the projection is one bf16 GEMM on ``weight``."""
        return (not (self.has_lora and not self.lora_merged) and not getattr(self, "use_fp8_rowwise", False)
                and not getattr(self, "use_mxfp8", False))

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.has_lora and not self.lora_merged:
            from ..lora.functional import fused_lora_forward
            return fused_lora_forward(self, x, residual)
        if getattr(self, "use_fp8_rowwise", False) and self.in_features % 16 == 0:
            from ..utils.fp8_utils import fp8_rowwise_linear
            y = fp8_rowwise_linear(x, self.weight, self.bias)
            return y if residual is None else y + residual
        if getattr(self, "use_mxfp8", False) and self.in_features % 32 == 0:
            from ..utils.fp8_utils import _MXFP8LinearFn
            y = _MXFP8LinearFn.apply(x, self.weight, self.bias)
            return y if residual is None else y + residual
        return ops.linear(x, self.weight, self.bias, residual)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, splits={dict(self.splits)}, bias={self.bias is not None}, lora={list(self.lora_A)}"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, offset: float = 0.0, dtype=torch.float32, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device) if offset == 0.0
                                   else torch.zeros(dim, dtype=dtype, device=device))
        self.eps = eps
        self.offset = offset

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.offset)

    def with_residual(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return ops.rmsnorm_residual(x, self.weight, self.eps, self.offset)


class Attention(nn.Module):
    def __init__(self, cfg: ChronicalsConfig, dtype, device=None):
        super().__init__()
        self.hq, self.hk, self.d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.qkv_proj = FusedLinear(cfg.hidden_size, OrderedDict(
            q_proj=self.hq * self.d, k_proj=self.hk * self.d, v_proj=self.hk * self.d),
            bias=cfg.attention_bias, dtype=dtype, device=device)
        self.o_proj = FusedLinear(self.hq * self.d, OrderedDict(o_proj=cfg.hidden_size), bias=False, dtype=dtype,
                                  device=device)
        self.interleaved_rope = False

    def forward(self, x, residual, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host):
        T = x.shape[0]
        qkv = self.qkv_proj(x)
        qkv = ops.qk_rope_(qkv, cos, sin, position_ids, self.hq, self.hk, self.d, self.interleaved_rope)
        o = ops.attention_qkv_packed(qkv, cu_seqlens, self.hq, self.hk, self.d, max_seqlen, seqlens_host)
        return self.o_proj(o, residual)


class MLP(nn.Module):
    def __init__(self, cfg: ChronicalsConfig, dtype, device=None):
        super().__init__()
        self.gate_up_proj = FusedLinear(cfg.hidden_size, OrderedDict(
            gate_proj=cfg.intermediate_size, up_proj=cfg.intermediate_size), bias=False, dtype=dtype, device=device)
        self.down_proj = FusedLinear(cfg.intermediate_size, OrderedDict(down_proj=cfg.hidden_size), bias=False,
                                     dtype=dtype, device=device)
        self.gelu = cfg.hidden_act in ("gelu", "gelu_pytorch_tanh", "gelu_new")

    def forward(self, x, residual):
        fl = self.gate_up_proj
        if not self.gelu and fl.is_plain():
            a = ops.linear_swiglu(x, fl.weight, fl.bias)       # activation in the projection's epilogue
        else:
            gu = fl(x)
            a = ops.geglu(gu) if self.gelu else ops.swiglu(gu)
        return self.down_proj(a, residual)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ChronicalsConfig, dtype, device=None, norm_offset: float = 0.0):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, norm_offset, dtype, device)
        self.self_attn = Attention(cfg, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, norm_offset, dtype, device)
        self.mlp = MLP(cfg, dtype, device)
        self._use_checkpoint = False
        self._offload = None            # an ActivationOffloadManager: checkpointed inputs wait in pinned host memory

    def _body(self, h, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host):
        # pre-norm residual blocks: the norm returns the stream itself as second value so that both gradient
        # contributions of the stream meet inside the norm's backward kernel
        n1, r1 = self.input_layernorm.with_residual(h)
        h = self.self_attn(n1, r1, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host)
        n2, r2 = self.post_attention_layernorm.with_residual(h)
        return self.mlp(n2, r2)

    def forward(self, h, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host=None):
        if self._use_checkpoint and self.training and torch.is_grad_enabled():
            if self._offload is not None:
                from ..training.async_activation_offload import OffloadActivations
                with OffloadActivations(manager=self._offload):
                    return _checkpoint(self._body, h, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host,
                                       use_reentrant=False)
            return _checkpoint(self._body, h, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host,
                               use_reentrant=False)
        return self._body(h, cos, sin, position_ids, cu_seqlens, max_seqlen, seqlens_host)


class DecoderModel(nn.Module):
    """``model.*`` of the HF layout: embedding, layers, final norm."""

    def __init__(self, cfg: ChronicalsConfig, dtype, device=None):
        super().__init__()
        off = 1.0 if cfg.model_type.startswith("gemma") else 0.0
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([DecoderLayer(cfg, dtype, device, off) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, off, dtype, device)


class CausalLM(nn.Module):
    """Decoder-only language model with a fused cross-entropy head.

    ``forward`` accepts either ``input_ids [B, S]`` (each row one document unless
    ``cu_seqlens``/``position_ids`` say otherwise) or already flat ``[T]`` ids.
    ``labels`` follow the HuggingFace convention (unshifted) when
    ``shift_labels=True``; pass ``shift_labels=False`` for pre-shifted labels.
    """

    def __init__(self, cfg: ChronicalsConfig, dtype: Optional[torch.dtype] = None, device=None):
        super().__init__()
        self.config = cfg
        dtype = dtype or cfg.torch_dtype
        self.model = DecoderModel(cfg, dtype, device)
        self.lm_head = None
        if not cfg.tie_word_embeddings:
            self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        self.embed_scale = math.sqrt(cfg.hidden_size) if cfg.model_type.startswith("gemma") else 1.0
        self._rope_len = 0
        self.register_buffer("rope_cos", torch.empty(0), persistent=False)
        self.register_buffer("rope_sin", torch.empty(0), persistent=False)
        self.label_smoothing = 0.0
        self.z_loss_weight = 0.0
        self.reset_parameters()

    # -- init -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def reset_parameters(self, std: float = 0.02, seed: Optional[int] = None) -> None:
        gen = None
        if seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() >= 2 and "lora_" not in name:
                if gen is not None:
                    p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=gen).to(p.dtype))
                else:
                    p.normal_(0.0, std)
            elif name.endswith("bias"):
                p.zero_()

    @property
    def output_weight(self) -> torch.Tensor:
        return self.lm_head.weight if self.lm_head is not None else self.model.embed_tokens.weight

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def num_parameters(self, only_trainable: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)

    def gradient_checkpointing_enable(self, ratio: float = 1.0, offload: bool = False, offload_config=None, **_) -> None:
        """Recompute the chosen layers in the backward pass; with ``offload`` the tensors those layers keep for
        it (their inputs) are moved to pinned host memory by one shared ``ActivationOffloadManager``."""
        n = len(self.model.layers)
        k = n if ratio >= 1.0 else max(1, int(round(n * ratio)))
        chosen = set(int(round(i * n / k)) for i in range(k)) if k < n else set(range(n))
        manager = None
        if offload:
            from ..training.async_activation_offload import ActivationOffloadManager
            manager = ActivationOffloadManager(offload_config)
        self.activation_offload = manager
        for i, layer in enumerate(self.model.layers):
            layer._use_checkpoint = i in chosen
            layer._offload = manager if i in chosen else None

    def gradient_checkpointing_disable(self) -> None:
        for layer in self.model.layers:
            layer._use_checkpoint = False
            layer._offload = None

    # -- rope ------------------------------------------------------------------------------------------------
    def _rope(self, need: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        if need > self._rope_len or self.rope_cos.device != torch.device(device):
            n = max(need, min(self.config.max_position_embeddings, 1 << 16), 16)
            n = max(n, need)
            cos, sin = ref.rope_cache(n, self.config.head_dim, self.config.rope_theta, self.config.rope_scaling, device)
            self.rope_cos, self.rope_sin, self._rope_len = cos.contiguous(), sin.contiguous(), n
        return self.rope_cos, self.rope_sin

    def prepare_rope(self, max_pos: int, device=None) -> None:
        """Build the cos/sin tables ahead of time (required before CUDA-graph capture)."""
        self._rope(max_pos, device or self.model.embed_tokens.weight.device)

    # -- forward ---------------------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None,
                seqlens_host: Optional[Sequence[int]] = None, shift_labels: bool = True,
                output_hidden_states: bool = False, return_logits: bool = False, return_dict: bool = True,
                **_) -> CausalLMOutput:
        dev = input_ids.device
        if input_ids.dim() == 2:
            B, S = input_ids.shape
        else:
            B, S = 1, input_ids.shape[0]
        T = B * S
        ids = input_ids.reshape(T)
        derived = False
        if cu_seqlens is None:
            if position_ids is not None and B == 1:
                from ..data.sequence_packer import create_cu_seqlens_from_position_ids
                cu_seqlens, max_seqlen = create_cu_seqlens_from_position_ids(position_ids.reshape(T))
            else:
                cu_seqlens = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev)
                max_seqlen = S
                derived = True
                if seqlens_host is None:
                    seqlens_host = [S] * B
        if position_ids is None:
            position_ids = torch.arange(S, device=dev).repeat(B) if derived else _positions_from_cu(cu_seqlens, T)
        pos = position_ids.reshape(T)
        if max_seqlen is None:
            max_seqlen = S
        cos, sin = self._rope(max(int(max_seqlen), 1), dev)

        h = ops.embedding(ids, self.model.embed_tokens.weight)
        if self.embed_scale != 1.0:
            h = h * self.embed_scale
        for layer in self.model.layers:
            h = layer(h, cos, sin, pos, cu_seqlens, max_seqlen, seqlens_host)
        h = self.model.norm(h)

        out = CausalLMOutput()
        if output_hidden_states:
            out.hidden_states = h.view(B, S, -1)
        if labels is not None:
            y = labels.reshape(B, S)
            if shift_labels:
                y = torch.cat((y[:, 1:], torch.full((B, 1), -100, dtype=y.dtype, device=y.device)), dim=1)
            out.loss = ops.linear_cross_entropy(h, self.output_weight, y.reshape(T), None, -100,
                                                self.label_smoothing, self.z_loss_weight, "mean")
        if return_logits or (labels is None and not output_hidden_states):
            out.logits = torch.nn.functional.linear(h, self.output_weight).view(B, S, -1)
        return out

    # -- HuggingFace-compatible state dict --------------------------------------------------------------------
    def hf_state_dict(self, include_lora: bool = False) -> "OrderedDict[str, torch.Tensor]":
        """Parameters under HuggingFace names (fused projections split; LoRA kept out unless asked)."""
        sd: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        sd["model.embed_tokens.weight"] = self.model.embed_tokens.weight.detach()
        for i, layer in enumerate(self.model.layers):
            pre = f"model.layers.{i}."
            for mod_name, fl in (("self_attn", layer.self_attn.qkv_proj), ("self_attn", layer.self_attn.o_proj),
                                 ("mlp", layer.mlp.gate_up_proj), ("mlp", layer.mlp.down_proj)):
                for split, sl in fl.split_slices().items():
                    sd[f"{pre}{mod_name}.{split}.weight"] = fl.weight.detach()[sl]
                    if fl.bias is not None:
                        sd[f"{pre}{mod_name}.{split}.bias"] = fl.bias.detach()[sl]
                    if include_lora and split in fl.lora_A:
                        sd[f"{pre}{mod_name}.{split}.lora_A.weight"] = fl.lora_A[split].detach()
                        sd[f"{pre}{mod_name}.{split}.lora_B.weight"] = fl.lora_B[split].detach()
            sd[pre + "input_layernorm.weight"] = layer.input_layernorm.weight.detach()
            sd[pre + "post_attention_layernorm.weight"] = layer.post_attention_layernorm.weight.detach()
        sd["model.norm.weight"] = self.model.norm.weight.detach()
        if self.lm_head is not None:
            sd["lm_head.weight"] = self.lm_head.weight.detach()
        return sd

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
        """Load tensors stored under HuggingFace names; returns the names that were not found."""
        missing: List[str] = []
        own = self.hf_state_dict(include_lora=True)
        for name, dst in own.items():
            src = sd.get(name)
            if src is None and name == "lm_head.weight" and "model.embed_tokens.weight" in sd:
                src = sd["model.embed_tokens.weight"]
            if src is None:
                if "lora_" not in name:
                    missing.append(name)
                continue
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
            dst.copy_(src.to(dst.dtype))
        if strict and missing:
            raise KeyError(f"missing keys in checkpoint: {missing[:8]}{'…' if len(missing) > 8 else ''}")
        return missing


def _positions_from_cu(cu_seqlens: torch.Tensor, T: int) -> torch.Tensor:
    """``position_ids`` restarting at every document start; padding positions are 0."""
    cu = cu_seqlens.long()
    idx = torch.arange(T, device=cu.device)
    doc = torch.searchsorted(cu[1:].contiguous(), idx, right=True).clamp_max(cu.numel() - 2)
    pos = idx - cu[doc]
    return torch.where(idx < cu[-1], pos, torch.zeros_like(pos))


Qwen2ForCausalLM = CausalLM
LlamaForCausalLM = CausalLM


def build_model(name_or_cfg, dtype: Optional[torch.dtype] = None, device=None, seed: Optional[int] = None) -> CausalLM:
    cfg = name_or_cfg if isinstance(name_or_cfg, ChronicalsConfig) else ChronicalsConfig.from_model_name(name_or_cfg)
    model = CausalLM(cfg, dtype=dtype, device=device)
    if seed is not None:
        model.reset_parameters(seed=seed)
    return model
