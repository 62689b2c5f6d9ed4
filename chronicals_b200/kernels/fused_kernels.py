"""Fused op front-ends: functions, autograd-backed modules and losses.

Covers the reference's kernel monolith (chronicals/kernels/triton_kernels.py:
RMSNorm :593-774, SwiGLU / SiLU·Mul :1067-1284, GeGLU :1370-1432, in-place
QK-RoPE :1785-2005, dispatchers and PyTorch fallbacks :2070-2277, chunked and
fused linear cross-entropy :2305-2813 and :3147-3419, Liger-style CE :2979-3125,
RMSNorm→Linear :4199-4303, Embedding(+RoPE) :4426-4560, GQA attention :4701-4791).
Every function dispatches to the sm_100a kernels for CUDA bf16 tensors and to
the PyTorch formulas otherwise; ``chronicals_b200.kernels.triton_kernels`` is an
alias of this module so reference import paths keep working.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import ref
from .cut_cross_entropy import (DEFAULT_CHUNK_SIZE, ChunkedCrossEntropyLoss, CutCrossEntropyLoss, cut_cross_entropy)

# ------------------------------------------------------------------------------------------- RMSNorm
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return ops.rmsnorm(x, weight, eps)


fused_rmsnorm = rmsnorm
rmsnorm_triton = rmsnorm
rmsnorm_with_grad = rmsnorm


def rmsnorm_pytorch(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return ref.rmsnorm(x, weight, eps)


class FusedRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, offset: float = 0.0, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.eps, self.offset = eps, offset

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.offset)


# ------------------------------------------------------------------------------------------- gated activations
def fused_swiglu(gate: torch.Tensor, up: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gate) * up``; with one argument the last dim holds ``gate | up``."""
    if up is None:
        return ops.swiglu(gate)
    return ops.swiglu(torch.cat((gate, up), dim=-1))


fused_swiglu_triton = fused_swiglu


def swiglu_pytorch(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return ref.swiglu(gate, up)


def fused_swiglu_pytorch(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Plain-PyTorch ``silu(gate) * up`` (the reference's fallback, triton_kernels.py:2115-2120)."""
    return torch.nn.functional.silu(gate) * up


def swiglu_with_grad(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``gate * silu(x)`` with autograd through the fused forward / backward kernels (reference
    triton_kernels.py:1217-1240: the FIRST argument goes through the activation)."""
    return fused_swiglu(x, gate)


def fused_geglu(gate: torch.Tensor, up: Optional[torch.Tensor] = None) -> torch.Tensor:
    if up is None:
        return ops.geglu(gate)
    return ops.geglu(torch.cat((gate, up), dim=-1))


class FusedSwiGLU(nn.Module):
    """SwiGLU MLP: one gate|up GEMM, fused activation, down GEMM."""

    def __init__(self, hidden_size: int, intermediate_size: int, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.gate_up_proj = nn.Linear(hidden_size, 2 * intermediate_size, bias=bias, device=device, dtype=dtype)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=bias, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gu = ops.linear(x, self.gate_up_proj.weight, self.gate_up_proj.bias)
        return ops.linear(ops.swiglu(gu), self.down_proj.weight, self.down_proj.bias)


class FusedSiLUMul(nn.Module):
    def forward(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        return fused_swiglu(gate, up)


class FusedGeGLU(nn.Module):
    def forward(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        return fused_geglu(gate, up)


# ------------------------------------------------------------------------------------------- RoPE
def precompute_rope_cache(seq_len: int, head_dim: int, theta: float = 10000.0, device=None,
                          scaling: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``cos, sin`` of shape ``[seq_len, head_dim // 2]`` (fp32)."""
    return ref.rope_cache(seq_len, head_dim, theta, scaling, device)


def _rope_4d(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
             position_ids: Optional[torch.Tensor], interleaved: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q [B, S, Hq, D]``, ``k [B, S, Hk, D]`` → rotated copies (packs into one buffer for the kernel)."""
    B, S, hq, d = q.shape
    hk = k.shape[2]
    if cos.dim() == 2 and cos.shape[-1] == d:           # full-width tables: keep the first half
        cos, sin = cos[..., : d // 2], sin[..., : d // 2]
    T = B * S
    pos = position_ids.reshape(T) if position_ids is not None else torch.arange(S, device=q.device).repeat(B)
    buf = torch.cat((q.reshape(T, hq * d), k.reshape(T, hk * d)), dim=1)
    if ops._fast(buf) and (hq * d + hk * d) % 8 == 0:
        # V is absent: pass a zero-width V by describing only q and k heads
        out = ops.qk_rope_(buf, cos.float().contiguous(), sin.float().contiguous(), pos, hq, hk, d, interleaved)
    else:
        qq = ref.apply_rope(q.reshape(T, hq, d), cos, sin, pos, interleaved)
        kk = ref.apply_rope(k.reshape(T, hk, d), cos, sin, pos, interleaved)
        return qq.view(B, S, hq, d), kk.view(B, S, hk, d)
    return out[:, : hq * d].reshape(B, S, hq, d), out[:, hq * d:].reshape(B, S, hk, d)


def fused_qk_rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                  position_ids: Optional[torch.Tensor] = None, interleaved: bool = False
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotary embedding of Q and K in one launch.  Default is the split-half (HuggingFace) pairing;
    ``interleaved=True`` pairs ``(2i, 2i+1)``."""
    if q.dim() == 3:                                       # packed [T, H, D]
        qq, kk = _rope_4d(q[None], k[None], cos, sin, position_ids[None] if position_ids is not None else None,
                          interleaved)
        return qq[0], kk[0]
    return _rope_4d(q, k, cos, sin, position_ids, interleaved)


fused_qk_rope_inplace = fused_qk_rope


def fused_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, position_ids: Optional[torch.Tensor] = None,
               interleaved: bool = False) -> torch.Tensor:
    """Single-tensor rotary embedding (``[..., T, H, D]``)."""
    d = x.shape[-1]
    if cos.shape[-1] == d:
        cos, sin = cos[..., : d // 2], sin[..., : d // 2]
    return ref.apply_rope(x, cos, sin, position_ids, interleaved)


def fused_rope_pytorch(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split-half rotation of ``q`` / ``k`` (``[batch, seq, heads, head_dim]``) with ``[seq, head_dim / 2]`` tables,
    written with elementary tensor operations (the reference's fallback, triton_kernels.py:2123-2160)."""
    S, d = q.shape[1], q.shape[-1]
    c = torch.cat((cos[:S], cos[:S]), dim=-1)[None, :, None, :].to(q.dtype)
    s = torch.cat((sin[:S], sin[:S]), dim=-1)[None, :, None, :].to(q.dtype)

    def rot(x):
        return torch.cat((-x[..., d // 2:], x[..., : d // 2]), dim=-1)
    return q * c + rot(q) * s, k * c + rot(k) * s


def rope_pytorch(q, k, cos, sin, position_ids=None):
    return fused_rope(q, cos, sin, position_ids), fused_rope(k, cos, sin, position_ids)


# ------------------------------------------------------------------------------------------- cross-entropy
def fused_cross_entropy(*args, **kwargs) -> torch.Tensor:
    """Both documented call forms:

    * ``fused_cross_entropy(logits, targets, vocab_size=…)`` — loss on materialised logits;
    * ``fused_cross_entropy(hidden, lm_head_weight, targets, chunk_size=…)`` — no logits.
    """
    kwargs.pop("vocab_size", None)
    if len(args) >= 3 and isinstance(args[2], torch.Tensor) and not args[2].is_floating_point():
        hidden, weight, targets = args[:3]
        return cut_cross_entropy(hidden, weight, targets, *args[3:], **kwargs)
    logits, targets = args[:2]
    return ops.cross_entropy_logits(logits, targets, kwargs.get("ignore_index", -100),
                                    kwargs.get("label_smoothing", 0.0), kwargs.get("z_loss_weight", 0.0),
                                    kwargs.get("reduction", "mean"))


fused_cross_entropy_triton = fused_cross_entropy
liger_cross_entropy = fused_cross_entropy


def fused_cross_entropy_pytorch(logits: torch.Tensor, labels: torch.Tensor, label_smoothing: float = 0.0,
                                z_loss_weight: float = 1e-4, ignore_index: int = -100
                                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(loss, d loss / d logits)`` from ``torch.nn.functional`` only: mean cross-entropy over the valid labels
    plus ``z_loss_weight * mean(logsumexp²)`` over ALL rows, as the reference's fallback computes it
    (triton_kernels.py:2070-2100)."""
    lg = logits.detach().float().requires_grad_(True)
    with torch.enable_grad():
        flat = lg.reshape(-1, lg.shape[-1])
        loss = torch.nn.functional.cross_entropy(flat, labels.reshape(-1), ignore_index=ignore_index,
                                                 label_smoothing=label_smoothing)
        loss = loss + z_loss_weight * torch.logsumexp(flat, dim=-1).pow(2).mean()
        (g,) = torch.autograd.grad(loss, (lg,))
    return loss.detach(), g.to(logits.dtype)


def cross_entropy_pytorch(logits, targets, ignore_index=-100, label_smoothing=0.0, z_loss_weight=0.0):
    return ref.cross_entropy_logits(logits, targets, ignore_index, label_smoothing, z_loss_weight)


def fused_linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                               bias: Optional[torch.Tensor] = None, chunk_size: int = DEFAULT_CHUNK_SIZE,
                               ignore_index: int = -100, label_smoothing: float = 0.0, z_loss_weight: float = 0.0
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(loss, z_loss)`` like the reference; ``loss`` already contains the z-loss term."""
    loss = cut_cross_entropy(hidden, weight, labels, bias, chunk_size, ignore_index, label_smoothing, z_loss_weight)
    if z_loss_weight:
        with torch.no_grad():
            plain = cut_cross_entropy(hidden.detach(), weight.detach(), labels, bias, chunk_size, ignore_index,
                                      label_smoothing, 0.0)
            z = loss.detach() - plain
    else:
        z = torch.zeros((), device=loss.device, dtype=loss.dtype)
    return loss, z


triton_fused_linear_cross_entropy = fused_linear_cross_entropy
fused_linear_cross_entropy_autograd = fused_linear_cross_entropy


def chunked_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, chunk_size: int = 4096,
                          ignore_index: int = -100) -> torch.Tensor:
    """Token-chunked CE on existing logits (keeps the fp32 upcast to one chunk at a time)."""
    lg = logits.reshape(-1, logits.shape[-1])
    y = labels.reshape(-1)
    tot = torch.zeros((), dtype=torch.float32, device=lg.device)
    for s in range(0, lg.shape[0], chunk_size):
        tot = tot + ops.cross_entropy_logits(lg[s:s + chunk_size], y[s:s + chunk_size], ignore_index, reduction="sum")
    return tot / (y != ignore_index).sum().clamp_min(1)


class FusedLinearCrossEntropyLoss(CutCrossEntropyLoss):
    """forward ``(hidden, weight, bias, labels)`` — argument order of the reference's module."""

    def forward(self, hidden, weight, bias=None, labels=None):        # type: ignore[override]
        if labels is None and bias is not None and not bias.is_floating_point():
            bias, labels = None, bias
        return super().forward(hidden, weight, labels, bias)


TritonFusedLinearCrossEntropyLoss = FusedLinearCrossEntropyLoss
LigerFusedLinearCrossEntropyLoss = FusedLinearCrossEntropyLoss


# ------------------------------------------------------------------------------------------- fused composites
def fused_rmsnorm_linear(x: torch.Tensor, norm_weight: torch.Tensor, weight: torch.Tensor,
                         bias: Optional[torch.Tensor] = None, eps: float = 1e-6) -> torch.Tensor:
    """``linear(rmsnorm(x))`` (norm kernel then the tcgen05 GEMM; differentiable)."""
    return ops.linear(ops.rmsnorm(x, norm_weight, eps), weight, bias)


class FusedRMSNormLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, eps: float = 1e-6, device=None,
                 dtype=None):
        super().__init__()
        self.norm_weight = nn.Parameter(torch.ones(in_features, device=device, dtype=dtype))
        self.linear = nn.Linear(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return fused_rmsnorm_linear(x, self.norm_weight, self.linear.weight, self.linear.bias, self.eps)


def fused_embedding_rope(input_ids: torch.Tensor, embedding: torch.Tensor, cos: Optional[torch.Tensor] = None,
                         sin: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None,
                         num_heads: int = 1) -> torch.Tensor:
    """Embedding gather; when ``cos``/``sin`` are given the rows are rotated per head, as the
    reference's kernel does (rotary embeddings normally belong on Q/K — see ``fused_qk_rope``)."""
    h = ops.embedding(input_ids, embedding)
    if cos is None:
        return h
    shp = h.shape
    d = shp[-1] // num_heads
    x = h.reshape(-1, input_ids.shape[-1], num_heads, d) if input_ids.dim() > 1 else h.reshape(1, -1, num_heads, d)
    return fused_rope(x, cos, sin, position_ids).reshape(shp)


class FusedEmbeddingRoPE(nn.Module):
    def __init__(self, vocab_size: int, hidden_size: int, num_heads: int = 1, max_seq_len: int = 4096,
                 theta: float = 10000.0, device=None, dtype=None):
        super().__init__()
        self.embedding = nn.Embedding(vocab_size, hidden_size, device=device, dtype=dtype)
        self.num_heads = num_heads
        cos, sin = precompute_rope_cache(max_seq_len, hidden_size // num_heads, theta, device)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def forward(self, input_ids: torch.Tensor, position_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        return fused_embedding_rope(input_ids, self.embedding.weight, self.cos, self.sin, position_ids, self.num_heads)


def fused_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                        softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Dense GQA attention ``q [B, Hq, S, D]``, ``k/v [B, Hk, S, D]`` → ``[B, Hq, S, D]``; runs as
    ``B`` equal-length documents of the varlen kernel."""
    B, hq, S, d = q.shape
    hk = k.shape[1]
    T = B * S
    cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=q.device)
    o = ops.attention_varlen(q.transpose(1, 2).reshape(T, hq, d), k.transpose(1, 2).reshape(T, hk, d),
                             v.transpose(1, 2).reshape(T, hk, d), cu, S, causal, softmax_scale, [S] * B)
    return o.view(B, S, hq, d).transpose(1, 2)


# ------------------------------------------------------------------------------------------- functional forward/backward pairs
# The reference exposes explicit ``*_forward`` / ``*_backward`` entry points and ``autograd.Function`` classes
# around its Triton kernels (triton_kernels.py:593-712, :1067-1178, :1370-1432, :1946-1988, :2308-2633,
# :2979-3106, :3147-3315).  Here every op already is an autograd function in ``chronicals_b200.ops``; these
# wrappers give the same call shapes on top of it.
def _vjp(fn, inputs, grad_out):
    xs = [t.detach().requires_grad_(True) for t in inputs]
    with torch.enable_grad():
        y = fn(*xs)
    return torch.autograd.grad(y, xs, grad_out, allow_unused=True)


def rmsnorm_forward(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, offset: float = 0.0
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(y, rstd)``; ``rstd`` is the per-row reciprocal RMS in fp32."""
    with torch.no_grad():
        y = ops.rmsnorm(x, weight, eps, offset)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + eps)
    return y, rstd


def rmsnorm_backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rstd: Optional[torch.Tensor] = None,
                     eps: float = 1e-6, offset: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(dx, dw)``; ``rstd`` is accepted for signature parity and recomputed by the kernel."""
    dx, dw = _vjp(lambda a, b: ops.rmsnorm(a, b, eps, offset), (x, weight), dy)
    return dx, dw


class LigerRMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps=1e-6, offset=0.0, *unused):
        y, rstd = rmsnorm_forward(x, weight, eps, offset)
        ctx.save_for_backward(x, weight, rstd)
        ctx.cfg = (eps, offset)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, rstd = ctx.saved_tensors
        dx, dw = rmsnorm_backward(dy.contiguous(), x, weight, rstd, *ctx.cfg)
        return (dx, dw) + (None,) * 8


def swiglu_forward(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return fused_swiglu(gate, up)


def swiglu_backward(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return _vjp(fused_swiglu, (gate, up), dout)


def geglu_forward(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return fused_geglu(gate, up)


def geglu_backward(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return _vjp(fused_geglu, (gate, up), dout)


class _GLUFunctionBase(torch.autograd.Function):
    _fwd = staticmethod(swiglu_forward)
    _bwd = staticmethod(swiglu_backward)

    @classmethod
    def forward(cls, ctx, gate, up):
        ctx.save_for_backward(gate, up)
        return cls._fwd(gate, up)

    @classmethod
    def backward(cls, ctx, dout):
        gate, up = ctx.saved_tensors
        return cls._bwd(dout.contiguous(), gate, up)


class LigerSwiGLUFunction(_GLUFunctionBase):
    pass


class LigerGeGLUFunction(_GLUFunctionBase):
    _fwd = staticmethod(geglu_forward)
    _bwd = staticmethod(geglu_backward)


class FusedQKRoPEFunction(torch.autograd.Function):
    """``apply(q, k, cos, sin, position_ids=None, interleaved=False) -> (q_rot, k_rot)``; the backward is the
    same rotation with the sine negated."""

    @staticmethod
    def forward(ctx, q, k, cos, sin, position_ids=None, interleaved=False):
        ctx.save_for_backward(cos, sin, position_ids if position_ids is not None else torch.empty(0))
        ctx.interleaved = interleaved
        with torch.no_grad():
            return fused_qk_rope(q, k, cos, sin, position_ids, interleaved)

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin, pos = ctx.saved_tensors
        with torch.no_grad():
            gq, gk = fused_qk_rope(dq.contiguous(), dk.contiguous(), cos, -sin, pos if pos.numel() else None, ctx.interleaved)
        return gq, gk, None, None, None, None


def fused_linear_cross_entropy_forward(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                                       bias: Optional[torch.Tensor] = None, chunk_size: int = DEFAULT_CHUNK_SIZE,
                                       ignore_index: int = -100, label_smoothing: float = 0.0, z_loss_weight: float = 0.0):
    """``(loss, z_loss, grad_hidden, grad_weight)`` computed in one call, as the reference's forward does."""
    h = hidden.detach().requires_grad_(True)
    w = weight.detach().requires_grad_(True)
    with torch.enable_grad():
        loss, z = fused_linear_cross_entropy(h, w, labels, bias, chunk_size, ignore_index, label_smoothing, z_loss_weight)
        gh, gw = torch.autograd.grad(loss, (h, w))
    return loss.detach(), z.detach(), gh, gw


triton_fused_linear_cross_entropy_forward = fused_linear_cross_entropy_forward


class FusedLinearCrossEntropyFunction(torch.autograd.Function):
    """Gradients are produced during the forward pass and only scaled in the backward pass."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, bias=None, chunk_size=DEFAULT_CHUNK_SIZE, ignore_index=-100,
                label_smoothing=0.0, z_loss_weight=0.0):
        loss, z, gh, gw = fused_linear_cross_entropy_forward(hidden, weight, labels, bias, chunk_size, ignore_index,
                                                             label_smoothing, z_loss_weight)
        ctx.save_for_backward(gh, gw)
        return loss

    @staticmethod
    def backward(ctx, gout):
        gh, gw = ctx.saved_tensors
        return (gh * gout).to(gh.dtype), (gw * gout).to(gw.dtype), None, None, None, None, None, None


TritonFusedLinearCrossEntropyFunction = FusedLinearCrossEntropyFunction


def liger_cross_entropy_forward(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                                label_smoothing: float = 0.0, z_loss_weight: float = 0.0):
    """``(loss, grad_logits)`` for materialised logits (the reference overwrites the logits with the gradient;
    here the gradient is a separate tensor)."""
    lg = logits.detach().requires_grad_(True)
    with torch.enable_grad():
        loss = ops.cross_entropy_logits(lg, labels, ignore_index, label_smoothing, z_loss_weight, "mean")
        (g,) = torch.autograd.grad(loss, (lg,))
    return loss.detach(), g


def liger_cross_entropy_backward(logits: torch.Tensor, grad_out: torch.Tensor) -> torch.Tensor:
    """Scale the gradient that the forward pass left in ``logits`` by the upstream gradient, in place
    (reference triton_kernels.py:3070-3090); a unit upstream gradient is a no-op and is detected on the device
    side-effect free, without reading it back."""
    if grad_out.numel() == 1:
        return logits.mul_(grad_out.reshape(()).to(logits.dtype))
    return logits.mul_(grad_out.to(logits.dtype).reshape(-1, *([1] * (logits.dim() - 1))))


class LigerCrossEntropyFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index=-100, label_smoothing=0.0, z_loss_weight=0.0):
        loss, g = liger_cross_entropy_forward(logits, labels, ignore_index, label_smoothing, z_loss_weight)
        ctx.save_for_backward(g)
        return loss

    @staticmethod
    def backward(ctx, gout):
        (g,) = ctx.saved_tensors
        return (g * gout).to(g.dtype), None, None, None, None


__all__ = [n for n in dir() if not n.startswith("_") and n not in ("math", "nn", "F", "torch", "ops", "ref",
                                                                    "Optional", "Tuple")]
