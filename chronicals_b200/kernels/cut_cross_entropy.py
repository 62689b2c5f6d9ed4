"""Cut cross-entropy: loss of ``hidden @ weight.T`` without materialising the logits.

Public names follow the reference module (chronicals/kernels/
cut_cross_entropy.py:59-90 ``get_optimal_chunk_size``, :1023-1078
``cut_cross_entropy``, :1081-1162 ``CutCrossEntropyLoss``, :1169-1276 chunked
variants, :1283-1372 ``AdaptiveCrossEntropyLoss``, :1379-1430 helpers).

On CUDA (bf16) the work is done by the fused tcgen05 kernels: the forward keeps
a running (max, sum-exp) per token in the GEMM epilogue while vocab tiles stream
through TMEM; the backward recomputes a vocab chunk's logits, turns them into
``softmax - target`` in registers, and feeds two gradient GEMMs.  Elsewhere a
vocab-chunked PyTorch implementation with the same structure runs.

Semantics: mean over labels ``!= ignore_index``; label smoothing as in
``torch.nn.functional.cross_entropy``; optional z-loss ``w * lse^2`` per token.
Labels must already be shifted.  Unlike the reference there is no host
synchronisation anywhere (its paths call ``.item()`` per chunk).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import ref

DEFAULT_CHUNK_SIZE = 8192
MIN_CHUNK_SIZE = 256


def get_optimal_chunk_size(vocab_size: int, hidden_size: int, available_vram_gb: float = 40.0) -> int:
    """Chunk-size policy of the reference: 80 % of memory over ``8 * hidden`` bytes, capped by
    vocabulary class, rounded down to a power of two, at least 256.  For the fused kernels the
    value is only a hint (the logits never reach memory)."""
    max_chunk = int(0.8 * available_vram_gb * 2**30 / (8 * max(1, hidden_size)))
    cap = 4096 if vocab_size < 64_000 else (8192 if vocab_size < 128_000 else 16384)
    c = max(MIN_CHUNK_SIZE, min(max_chunk, cap))
    return 1 << int(math.log2(c))


def cut_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                      bias: Optional[torch.Tensor] = None, chunk_size: int = DEFAULT_CHUNK_SIZE,
                      ignore_index: int = -100, label_smoothing: float = 0.0, z_loss_weight: float = 0.0,
                      use_triton: bool = True, reduction: str = "mean") -> torch.Tensor:
    """``use_triton`` is accepted for signature compatibility: it selects the fused kernel path when
    the inputs live on a GPU (there is no Triton in this framework)."""
    if not use_triton and hidden.is_cuda:
        return ref.linear_cross_entropy_chunked(hidden.reshape(-1, hidden.shape[-1]), weight, labels.reshape(-1), bias,
                                                ignore_index, label_smoothing, z_loss_weight, reduction, chunk_size)
    return ops.linear_cross_entropy(hidden, weight, labels, bias, ignore_index, label_smoothing, z_loss_weight,
                                    reduction, chunk_size)


class CutCrossEntropyLoss(nn.Module):
    def __init__(self, chunk_size: Optional[int] = None, ignore_index: int = -100, label_smoothing: float = 0.0,
                 z_loss_weight: float = 0.0, reduction: str = "mean"):
        super().__init__()
        self.chunk_size = chunk_size
        self.ignore_index = ignore_index
        self.label_smoothing = label_smoothing
        self.z_loss_weight = z_loss_weight
        self.reduction = reduction

    def forward(self, hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        chunk = self.chunk_size or get_optimal_chunk_size(weight.shape[0], weight.shape[1])
        return cut_cross_entropy(hidden, weight, labels, bias, chunk, self.ignore_index, self.label_smoothing,
                                 self.z_loss_weight, reduction=self.reduction)


def chunked_cross_entropy_loss(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                               bias: Optional[torch.Tensor] = None, chunk_size: int = DEFAULT_CHUNK_SIZE,
                               ignore_index: int = -100, label_smoothing: float = 0.0,
                               z_loss_weight: float = 0.0) -> torch.Tensor:
    """The vocab-chunked PyTorch implementation on any device."""
    return ref.linear_cross_entropy_chunked(hidden.reshape(-1, hidden.shape[-1]), weight, labels.reshape(-1), bias,
                                            ignore_index, label_smoothing, z_loss_weight, "mean", chunk_size)


class ChunkedCrossEntropyLoss(CutCrossEntropyLoss):
    def forward(self, hidden, weight, labels, bias=None):
        return chunked_cross_entropy_loss(hidden, weight, labels, bias, self.chunk_size or DEFAULT_CHUNK_SIZE,
                                          self.ignore_index, self.label_smoothing, self.z_loss_weight)


class AdaptiveCrossEntropyLoss(nn.Module):
    """Chooses by vocabulary size (thresholds of the reference trainer): materialised logits for
    small vocabularies, chunked for mid-size, cut cross-entropy for large."""

    def __init__(self, small_vocab_threshold: int = 32000, large_vocab_threshold: int = 100000,
                 ignore_index: int = -100, label_smoothing: float = 0.0, z_loss_weight: float = 0.0):
        super().__init__()
        self.small, self.large = small_vocab_threshold, large_vocab_threshold
        self.kw = dict(ignore_index=ignore_index, label_smoothing=label_smoothing, z_loss_weight=z_loss_weight)

    def select(self, vocab_size: int) -> str:
        if vocab_size <= self.small:
            return "standard"
        return "cce" if vocab_size >= self.large else "chunked"

    def forward(self, hidden, weight, labels, bias=None):
        mode = self.select(weight.shape[0])
        if mode == "standard":
            logits = torch.nn.functional.linear(hidden.reshape(-1, hidden.shape[-1]), weight, bias)
            return ops.cross_entropy_logits(logits, labels.reshape(-1), **self.kw)
        if mode == "chunked":
            return chunked_cross_entropy_loss(hidden, weight, labels, bias, **self.kw)
        return cut_cross_entropy(hidden, weight, labels, bias, **self.kw)


def compute_z_loss(logits: torch.Tensor, z_loss_weight: float = 1e-4) -> torch.Tensor:
    return z_loss_weight * torch.logsumexp(logits.float(), dim=-1).pow(2).mean()


def estimate_memory_savings(batch_tokens: int, vocab_size: int, hidden_size: int, chunk_size: int = DEFAULT_CHUNK_SIZE,
                            bytes_per_el: int = 4) -> Dict[str, float]:
    """Bytes of logits a materialising implementation holds vs. what the chunked / fused paths hold."""
    full = batch_tokens * vocab_size * bytes_per_el
    chunked = batch_tokens * min(chunk_size, vocab_size) * 2          # one bf16 d(logits) chunk in the backward
    fused_fwd = batch_tokens * 4 * 8                                   # per-token partial statistics
    return {"standard_gb": full / 2**30, "chunked_gb": chunked / 2**30, "fused_forward_gb": fused_fwd / 2**30,
            "reduction_factor": full / max(1, chunked)}


class CutCrossEntropyForward:
    """Forward half as a separate object (reference: cut_cross_entropy.py:559-692): returns
    ``(loss, lse, target_logit, valid_mask)`` without materialising logits."""

    @staticmethod
    def forward(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, bias: Optional[torch.Tensor] = None,
                chunk_size: int = DEFAULT_CHUNK_SIZE, ignore_index: int = -100, label_smoothing: float = 0.0,
                z_loss_weight: float = 0.0):
        h = hidden.reshape(-1, hidden.shape[-1])
        y = labels.reshape(-1)
        valid = y != ignore_index
        with torch.no_grad():
            rows = cut_cross_entropy(h, weight, y, bias, chunk_size, ignore_index, 0.0, 0.0, reduction="none")
            loss = cut_cross_entropy(h, weight, y, bias, chunk_size, ignore_index, label_smoothing, z_loss_weight)
            safe = y.clamp_min(0)
            tgt = (h.float() * weight[safe].float()).sum(-1)
            if bias is not None:
                tgt = tgt + bias[safe].float()
            tgt = tgt * valid
            lse = rows.float() + tgt                       # per-row loss = lse - target logit
        return loss, lse, tgt, valid


class CutCrossEntropyBackward:
    """Backward half (reference: cut_cross_entropy.py:695-808): ``(grad_hidden, grad_weight, grad_bias)``."""

    @staticmethod
    def backward(grad_output: torch.Tensor, hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, chunk_size: int = DEFAULT_CHUNK_SIZE, ignore_index: int = -100,
                 label_smoothing: float = 0.0, z_loss_weight: float = 0.0):
        h = hidden.detach().requires_grad_(True)
        w = weight.detach().requires_grad_(True)
        b = bias.detach().requires_grad_(True) if bias is not None else None
        with torch.enable_grad():
            loss = cut_cross_entropy(h, w, labels, b, chunk_size, ignore_index, label_smoothing, z_loss_weight)
            grads = torch.autograd.grad(loss, (h, w) + ((b,) if b is not None else ()), grad_output)
        return grads[0], grads[1], (grads[2] if b is not None else None)


class CutCrossEntropyFunction(torch.autograd.Function):
    """``apply(hidden, weight, labels, bias, chunk_size, ignore_index, label_smoothing, z_loss_weight)``"""

    @staticmethod
    def forward(ctx, hidden, weight, labels, bias=None, chunk_size=DEFAULT_CHUNK_SIZE, ignore_index=-100,
                label_smoothing=0.0, z_loss_weight=0.0):
        ctx.save_for_backward(hidden, weight, labels, bias if bias is not None else torch.empty(0))
        ctx.cfg = (chunk_size, ignore_index, label_smoothing, z_loss_weight)
        with torch.no_grad():
            return cut_cross_entropy(hidden, weight, labels, bias, chunk_size, ignore_index, label_smoothing, z_loss_weight)

    @staticmethod
    def backward(ctx, gout):
        hidden, weight, labels, bias = ctx.saved_tensors
        gh, gw, gb = CutCrossEntropyBackward.backward(gout, hidden, weight, labels, bias if bias.numel() else None, *ctx.cfg)
        return gh, gw, None, gb, None, None, None, None


TritonCCEFunction = CutCrossEntropyFunction
