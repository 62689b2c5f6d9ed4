"""Fused LoRA linear: ``Y = X W^T + s (drop(X) A^T) B^T + b``.

Reference: chronicals/kernels/fused_lora_kernels.py:515-666 (``fused_lora_down_dropout``,
``fused_lora_linear``), :703-772 autograd function, :795-949 ``FusedLoRALinear`` /
``FusedLoRAAdapter``, :956-1013 model helpers, :1020-1081 benchmark.  PEFT convention:
``A [r, in]`` Kaiming-uniform, ``B [out, r]`` zeros.  The base GEMM, the rank-r down
projection and the up projection (whose epilogue adds the base output) run on the tcgen05
GEMM; the frozen weight gets no gradient GEMM.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..lora.lora_optimized import apply_lora_to_model as _apply_lora_to_model
from ..lora.lora_optimized import count_lora_params, get_lora_params


def fused_lora_down_dropout(x: torch.Tensor, lora_A: torch.Tensor, dropout: float = 0.0, training: bool = True
                            ) -> torch.Tensor:
    """``H = dropout(X) A^T`` (``[..., r]``)."""
    xd = F.dropout(x, dropout, training) if dropout > 0 else x
    return ops.linear(xd, lora_A)


def fused_lora_linear(x: torch.Tensor, W: torch.Tensor, A: torch.Tensor, B: torch.Tensor,
                      bias: Optional[torch.Tensor] = None, lora_alpha: float = 16.0, lora_dropout: float = 0.0,
                      training: bool = True) -> torch.Tensor:
    scaling = lora_alpha / A.shape[0]
    base = ops.linear(x, W, bias)
    h = fused_lora_down_dropout(x, A, lora_dropout, training)
    return ops.linear(h, B * scaling, None, base)


class FusedLoRALinearFunction(torch.autograd.Function):
    """``apply(x, W, A, B, bias, scaling)``: frozen ``W`` (no weight gradient, as in the reference's
    fused_lora_kernels.py:703-772), gradients for ``x``, ``A``, ``B`` and ``bias``."""

    @staticmethod
    def forward(ctx, x, W, A, B, bias=None, scaling=1.0):
        x2 = x.reshape(-1, x.shape[-1])
        with torch.no_grad():
            h = ops.linear(x2, A)
            y = ops.linear(h, B * scaling, None, ops.linear(x2, W, bias))
        ctx.save_for_backward(x2, W, A, B, h)
        ctx.scaling, ctx.has_bias, ctx.shape = scaling, bias is not None, x.shape
        return y.view(*x.shape[:-1], W.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, W, A, B, h = ctx.saved_tensors
        s = ctx.scaling
        dy2 = dy.reshape(-1, dy.shape[-1])
        with torch.no_grad():
            dh = ops.linear(dy2, (B * s).t().contiguous())                 # [T, r]
            dx = ops.linear(dy2, W.t().contiguous()) + ops.linear(dh, A.t().contiguous())
            dA = (dh.float().t() @ x2.float()).to(A.dtype)
            dB = (s * (dy2.float().t() @ h.float())).to(B.dtype)
            db = dy2.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx.view(ctx.shape), None, dA, dB, db, None


def fused_lora_linear_with_grad(x: torch.Tensor, W: torch.Tensor, A: torch.Tensor, B: torch.Tensor,
                                bias: Optional[torch.Tensor] = None, lora_alpha: float = 1.0, lora_dropout: float = 0.0,
                                training: bool = True) -> torch.Tensor:
    """``x Wᵀ + lora_alpha · (dropout(x) Aᵀ) Bᵀ + bias`` with gradients for ``x``, ``A``, ``B`` and ``bias`` and a
    frozen ``W`` (reference fused_lora_kernels.py:775-789, where ``lora_alpha`` is the final scaling factor).
    Dropout, when active, is applied to the adapter branch's input outside the fused function."""
    if training and lora_dropout > 0.0:
        base = ops.linear(x, W, bias)
        h = ops.linear(torch.nn.functional.dropout(x, lora_dropout, True), A)
        return base + lora_alpha * ops.linear(h, B)
    return FusedLoRALinearFunction.apply(x, W, A, B, bias, lora_alpha)


def lora_linear_pytorch(x, W, A, B, bias=None, lora_alpha: float = 16.0, lora_dropout: float = 0.0,
                        training: bool = True) -> torch.Tensor:
    xd = F.dropout(x, lora_dropout, training) if lora_dropout > 0 else x
    return F.linear(x, W, bias) + (lora_alpha / A.shape[0]) * F.linear(F.linear(xd, A), B)


class FusedLoRALinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, rank: int = 16, lora_alpha: float = 32.0,
                 lora_dropout: float = 0.0, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features, self.rank = in_features, out_features, rank
        self.lora_alpha, self.lora_dropout, self.scaling = lora_alpha, lora_dropout, lora_alpha / rank
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype),
                                   requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype), requires_grad=False) if bias else None
        self.lora_A = nn.Parameter(torch.empty(rank, in_features, device=device, dtype=dtype))
        self.lora_B = nn.Parameter(torch.zeros(out_features, rank, device=device, dtype=dtype))
        self.merged = False
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))

    @classmethod
    def from_linear(cls, linear: nn.Linear, rank: int = 16, lora_alpha: float = 32.0, lora_dropout: float = 0.0):
        m = cls(linear.in_features, linear.out_features, rank, lora_alpha, lora_dropout, linear.bias is not None,
                linear.weight.device, linear.weight.dtype)
        with torch.no_grad():
            m.weight.copy_(linear.weight)
            if linear.bias is not None:
                m.bias.copy_(linear.bias)
        return m

    @torch.no_grad()
    def merge(self) -> None:
        if not self.merged:
            self.weight.add_((self.scaling * (self.lora_B.float() @ self.lora_A.float())).to(self.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self) -> None:
        if self.merged:
            self.weight.sub_((self.scaling * (self.lora_B.float() @ self.lora_A.float())).to(self.weight.dtype))
            self.merged = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.merged:
            return ops.linear(x, self.weight, self.bias)
        return fused_lora_linear(x, self.weight, self.lora_A, self.lora_B, self.bias, self.lora_alpha,
                                 self.lora_dropout, self.training)


class FusedLoRAAdapter(nn.Module):
    """The adapter alone: ``s (drop(x) A^T) B^T`` to be added to some other module's output."""

    def __init__(self, in_features: int, out_features: int, rank: int = 16, lora_alpha: float = 32.0,
                 lora_dropout: float = 0.0, device=None, dtype=None):
        super().__init__()
        self.lora_A = nn.Parameter(torch.empty(rank, in_features, device=device, dtype=dtype))
        self.lora_B = nn.Parameter(torch.zeros(out_features, rank, device=device, dtype=dtype))
        self.scaling, self.lora_dropout = lora_alpha / rank, lora_dropout
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = fused_lora_down_dropout(x, self.lora_A, self.lora_dropout, self.training)
        return ops.linear(h, self.lora_B * self.scaling)


def apply_lora_to_model(model: nn.Module, target_modules: Optional[List[str]] = None, rank: int = 16,
                        alpha: float = 32.0, dropout: float = 0.0) -> nn.Module:
    return _apply_lora_to_model(model, rank, alpha, target_modules, "kaiming", dropout)


def benchmark_lora(tokens: int = 8192, in_features: int = 896, out_features: int = 4864, rank: int = 16,
                   iters: int = 20) -> Dict[str, float]:
    if not torch.cuda.is_available():
        return {}
    dev, dt = "cuda", torch.bfloat16
    x = torch.randn(tokens, in_features, device=dev, dtype=dt)
    m = FusedLoRALinear(in_features, out_features, rank, device=dev, dtype=dt)
    res = {}
    for name, fn in (("fused_ms", lambda: m(x)),
                     ("pytorch_ms", lambda: lora_linear_pytorch(x, m.weight, m.lora_A, m.lora_B))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        res[name] = a.elapsed_time(b) / iters
    return res


__all__ = ["fused_lora_down_dropout", "fused_lora_linear", "fused_lora_linear_with_grad", "lora_linear_pytorch", "FusedLoRALinearFunction", "FusedLoRALinear",
           "FusedLoRAAdapter", "apply_lora_to_model", "get_lora_params", "count_lora_params", "benchmark_lora"]
