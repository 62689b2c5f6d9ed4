"""Rotary embedding entry points incl. the packed variable-length form.

Reference: chronicals/kernels/fused_rope.py:474-757 wrappers (Q+K, Q only,
``cu_seqlens`` varlen), :810-835 ``fused_qk_rope``, :924-1013 cache builders
(plain and Llama-3 extended), :1020-1087 ``FusedRotaryEmbedding``, :1094-1154
benchmark.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import ref
from .fused_kernels import fused_qk_rope, fused_rope, precompute_rope_cache


def precompute_rope_cache_llama3(seq_len: int, head_dim: int, theta: float = 500000.0, factor: float = 8.0,
                                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                                 original_max_position: int = 8192, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    return ref.rope_cache(seq_len, head_dim, theta, {
        "type": "llama3", "factor": factor, "low_freq_factor": low_freq_factor, "high_freq_factor": high_freq_factor,
        "original_max_position_embeddings": original_max_position}, device)


def fused_q_rope_inplace(q: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                         position_ids: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """Q-only rotation."""
    return fused_rope(q, cos, sin, position_ids, interleaved)


def fused_qk_rope_inplace(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                          position_ids: Optional[torch.Tensor] = None, interleaved: bool = True,
                          long_context: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotate ``q`` and ``k`` (``[batch, seq, heads, head_dim]``) and write the result back into the same
    tensors (reference fused_rope.py:474-571, whose default pairing is interleaved).  ``long_context`` selected
    64-bit indexing there; the kernel here always indexes with 64-bit offsets."""
    with torch.no_grad():
        rq, rk = fused_qk_rope(q, k, cos, sin, position_ids, interleaved)
        if rq.data_ptr() != q.data_ptr():
            q.copy_(rq)
        if rk.data_ptr() != k.data_ptr():
            k.copy_(rk)
    return q, k


def fused_qk_rope_inplace_backward(dq: torch.Tensor, dk: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                                   position_ids: Optional[torch.Tensor] = None, interleaved: bool = True,
                                   long_context: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gradient of the in-place rotation: the rotation by the negated angle, again in place (reference :574-650)."""
    return fused_qk_rope_inplace(dq, dk, cos, -sin, position_ids, interleaved, long_context)


def precompute_rope_cache_extended(max_seq_len: int, head_dim: int, base: float = 10000.0, scaling_factor: float = 1.0,
                                   low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                                   original_max_seq: int = 8192, device="cpu",
                                   dtype: torch.dtype = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[max_seq_len, head_dim / 2]`` cos / sin tables with Llama-3 style frequency interpolation: wavelengths
    longer than ``original_max_seq / low_freq_factor`` are stretched by ``scaling_factor``, those shorter than
    ``original_max_seq / high_freq_factor`` are kept, the band between is blended linearly in wavelength
    (reference :957-1013, which blends in wavelength rather than in rotations per context as HuggingFace does)."""
    import math
    half = head_dim // 2
    inv = 1.0 / (base ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))
    lo_len, hi_len = original_max_seq / low_freq_factor, original_max_seq / high_freq_factor
    wavelen = 2 * math.pi / inv
    if lo_len == hi_len:
        smooth = (wavelen > lo_len).float()
    else:
        smooth = ((wavelen - hi_len) / (lo_len - hi_len)).clamp(0.0, 1.0)
    inv = inv * (1 - smooth) + inv / scaling_factor * smooth
    ang = torch.outer(torch.arange(max_seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def positions_from_cu_seqlens(cu_seqlens: torch.Tensor, total_tokens: int) -> torch.Tensor:
    """Per-token position inside its document (binary search in ``cu_seqlens``; padding → 0)."""
    from ..models.decoder import _positions_from_cu
    return _positions_from_cu(cu_seqlens, total_tokens)


def fused_qk_rope_variable_length(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                                  cu_seqlens: torch.Tensor, interleaved: bool = False):
    """Packed ``q [T, Hq, D]``, ``k [T, Hk, D]``; positions restart at every document start."""
    pos = positions_from_cu_seqlens(cu_seqlens, q.shape[0])
    return fused_qk_rope(q, k, cos, sin, pos, interleaved)


class FusedRotaryEmbedding(nn.Module):
    def __init__(self, head_dim: int, max_position_embeddings: int = 4096, base: float = 10000.0,
                 scaling: Optional[dict] = None, interleaved: bool = False, device=None):
        super().__init__()
        cos, sin = ref.rope_cache(max_position_embeddings, head_dim, base, scaling, device)
        self.register_buffer("cos_cached", cos, persistent=False)
        self.register_buffer("sin_cached", sin, persistent=False)
        self.interleaved = interleaved

    def forward(self, q: torch.Tensor, k: torch.Tensor, position_ids: Optional[torch.Tensor] = None,
                cu_seqlens: Optional[torch.Tensor] = None):
        if cu_seqlens is not None:
            return fused_qk_rope_variable_length(q, k, self.cos_cached, self.sin_cached, cu_seqlens, self.interleaved)
        return fused_qk_rope(q, k, self.cos_cached, self.sin_cached, position_ids, self.interleaved)


def benchmark_rope(batch: int = 8, seq: int = 1024, hq: int = 14, hk: int = 2, d: int = 64, iters: int = 20
                   ) -> Dict[str, float]:
    """CUDA-event timing of the fused kernel against the PyTorch formula (GPU only)."""
    if not torch.cuda.is_available():
        return {}
    dev = "cuda"
    q = torch.randn(batch, seq, hq, d, device=dev, dtype=torch.bfloat16)
    k = torch.randn(batch, seq, hk, d, device=dev, dtype=torch.bfloat16)
    cos, sin = precompute_rope_cache(seq, d, 1e6, dev)
    res = {}
    for name, fn in (("fused_ms", lambda: fused_qk_rope(q, k, cos, sin)),
                     ("pytorch_ms", lambda: (ref.apply_rope(q, cos, sin), ref.apply_rope(k, cos, sin)))):
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


from .fused_kernels import FusedQKRoPEFunction  # noqa: E402

__all__ = ["fused_qk_rope", "fused_q_rope_inplace", "fused_qk_rope_inplace", "fused_qk_rope_inplace_backward",
           "precompute_rope_cache_extended", "fused_qk_rope_variable_length", "precompute_rope_cache",
           "precompute_rope_cache_llama3", "FusedRotaryEmbedding", "positions_from_cu_seqlens", "benchmark_rope",
           "FusedQKRoPEFunction"]
