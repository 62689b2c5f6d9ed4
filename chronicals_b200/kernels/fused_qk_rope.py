"""Fused Q/K rotary embedding with scaling variants.

Reference: chronicals/kernels/fused_qk_rope.py:474-706 forward/backward and
``fused_qk_rope``, :709-769 packed-QKV in-place form, :776-928 cache builders
(plain, NTK, YaRN), :970-1058 ``FusedQKRoPE`` module, :1065-1103 ``apply_rope``.
The reference's Triton default pairs ``(2i, 2i+1)`` while its own fallback and
HuggingFace use the split-half pairing; here split-half is the default
everywhere and ``interleaved=True`` selects the other.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import ref
from .fused_kernels import fused_qk_rope, fused_rope, precompute_rope_cache


def precompute_rope_cache_ntk(seq_len: int, head_dim: int, theta: float = 10000.0, scaling_factor: float = 2.0,
                              device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    return ref.rope_cache(seq_len, head_dim, theta, {"type": "ntk", "factor": scaling_factor}, device)


def precompute_rope_cache_yarn(seq_len: int, head_dim: int, theta: float = 10000.0, scaling_factor: float = 4.0,
                               original_max_position: int = 4096, beta_fast: float = 32.0, beta_slow: float = 1.0,
                               device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    return ref.rope_cache(seq_len, head_dim, theta, {"type": "yarn", "factor": scaling_factor,
                                                     "original_max_position_embeddings": original_max_position,
                                                     "beta_fast": beta_fast, "beta_slow": beta_slow}, device)


def fused_qkv_rope_inplace(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                           position_ids: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """Packed ``[B, S, 3, H, D]`` (or ``[T, 3, H, D]``): Q and K rotated, V untouched."""
    shape = qkv.shape
    H, D = shape[-2], shape[-1]
    flat = qkv.reshape(-1, 3 * H * D)
    T = flat.shape[0]
    if position_ids is None:
        S = shape[-4] if qkv.dim() == 5 else T
        position_ids = torch.arange(S, device=qkv.device).repeat(T // S)
    out = ops.qk_rope_(flat, cos, sin, position_ids.reshape(T), H, H, D, interleaved)
    return out.reshape(shape)


class FusedQKRoPE(nn.Module):
    """Owns the cos/sin tables (``scaling_type`` none / ntk / yarn / llama3 / linear) and rotates Q, K."""

    def __init__(self, head_dim: int, max_seq_len: int = 4096, theta: float = 10000.0, scaling_type: str = "none",
                 scaling_factor: float = 1.0, original_max_position: int = 4096, interleaved: bool = False, device=None):
        super().__init__()
        self.head_dim, self.interleaved = head_dim, interleaved
        scaling = None if scaling_type in ("none", None) else {
            "type": scaling_type, "factor": scaling_factor, "original_max_position_embeddings": original_max_position}
        cos, sin = ref.rope_cache(max_seq_len, head_dim, theta, scaling, device)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def forward(self, q: torch.Tensor, k: torch.Tensor, position_ids: Optional[torch.Tensor] = None):
        return fused_qk_rope(q, k, self.cos, self.sin, position_ids, self.interleaved)


def apply_rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
               position_ids: Optional[torch.Tensor] = None, interleaved: bool = False):
    return fused_qk_rope(q, k, cos, sin, position_ids, interleaved)


def fused_qk_rope_forward(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                          position_ids: Optional[torch.Tensor] = None, interleaved: bool = False, inplace: bool = False):
    """Functional forward (reference: fused_qk_rope.py:474-568); ``inplace`` is accepted for parity — the
    packed-QKV in-place rotation is :func:`fused_qkv_rope_inplace`."""
    with torch.no_grad():
        return fused_qk_rope(q, k, cos, sin, position_ids, interleaved)


def fused_qk_rope_backward(dq: torch.Tensor, dk: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                           position_ids: Optional[torch.Tensor] = None, interleaved: bool = False):
    """Gradient of the rotation = rotation by the negated angle."""
    with torch.no_grad():
        return fused_qk_rope(dq, dk, cos, -sin, position_ids, interleaved)


from .fused_kernels import FusedQKRoPEFunction  # noqa: E402  (same autograd function under this module's name)

__all__ = ["fused_qk_rope", "fused_qkv_rope_inplace", "precompute_rope_cache", "precompute_rope_cache_ntk",
           "precompute_rope_cache_yarn", "FusedQKRoPE", "apply_rope", "fused_rope", "fused_qk_rope_forward",
           "fused_qk_rope_backward", "FusedQKRoPEFunction"]
