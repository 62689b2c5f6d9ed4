"""Varlen causal GQA attention over packed documents.

Replaces the reference's calls into flash-attn / SDPA
(chronicals/kernels/flash_attention_optimizer.py:845-994, :1388-1462).
Inputs are packed ``q [T, Hq, D]``, ``k/v [T, Hk, D]`` plus ``cu_seqlens``;
the KV head of a query head is ``hq // (Hq // Hk)`` (no ``repeat_interleave``).
Tokens at or after ``cu_seqlens[-1]`` are padding and produce zeros.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import ref
from . import _ext


def _sdpa_docs(q, k, v, bounds: Sequence[int], causal: bool, scale: float) -> torch.Tensor:
    """Library path: one SDPA call when all documents have equal length, else one per document."""
    T, hq, d = q.shape
    hk = k.shape[1]
    lens = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
    out = torch.zeros_like(q) if bounds[-1] < T else torch.empty_like(q)
    if lens and all(l == lens[0] for l in lens) and lens[0] > 0:
        n, L = len(lens), lens[0]
        tot = n * L
        qq = q[:tot].view(n, L, hq, d).transpose(1, 2)
        kk = k[:tot].view(n, L, hk, d).transpose(1, 2)
        vv = v[:tot].view(n, L, hk, d).transpose(1, 2)
        o = F.scaled_dot_product_attention(qq, kk, vv, is_causal=causal, scale=scale, enable_gqa=hq != hk)
        out[:tot] = o.transpose(1, 2).reshape(tot, hq, d)
        return out
    pieces = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        if b <= a:
            continue
        o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None],
                                           v[a:b].transpose(0, 1)[None], is_causal=causal, scale=scale,
                                           enable_gqa=hq != hk)
        pieces.append(o[0].transpose(0, 1))
    if pieces:
        cat = torch.cat(pieces, dim=0)
        out = torch.cat((cat, out[bounds[-1]:]), dim=0) if bounds[-1] < T else cat
    return out


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                     max_seqlen: Optional[int] = None, causal: bool = True, softmax_scale: Optional[float] = None,
                     seqlens_host: Optional[Sequence[int]] = None) -> torch.Tensor:
    d = q.shape[-1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    if q.is_cuda and not _ext.reference_forced() and q.dtype == torch.bfloat16 and _ext.available() and _ext.has_symbol("cb_attn_fwd") \
            and d in (64, 128) and causal:
        from .attention_cuda import attention_varlen_cuda
        return attention_varlen_cuda(q, k, v, cu_seqlens, max_seqlen, scale)
    if q.is_cuda:
        if seqlens_host is not None:
            bounds = [0]
            for l in seqlens_host:
                bounds.append(bounds[-1] + int(l))
        else:
            bounds = cu_seqlens.tolist()
        return _sdpa_docs(q, k, v, bounds, causal, scale)
    return ref.attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, scale)
