"""Pure-PyTorch implementations of every fused op.

These run on any device, are differentiable through ordinary autograd, and
serve two purposes: they are the CPU execution path, and they are the oracle
the CUDA kernels are tested against.  The formulas follow the reference's own
(chronicals/kernels/triton_kernels.py:303-374 RMSNorm, :830-986 SwiGLU,
:1296-1367 GeGLU, :2070-2160 RoPE fallback; chronicals/kernels/
cut_cross_entropy.py:427-552 loss; chronicals/optimizers/fused_adamw.py:45-101
AdamW), with the reference's known defects not reproduced: label smoothing
follows ``torch.nn.functional.cross_entropy`` and RoPE defaults to the
split-half (HF) convention.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- norms / activations
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, offset: float = 0.0) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * (weight.float() + offset)).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``h = x + residual`` then RMSNorm(h); returns ``(normed, h)``."""
    h = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(h, weight, eps), h


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def swiglu_packed(gate_up: torch.Tensor) -> torch.Tensor:
    """Input ``[..., 2I]`` holding ``gate | up`` halves."""
    g, u = gate_up.chunk(2, dim=-1)
    return swiglu(g, u)


def geglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (F.gelu(gate.float(), approximate="tanh") * up.float()).to(gate.dtype)


def geglu_packed(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.chunk(2, dim=-1)
    return geglu(g, u)


# --------------------------------------------------------------------------- RoPE
def rope_inv_freq(head_dim: int, theta: float = 1e4, scaling: Optional[dict] = None,
                  device=None) -> Tuple[torch.Tensor, float]:
    """Inverse frequencies and the attention scaling factor.

    ``scaling``: ``None`` | ``{"type": "ntk", "factor": f}`` |
    ``{"type": "yarn", "factor": f, "original_max_position_embeddings": n, ...}`` |
    ``{"type": "llama3", "factor": f, "low_freq_factor", "high_freq_factor",
    "original_max_position_embeddings"}`` | ``{"type": "linear", "factor": f}``
    (reference: fused_qk_rope.py:814-928, fused_rope.py:957-1013).
    """
    idx = torch.arange(0, head_dim, 2, dtype=torch.float64, device=device)
    attn_scale = 1.0
    st = (scaling or {}).get("type", (scaling or {}).get("rope_type")) if scaling else None
    if st in (None, "default", "none"):
        inv = 1.0 / (theta ** (idx / head_dim))
    elif st == "linear":
        inv = 1.0 / (theta ** (idx / head_dim)) / float(scaling["factor"])
    elif st == "ntk":
        f = float(scaling["factor"])
        theta2 = theta * f ** (head_dim / max(head_dim - 2, 1))
        inv = 1.0 / (theta2 ** (idx / head_dim))
    elif st == "yarn":
        f = float(scaling["factor"])
        orig = int(scaling.get("original_max_position_embeddings", 4096))
        beta_fast = float(scaling.get("beta_fast", 32.0))
        beta_slow = float(scaling.get("beta_slow", 1.0))
        base_inv = 1.0 / (theta ** (idx / head_dim))

        def corr_dim(n_rot: float) -> float:
            return head_dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

        lo = max(math.floor(corr_dim(beta_fast)), 0)
        hi = min(math.ceil(corr_dim(beta_slow)), head_dim // 2 - 1)
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float64, device=device) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        extrap_mask = 1.0 - ramp           # 1 → keep original (high-frequency) dims
        inv = base_inv / f * (1 - extrap_mask) + base_inv * extrap_mask
        attn_scale = float(scaling.get("attention_factor", 0.1 * math.log(f) + 1.0)) if f > 1 else 1.0
    elif st == "llama3":
        f = float(scaling["factor"])
        lo_f = float(scaling.get("low_freq_factor", 1.0))
        hi_f = float(scaling.get("high_freq_factor", 4.0))
        orig = int(scaling.get("original_max_position_embeddings", 8192))
        base_inv = 1.0 / (theta ** (idx / head_dim))
        wavelen = 2 * math.pi / base_inv
        smooth = ((orig / wavelen) - lo_f) / (hi_f - lo_f)
        mid = (1 - smooth) * base_inv / f + smooth * base_inv
        inv = torch.where(wavelen > orig / lo_f, base_inv / f,
                          torch.where(wavelen < orig / hi_f, base_inv, mid))
    else:
        raise ValueError(f"unknown rope scaling type {st!r}")
    return inv.float(), attn_scale


def rope_cache(max_pos: int, head_dim: int, theta: float = 1e4, scaling: Optional[dict] = None,
               device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``cos, sin`` of shape ``[max_pos, head_dim // 2]`` in fp32."""
    inv, attn_scale = rope_inv_freq(head_dim, theta, scaling, device)
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return ang.cos() * attn_scale, ang.sin() * attn_scale


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, position_ids: Optional[torch.Tensor] = None,
               interleaved: bool = False, inverse: bool = False) -> torch.Tensor:
    """Rotate ``x [..., T, H, D]`` (token dim third from the end).

    ``cos/sin`` are ``[P, D/2]`` tables; ``position_ids`` ``[..., T]`` selects
    rows (defaults to ``arange(T)``).  ``inverse`` negates sin (the backward).
    """
    T, D = x.shape[-3], x.shape[-1]
    if position_ids is None:
        c, s = cos[:T], sin[:T]
    else:
        c, s = cos[position_ids], sin[position_ids]
    c = c.unsqueeze(-2).float()
    s = s.unsqueeze(-2).float()
    if inverse:
        s = -s
    xf = x.float()
    if interleaved:
        x1, x2 = xf[..., 0::2], xf[..., 1::2]
        o1 = x1 * c - x2 * s
        o2 = x2 * c + x1 * s
        out = torch.stack((o1, o2), dim=-1).flatten(-2)
    else:
        x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)
    return out.to(x.dtype)


# --------------------------------------------------------------------------- attention
def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                     max_seqlen: Optional[int] = None, causal: bool = True,
                     softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Packed attention: ``q [T, Hq, D]``, ``k/v [T, Hk, D]``; documents are the
    intervals of ``cu_seqlens``; tokens past ``cu_seqlens[-1]`` are padding and
    produce zeros.  Math in fp32."""
    T, hq, d = q.shape
    hk = k.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    bounds = cu_seqlens.tolist()
    rep = hq // hk
    for a, b in zip(bounds[:-1], bounds[1:]):
        if b <= a:
            continue
        qi = q[a:b].float().transpose(0, 1)                       # [Hq, L, D]
        ki = k[a:b].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vi = v[a:b].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.matmul(qi, ki.transpose(-1, -2)) * scale
        if causal:
            L = b - a
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[a:b] = torch.matmul(p, vi).transpose(0, 1).to(q.dtype)
    return out


# --------------------------------------------------------------------------- cross-entropy
def linear_cross_entropy_dense(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                               bias: Optional[torch.Tensor] = None, ignore_index: int = -100,
                               label_smoothing: float = 0.0, z_loss_weight: float = 0.0,
                               reduction: str = "mean") -> torch.Tensor:
    """The oracle: materialise logits in fp32 and use ``F.cross_entropy``."""
    h = hidden.reshape(-1, hidden.shape[-1]).float()
    y = labels.reshape(-1)
    logits = h @ weight.float().t()
    if bias is not None:
        logits = logits + bias.float()
    loss = F.cross_entropy(logits, y, ignore_index=ignore_index, label_smoothing=label_smoothing, reduction="none")
    if z_loss_weight:
        lse = torch.logsumexp(logits, dim=-1)
        loss = loss + z_loss_weight * lse.pow(2) * (y != ignore_index)
    if reduction == "none":
        return loss
    if reduction == "sum":
        return loss.sum()
    n = (y != ignore_index).sum().clamp_min(1)
    return loss.sum() / n


class _ChunkedLinearCE(torch.autograd.Function):
    """Vocab-chunked linear + cross-entropy that never holds ``[T, V]``.

    Forward keeps a running (max, sum-exp) per token over vocab chunks;
    backward recomputes each chunk's logits and feeds ``softmax − target``
    straight into the two gradient products.  Same structure as the CUDA path,
    in plain PyTorch.
    """

    @staticmethod
    def forward(ctx, hidden, weight, bias, labels, ignore_index, label_smoothing, z_loss_weight, chunk):
        h = hidden.float()
        T = h.shape[0]
        V = weight.shape[0]
        dev = h.device
        m = torch.full((T,), float("-inf"), device=dev)
        s = torch.zeros(T, device=dev)
        tgt = torch.zeros(T, device=dev)
        sum_logits = torch.zeros(T, device=dev)
        valid = labels != ignore_index
        safe = labels.clamp_min(0)
        for c0 in range(0, V, chunk):
            c1 = min(V, c0 + chunk)
            lg = h @ weight[c0:c1].float().t()
            if bias is not None:
                lg = lg + bias[c0:c1].float()
            cm = lg.max(dim=-1).values
            nm = torch.maximum(m, cm)
            s = s * torch.exp(m - nm) + torch.exp(lg - nm[:, None]).sum(-1)
            m = nm
            inside = valid & (safe >= c0) & (safe < c1)
            if inside.any():
                rows = inside.nonzero(as_tuple=True)[0]
                tgt[rows] = lg[rows, safe[rows] - c0]
            if label_smoothing:
                sum_logits += lg.sum(-1)
        lse = m + torch.log(s)
        loss = lse - tgt
        if label_smoothing:
            loss = (1 - label_smoothing) * loss + label_smoothing * (lse - sum_logits / V)
        if z_loss_weight:
            loss = loss + z_loss_weight * lse * lse
        loss = torch.where(valid, loss, torch.zeros_like(loss))
        ctx.save_for_backward(hidden, weight, bias if bias is not None else torch.empty(0), labels, lse)
        ctx.cfg = (ignore_index, label_smoothing, z_loss_weight, chunk, bias is not None)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        hidden, weight, bias, labels, lse = ctx.saved_tensors
        ignore_index, eps, zw, chunk, has_bias = ctx.cfg
        h = hidden.float()
        V = weight.shape[0]
        valid = labels != ignore_index
        safe = labels.clamp_min(0)
        g = (grad_loss.float() * valid)[:, None]
        dh = torch.zeros_like(h)
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        db = torch.zeros(V, dtype=torch.float32, device=weight.device) if has_bias else None
        coef = 1.0 + 2.0 * zw * lse if zw else None
        for c0 in range(0, V, chunk):
            c1 = min(V, c0 + chunk)
            wc = weight[c0:c1].float()
            lg = h @ wc.t()
            if has_bias:
                lg = lg + bias[c0:c1].float()
            p = torch.exp(lg - lse[:, None])
            if coef is not None:
                p = p * coef[:, None]
            if eps:
                p = p - eps / V
            inside = valid & (safe >= c0) & (safe < c1)
            rows = inside.nonzero(as_tuple=True)[0]
            p[rows, safe[rows] - c0] -= (1.0 - eps)
            p = p * g
            dh += p @ wc
            dw[c0:c1] = p.t() @ h
            if db is not None:
                db[c0:c1] = p.sum(0)
        return (dh.to(hidden.dtype), dw.to(weight.dtype), db.to(bias.dtype) if has_bias else None,
                None, None, None, None, None)


def linear_cross_entropy_chunked(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                                 bias: Optional[torch.Tensor] = None, ignore_index: int = -100,
                                 label_smoothing: float = 0.0, z_loss_weight: float = 0.0,
                                 reduction: str = "mean", chunk_size: int = 8192) -> torch.Tensor:
    h = hidden.reshape(-1, hidden.shape[-1])
    y = labels.reshape(-1)
    per_tok = _ChunkedLinearCE.apply(h, weight, bias, y, ignore_index, label_smoothing, z_loss_weight, int(chunk_size))
    if reduction == "none":
        return per_tok
    if reduction == "sum":
        return per_tok.sum()
    return per_tok.sum() / (y != ignore_index).sum().clamp_min(1)


def cross_entropy_logits(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         label_smoothing: float = 0.0, z_loss_weight: float = 0.0,
                         reduction: str = "mean") -> torch.Tensor:
    """Logits-in cross-entropy with z-loss (reference triton_kernels.py:127-257)."""
    lg = logits.reshape(-1, logits.shape[-1]).float()
    y = labels.reshape(-1)
    loss = F.cross_entropy(lg, y, ignore_index=ignore_index, label_smoothing=label_smoothing, reduction="none")
    if z_loss_weight:
        loss = loss + z_loss_weight * torch.logsumexp(lg, -1).pow(2) * (y != ignore_index)
    if reduction == "none":
        return loss
    if reduction == "sum":
        return loss.sum()
    return loss.sum() / (y != ignore_index).sum().clamp_min(1)


# --------------------------------------------------------------------------- optimizer math
def adamw_step_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int, lr: float,
                beta1: float, beta2: float, eps: float, weight_decay: float, clip_coef: float = 1.0,
                master: Optional[torch.Tensor] = None) -> None:
    """One AdamW update in the reference's order (fused_adamw.py:45-101):
    clip-scale g, decoupled decay, moments, bias-corrected step.  ``master``
    (fp32) receives the update when given; ``p`` is then its rounded copy."""
    gf = g.float() * clip_coef
    w = master if master is not None else p.float()
    w.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    w.addcdiv_(m, denom, value=-lr / bc1)
    if master is not None or p.dtype != torch.float32:
        p.copy_(w)
    elif w.data_ptr() != p.data_ptr():
        p.copy_(w)


def clip_coef_from_sqnorm(sq_norm: torch.Tensor, max_norm: float) -> torch.Tensor:
    """``min(1, max_norm / (‖g‖ + 1e-6))`` (reference fused_adamw.py:205-219)."""
    return torch.clamp(max_norm / (sq_norm.sqrt() + 1e-6), max=1.0)


# --------------------------------------------------------------------------- MXFP8 (OCP microscaling)
E4M3_MAX = 448.0
E5M2_MAX = 57344.0
MX_BLOCK = 32


def _round_to_fp8(x: torch.Tensor, fmt: str) -> torch.Tensor:
    dt = torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2
    mx = E4M3_MAX if fmt == "e4m3" else E5M2_MAX
    return x.clamp(-mx, mx).to(dt)


def mxfp8_quantize(x: torch.Tensor, fmt: str = "e4m3") -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise along the last dim in blocks of 32 with power-of-two (e8m0)
    scales: ``scale = 2^ceil(log2(amax / fmt_max))``; returns the fp8 tensor
    and the biased uint8 exponents ``[..., K/32]`` (bias 127)."""
    K = x.shape[-1]
    assert K % MX_BLOCK == 0, "last dim must be a multiple of 32"
    mx = E4M3_MAX if fmt == "e4m3" else E5M2_MAX
    xb = x.float().reshape(*x.shape[:-1], K // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(-1)
    # exponent e with 2^e >= amax/mx, computed exactly via frexp
    ratio = amax / mx
    mant, exp = torch.frexp(ratio)                      # ratio = mant * 2^exp, mant in [0.5, 1)
    e = torch.where(mant == 0.5, exp - 1, exp)          # exact powers of two need no round-up
    e = torch.where(amax == 0, torch.full_like(e, -127), e).clamp(-127, 127)
    scale = torch.exp2(e.float())
    q = _round_to_fp8(xb / scale[..., None], fmt).reshape(x.shape)
    return q, (e + 127).to(torch.uint8)


def mxfp8_dequantize(q: torch.Tensor, scales_e8m0: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    K = q.shape[-1]
    qb = q.float().reshape(*q.shape[:-1], K // MX_BLOCK, MX_BLOCK)
    scale = torch.exp2(scales_e8m0.float() - 127.0)
    return (qb * scale[..., None]).reshape(q.shape).to(dtype)


def mxfp8_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reference result of a block-scaled MXFP8 GEMM: quantise both operands
    along K, dequantise exactly, multiply in fp32."""
    xq, xs = mxfp8_quantize(x)
    wq, ws = mxfp8_quantize(w)
    y = mxfp8_dequantize(xq, xs) @ mxfp8_dequantize(wq, ws).t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


# --------------------------------------------------------------------------- block-wise 8-bit optimizer state
def quantize_blockwise_8bit(x: torch.Tensor, block: int = 256, signed: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Linear absmax quantisation in blocks of ``block`` elements."""
    flat = x.float().reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = F.pad(flat, (0, pad))
    b = flat.view(-1, block)
    absmax = b.abs().amax(-1).clamp_min(1e-30)
    if signed:
        q = torch.round(b / absmax[:, None] * 127.0).clamp(-127, 127).to(torch.int8)
    else:
        q = torch.round(b / absmax[:, None] * 255.0).clamp(0, 255).to(torch.uint8)
    return q.view(-1)[: x.numel()] if not pad else q.view(-1), absmax


def dequantize_blockwise_8bit(q: torch.Tensor, absmax: torch.Tensor, shape: Sequence[int], block: int = 256,
                              signed: bool = True) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    flat = q.float()
    pad = (-flat.numel()) % block
    if pad:
        flat = F.pad(flat, (0, pad))
    b = flat.view(-1, block)
    out = b * (absmax[:, None] / (127.0 if signed else 255.0))
    return out.view(-1)[:n].view(*shape)
