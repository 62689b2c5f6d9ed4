"""Fused operators: one public function per op, two implementations each.

* CUDA tensors in bf16 run the hand-written sm_100a kernels (``_ext``), wrapped
  in ``torch.autograd.Function`` so forward and backward are both ours.
* Everything else (CPU, fp32) runs the pure-PyTorch formulas in ``ref`` through
  ordinary autograd.  That path is also the test oracle.

On a CUDA device the kernel library is mandatory; a missing library raises.
"""
from __future__ import annotations

import math
import os
import weakref
from typing import Optional, Tuple

import torch

from . import ref
from . import _ext

__all__ = [
    "linear", "gemm", "gemm_dual", "gemm_splitk", "colsum", "rmsnorm", "rmsnorm_residual", "add_rmsnorm", "swiglu", "geglu", "qk_rope_", "embedding",
    "attention_varlen", "attention_qkv_packed", "linear_cross_entropy", "cross_entropy_logits", "kernels_active",
]


# how often an op left the hand-written kernels for a library routine on a CUDA device (by reason)
FALLBACKS: dict = {}
_FUSED_GLU = os.environ.get("CHRONICALS_FUSED_GLU", "1")      # "0": projection and activation as two kernels


def _fast(*tensors: torch.Tensor) -> bool:
    """True when the CUDA kernels handle these tensors (all CUDA + bf16)."""
    if _ext.reference_forced():
        return False
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16:
            return False
    return True


def kernels_active(device="cuda") -> bool:
    return torch.cuda.is_available() and _ext.available()


# ============================================================================ GEMM
def _gemm_ok(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, addend: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, block_n: int = 0, pair_flags: Optional[int] = None) -> torch.Tensor:
    """``C[M,N] = op(A) @ op(B)^T (+bias) (+addend) (+C)`` on the tcgen05 kernel.

    ``a_mn=False``: ``a`` is ``[M, K]``; ``a_mn=True``: ``a`` is ``[K, M]``
    (the operand is used transposed without a copy).  Same for ``b`` with N.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if not (_gemm_ok(a) and _gemm_ok(b) and out.stride(1) == 1):
        # shapes the TMA path cannot address (row pitch not a multiple of 16 bytes): library fallback, counted
        # and reported once so that it never happens unnoticed
        FALLBACKS["gemm_unaligned"] = FALLBACKS.get("gemm_unaligned", 0) + 1
        if FALLBACKS["gemm_unaligned"] == 1 and a.is_cuda:
            import warnings
            warnings.warn(f"ops.gemm: operand pitch not 16-byte aligned (shapes {tuple(a.shape)} x {tuple(b.shape)}); "
                          "this product runs as an fp32 library matmul (see ops.FALLBACKS)", RuntimeWarning, stacklevel=2)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        r = (A.float() @ B.float())
        if bias is not None:
            r = r + bias.float()
        if addend is not None:
            r = r + addend.float()
        if accumulate:
            r = r + out.float()
        out.copy_(r)
        return out
    if addend is not None:
        assert addend.stride(1) == 1 and addend.dtype == torch.bfloat16
    if pair_flags is not None:
        # the CTA-pair kernel with explicit options (tests, benchmarks): bit 0 = whole tiles only, bit 1 = always
        # split a partial last round along K,
        # bits 8.. = tile width 256 / 224 / 192
        code = _ext.lib().cb_gemm2sm_bf16_ex(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), _ext.ptr(bias), _ext.ptr(addend), M, N, K,
            a.stride(0), b.stride(0), out.stride(0), addend.stride(0) if addend is not None else 0,
            int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), int(pair_flags),
            _ext.status_buffer(a.device).data_ptr(), _ext.stream_ptr())
        _ext.check(code, "gemm2sm_bf16_ex")
        return out
    code = _ext.lib().cb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), _ext.ptr(bias), _ext.ptr(addend), M, N, K,
        a.stride(0), b.stride(0), out.stride(0), addend.stride(0) if addend is not None else 0,
        int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), block_n,
        _ext.status_buffer(a.device).data_ptr(), _ext.stream_ptr())
    _ext.check(code, "gemm_bf16")
    return out


def gemm_dual(a: torch.Tensor, b: torch.Tensor, a2: torch.Tensor, b2: torch.Tensor, *, b_mn: bool = False,
              bias: Optional[torch.Tensor] = None, addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``A op(B)ᵀ + A2 op(B2)ᵀ (+bias) (+addend)`` in one kernel: the k-blocks of the second, low-rank product follow
    those of the first in the same tensor-core accumulators (``a [M, K]``, ``a2 [M, K2]``; ``b [N, K]`` and
    ``b2 [N, K2]``, or ``[K, N]`` / ``[K2, N]`` with ``b_mn``).  A frozen projection and its LoRA branch meet
    without a second pass over the output."""
    M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    K2 = a2.shape[1]
    ok = (_fast(a, b, a2, b2) and all(_gemm_ok(t) for t in (a, b, a2, b2))
          and (addend is None or (addend.stride(1) == 1 and addend.dtype == torch.bfloat16)))
    if ok:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
        code = _ext.lib().cb_gemm2sm_bf16_dual(
            a.data_ptr(), b.data_ptr(), a2.data_ptr(), b2.data_ptr(), out.data_ptr(), _ext.ptr(bias), _ext.ptr(addend),
            M, N, K, K2, a.stride(0), b.stride(0), a2.stride(0), b2.stride(0), out.stride(0),
            addend.stride(0) if addend is not None else 0, int(b_mn), _ext.status_buffer(a.device).data_ptr(),
            _ext.stream_ptr())
        if code == 0:
            return out
        if code > 0:
            _ext.check(code, "gemm2sm_bf16_dual")
    out = gemm(a, b, b_mn=b_mn, bias=bias, addend=addend)
    return gemm(a2, b2, b_mn=b_mn, out=out, accumulate=True)


def gemm_splitk(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False) -> torch.Tensor:
    """fp32 ``op(A) @ op(B)^T`` for skinny outputs with a long inner dimension (adapter weight gradients):
    the K range is split across CTAs and the partial tiles are summed with ``red.global.add``."""
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    if not (_gemm_ok(a) and _gemm_ok(b) and _fast(a, b)):
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        return A.float() @ B.float()
    out = torch.empty(M, N, dtype=torch.float32, device=a.device)
    code = _ext.lib().cb_gemm_bf16_splitk(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                          out.stride(0), int(a_mn), int(b_mn), _ext.status_buffer(a.device).data_ptr(),
                                          _ext.stream_ptr())
    _ext.check(code, "gemm_splitk")
    return out


def colsum(x: torch.Tensor) -> torch.Tensor:
    """Column sums of a 2-D tensor in its own dtype with fp32 accumulation (bias gradients)."""
    if _fast(x) and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 \
            and x.data_ptr() % 16 == 0:
        L = _ext.lib()
        M, N = x.shape
        part = torch.empty(L.cb_colsum_blocks(M) * N, dtype=torch.float32, device=x.device)
        out = torch.empty(N, dtype=x.dtype, device=x.device)
        _ext.check(L.cb_colsum_bf16(x.data_ptr(), out.data_ptr(), part.data_ptr(), M, N, x.stride(0), _ext.stream_ptr()),
                   "colsum")
        return out
    return x.float().sum(0).to(x.dtype)


_SM_COUNT = {}


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def wgrad(dy2: torch.Tensor, x2: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dW = dYᵀ X`` (``[out, in]``) of a linear layer.  A small weight with many tokens gives fewer output
    tiles than half the SMs and a long inner dimension (QKV and attention-output projections of a 0.5B model:
    63 and 49 tiles of 128 × 128 over 8192 tokens), so the token range is split across CTAs, the partial tiles
    are added in fp32 by TMA reduce and the sum is rounded once; everything else is one bf16-output GEMM.
    ``out`` (bf16 ``[out, in]``, contiguous) receives the result when given."""
    n_out, n_in, T = dy2.shape[1], x2.shape[1], dy2.shape[0]
    if not _fast(dy2, x2):
        r = dy2.t() @ x2
        return r if out is None else out.copy_(r)
    if T >= 2048 and _gemm_ok(dy2) and _gemm_ok(x2):
        tiles = ((n_out + 127) // 128) * ((n_in + 127) // 128)
        if 2 * tiles <= _sm_count(dy2.device):
            r = gemm_splitk(dy2, x2, a_mn=True, b_mn=True)
            return r.to(dy2.dtype) if out is None else out.copy_(r)
    return gemm(dy2, x2, a_mn=True, b_mn=True, out=out)


def grad_destination(param: torch.Tensor) -> Optional[torch.Tensor]:
    """Where a weight-gradient kernel may write its result directly, or None.  An optimizer that keeps all
    gradients in one flat buffer (``parallel.zero.ShardedFusedAdamW``) attaches ``_cb_grad_out`` to its
    parameters: a callable that returns a fresh view of the parameter's slot while the slot holds nothing of the
    current step yet.  The backward pass then returns that view as the gradient, autograd adopts it without a
    copy, and no separate gradient tensor is ever allocated."""
    fn = getattr(param, "_cb_grad_out", None)
    return fn() if fn is not None else None


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w, bias, res2):
        # 2-D in, 2-D out: the output is a fresh tensor (never a view), so later in-place ops
        # on it (the rotary embedding) are legal for autograd
        y = gemm(x2, w, bias=bias, addend=res2)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.has_res = res2 is not None
        # saved tensors come back as new Python objects; the parameter object itself carries the optimizer's
        # gradient destination
        ctx.weight_ref = weakref.ref(w) if hasattr(w, "_cb_grad_out") else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True)                             # dX = dY @ W
        if ctx.needs_input_grad[1]:
            dw = wgrad(dy2, x2, out=grad_destination(ctx.weight_ref()) if ctx.weight_ref is not None else None)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = colsum(dy2)
        dres = dy2 if ctx.has_res else None
        return dx, dw, db, dres


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T + bias (+ residual)``; the residual add is fused in the GEMM epilogue."""
    if _fast(x, w, bias, residual):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        y = _LinearFn.apply(x2, w, bias, res2)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], w.shape[0])
    y = torch.nn.functional.linear(x, w, bias)
    return y + residual if residual is not None else y


# ============================================================================ RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps, offset):
        N = x.shape[-1]
        x2 = x.reshape(-1, N)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        h = None
        if residual is not None:
            r2 = residual.reshape(-1, N)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            h = torch.empty_like(x2)
        code = _ext.lib().cb_rmsnorm_fwd(x2.data_ptr(), _ext.ptr(r2) if residual is not None else None, w.data_ptr(),
                                         y.data_ptr(), _ext.ptr(h), rstd.data_ptr(), M, N, eps, offset,
                                         _ext.stream_ptr())
        _ext.check(code, "rmsnorm_fwd")
        ctx.save_for_backward(h if h is not None else x2, w, rstd)
        ctx.offset = offset
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        ctx.set_materialize_grads(False)
        if residual is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        M, N = h.shape
        if dy is None:
            dy = torch.zeros_like(h)
        dy2 = dy.reshape(M, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dh is not None:
            dres = dh.reshape(M, N)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        L = _ext.lib()
        blocks = L.cb_rmsnorm_bwd_blocks(M, N)
        part = torch.empty(blocks * N, dtype=torch.float32, device=h.device)
        dx = torch.empty_like(h)
        dw = torch.empty_like(w)
        code = L.cb_rmsnorm_bwd(dy2.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _ext.ptr(dres),
                                dx.data_ptr(), dw.data_ptr(), part.data_ptr(), M, N, ctx.offset, 0, _ext.stream_ptr())
        _ext.check(code, "rmsnorm_bwd")
        dxv = dx.view(ctx.shape)
        return dxv, (dxv if ctx.has_res else None), dw, None, None


class _RMSNormPassFn(torch.autograd.Function):
    """``(rmsnorm(x), x)``: the second output is the input itself, handed on as the residual of the following
    projection.  Its gradient comes back here and is added inside the RMSNorm backward kernel (``dres_in``), so the
    two gradient contributions of the residual stream are summed without a separate elementwise kernel."""

    @staticmethod
    def forward(ctx, x, w, eps, offset):
        N = x.shape[-1]
        x2 = x.reshape(-1, N)
        M = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        code = _ext.lib().cb_rmsnorm_fwd(x2.data_ptr(), None, w.data_ptr(), y.data_ptr(), None, rstd.data_ptr(), M, N, eps,
                                         offset, _ext.stream_ptr())
        _ext.check(code, "rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.offset = offset
        ctx.shape = x.shape
        ctx.set_materialize_grads(False)
        return y.view(x.shape), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dpass):
        x2, w, rstd = ctx.saved_tensors
        M, N = x2.shape
        if dy is None:
            return (dpass, None, None, None)
        dy2 = dy.reshape(M, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dpass is not None:
            dres = dpass.reshape(M, N)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        L = _ext.lib()
        part = torch.empty(L.cb_rmsnorm_bwd_blocks(M, N) * N, dtype=torch.float32, device=x2.device)
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        code = L.cb_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(), _ext.ptr(dres), dx.data_ptr(),
                                dw.data_ptr(), part.data_ptr(), M, N, ctx.offset, 0, _ext.stream_ptr())
        _ext.check(code, "rmsnorm_bwd")
        return dx.view(ctx.shape), dw, None, None


def rmsnorm_residual(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, offset: float = 0.0
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(rmsnorm(x), x)`` for the pre-norm residual pattern ``x + f(rmsnorm(x))``: use the second value as the
    residual so that its gradient is folded into the norm's backward kernel."""
    if _rms_fast(x, weight) and x.is_contiguous():
        return _RMSNormPassFn.apply(x, weight, eps, offset)
    return ref.rmsnorm(x, weight, eps, offset), x


def _rms_fast(x, w) -> bool:
    return _fast(x, w) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, offset: float = 0.0) -> torch.Tensor:
    if _rms_fast(x, weight):
        return _RMSNormFn.apply(x, None, weight, eps, offset)[0]
    return ref.rmsnorm(x, weight, eps, offset)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``h = x + residual; y = rmsnorm(h)``; returns ``(y, h)`` from one kernel."""
    if _rms_fast(x, weight) and _fast(residual):
        return _RMSNormFn.apply(x, residual, weight, eps, 0.0)
    return ref.add_rmsnorm(x, residual, weight, eps)


# ============================================================================ gated activations
class _GLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up, gelu):
        I = gate_up.shape[-1] // 2
        gu = gate_up.reshape(-1, 2 * I)
        if not gu.is_contiguous():
            gu = gu.contiguous()
        M = gu.shape[0]
        out = torch.empty(M, I, dtype=gu.dtype, device=gu.device)
        code = _ext.lib().cb_glu_fwd(gu.data_ptr(), gu.data_ptr() + 2 * I, out.data_ptr(), M, I, 2 * I, I, int(gelu),
                                     _ext.stream_ptr())
        _ext.check(code, "glu_fwd")
        ctx.save_for_backward(gu)
        ctx.gelu = gelu
        ctx.shape = gate_up.shape
        return out.view(*gate_up.shape[:-1], I)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        M, I2 = gu.shape
        I = I2 // 2
        d2 = dout.reshape(M, I)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(gu)
        code = _ext.lib().cb_glu_bwd(d2.data_ptr(), gu.data_ptr(), gu.data_ptr() + 2 * I, dgu.data_ptr(),
                                     dgu.data_ptr() + 2 * I, M, I, I, I2, I2, int(ctx.gelu), _ext.stream_ptr())
        _ext.check(code, "glu_bwd")
        return dgu.view(ctx.shape), None


class _LinearSwiGLUFn(torch.autograd.Function):
    """``act = silu(x Wgᵀ + bg) * (x Wuᵀ + bu)`` for the fused gate | up weight ``w [2I, K]``.

    Forward: one CTA-pair GEMM whose epilogue stores gate | up (kept for the backward pass) and the activation
    (``cb_gemm2sm_bf16_glu``), so the ``[T, 2I]`` tensor is not read back by a separate activation kernel.
    Backward: the stand-alone gated-activation backward on the stored gate | up, then the usual dgrad / wgrad.
    The reference patches Liger's SwiGLU MLP in for the same purpose (chronicals/training/chronicals_trainer.py:704-816)."""

    @staticmethod
    def forward(ctx, x2, w, bias):
        M, K = x2.shape
        I = w.shape[0] // 2
        gu = torch.empty(M, 2 * I, dtype=x2.dtype, device=x2.device)
        act = torch.empty(M, I, dtype=x2.dtype, device=x2.device)
        code = _ext.lib().cb_gemm2sm_bf16_glu(x2.data_ptr(), w.data_ptr(), gu.data_ptr(), act.data_ptr(), _ext.ptr(bias),
                                              M, I, K, x2.stride(0), w.stride(0), gu.stride(0), act.stride(0),
                                              _ext.status_buffer(x2.device).data_ptr(), _ext.stream_ptr())
        if code > 0:
            _ext.check(code, "gemm2sm_bf16_glu")
        if code != 0:                                            # shape not covered: projection, then activation
            gemm(x2, w, bias=bias, out=gu)
            c2 = _ext.lib().cb_glu_fwd(gu.data_ptr(), gu.data_ptr() + 2 * I, act.data_ptr(), M, I, 2 * I, I, 0, _ext.stream_ptr())
            _ext.check(c2, "glu_fwd")
        ctx.save_for_backward(x2, w, gu)
        ctx.has_bias = bias is not None
        ctx.weight_ref = weakref.ref(w) if hasattr(w, "_cb_grad_out") else None
        return act

    @staticmethod
    def backward(ctx, dact):
        x2, w, gu = ctx.saved_tensors
        M, I2 = gu.shape
        I = I2 // 2
        d2 = dact.reshape(M, I)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(gu)
        code = _ext.lib().cb_glu_bwd(d2.data_ptr(), gu.data_ptr(), gu.data_ptr() + 2 * I, dgu.data_ptr(),
                                     dgu.data_ptr() + 2 * I, M, I, I, I2, I2, 0, _ext.stream_ptr())
        _ext.check(code, "glu_bwd")
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dgu, w, b_mn=True)
        if ctx.needs_input_grad[1]:
            dw = wgrad(dgu, x2, out=grad_destination(ctx.weight_ref()) if ctx.weight_ref is not None else None)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = colsum(dgu)
        return dx, dw, db


def linear_swiglu(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gate) * up`` of the fused gate | up projection ``x @ w.T + bias`` (``w [2I, K]``, gate rows first),
    with the activation computed in the projection's epilogue where the shape allows (``I % 128 == 0``).
    ``CHRONICALS_FUSED_GLU=0`` in the environment keeps projection and activation apart."""
    I = w.shape[0] // 2
    # Measured (8192 tokens): 0.5B shapes 0.142 ms fused against 0.161 ms for GEMM + activation kernel, 7B shapes
    # 1.517 against 1.869 ms.  The activation has to be cheap for that: the four epilogue warps of a CTA run one per
    # scheduler, and with an exp2 + reciprocal sigmoid the epilogue of the K = 896 tiles outlasted the next tile's
    # main loop (0.311 ms); the tanh.approx form fits.
    pays = _FUSED_GLU != "0"
    if (pays and _fast(x, w, bias) and I % 128 == 0 and x.shape[-1] % 8 == 0 and _ext.has_symbol("cb_gemm2sm_bf16_glu")
            and w.stride(1) == 1):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        a = _LinearSwiGLUFn.apply(x2, w, bias)
        return a if x.dim() == 2 else a.view(*x.shape[:-1], I)
    return swiglu(linear(x, w, bias))


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for a ``[..., 2I]`` tensor holding ``gate | up``."""
    if _fast(gate_up) and (gate_up.shape[-1] // 2) % 8 == 0:
        return _GLUFn.apply(gate_up, False)
    return ref.swiglu_packed(gate_up)


def geglu(gate_up: torch.Tensor) -> torch.Tensor:
    if _fast(gate_up) and (gate_up.shape[-1] // 2) % 8 == 0:
        return _GLUFn.apply(gate_up, True)
    return ref.geglu_packed(gate_up)


# ============================================================================ RoPE
def _rope_launch(qkv: torch.Tensor, cos, sin, pos, hq, hk, d, interleaved, inverse):
    T = qkv.shape[0]
    ld = qkv.stride(0)
    code = _ext.lib().cb_qk_rope(qkv.data_ptr(), qkv.data_ptr() + 2 * hq * d, cos.data_ptr(), sin.data_ptr(),
                                 _ext.ptr(pos), T, hq, hk, d, ld, ld, int(interleaved), int(inverse), cos.shape[0],
                                 _ext.stream_ptr())
    _ext.check(code, "qk_rope")


class _QKRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, pos, hq, hk, d, interleaved):
        _rope_launch(qkv, cos, sin, pos, hq, hk, d, interleaved, False)
        ctx.mark_dirty(qkv)
        ctx.save_for_backward(cos, sin, pos if pos is not None else torch.empty(0))
        ctx.cfg = (hq, hk, d, interleaved, pos is not None)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        cos, sin, pos = ctx.saved_tensors
        hq, hk, d, interleaved, has_pos = ctx.cfg
        # the incoming gradient is a fresh buffer owned by this node (produced by the attention
        # backward), so the inverse rotation runs in place on it
        g = dqkv if dqkv.is_contiguous() else dqkv.contiguous()
        _rope_launch(g, cos, sin, pos if has_pos else None, hq, hk, d, interleaved, True)
        return g, None, None, None, None, None, None, None


def qk_rope_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, position_ids: Optional[torch.Tensor],
             num_q_heads: int, num_kv_heads: int, head_dim: int, interleaved: bool = False) -> torch.Tensor:
    """Rotate the Q and K heads of a packed ``[T, (hq + 2 hk) * d]`` QKV buffer
    (V untouched).  In place on CUDA; returns the rotated buffer."""
    if _fast(qkv) and qkv.dim() == 2 and head_dim % 16 == 0 and cos.is_cuda:
        if position_ids is not None and position_ids.dtype != torch.int64:
            position_ids = position_ids.long()
        return _QKRopeFn.apply(qkv, cos, sin, position_ids, num_q_heads, num_kv_heads, head_dim, interleaved)
    T = qkv.shape[0]
    nq, nk = num_q_heads * head_dim, num_kv_heads * head_dim
    q = qkv[:, :nq].reshape(T, num_q_heads, head_dim)
    k = qkv[:, nq:nq + nk].reshape(T, num_kv_heads, head_dim)
    q = ref.apply_rope(q, cos, sin, position_ids, interleaved)
    k = ref.apply_rope(k, cos, sin, position_ids, interleaved)
    return torch.cat((q.reshape(T, nq), k.reshape(T, nk), qkv[:, nq + nk:]), dim=-1)


# ============================================================================ embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1)
        T = flat.numel()
        V, N = table.shape
        out = torch.empty(T, N, dtype=table.dtype, device=table.device)
        code = _ext.lib().cb_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(), T, N, V,
                                           _ext.stream_ptr())
        _ext.check(code, "embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.tshape = table.shape
        return out.view(*ids.shape, N)

    @staticmethod
    def backward(ctx, dout):
        (flat,) = ctx.saved_tensors
        V, N = ctx.tshape
        T = flat.numel()
        d2 = dout.reshape(T, N)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        sorted_ids, perm = torch.sort(flat)
        dtable = torch.zeros(V, N, dtype=dout.dtype, device=dout.device)
        code = _ext.lib().cb_embedding_bwd(sorted_ids.data_ptr(), perm.data_ptr(), d2.data_ptr(), dtable.data_ptr(),
                                           T, N, V, 0, _ext.stream_ptr())
        _ext.check(code, "embedding_bwd")
        return None, dtable


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if _fast(table) and ids.is_cuda and table.shape[1] % 8 == 0 and table.is_contiguous():
        return _EmbeddingFn.apply(ids.long(), table)
    return torch.nn.functional.embedding(ids, table)


# ============================================================================ attention
def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                     max_seqlen: Optional[int] = None, causal: bool = True,
                     softmax_scale: Optional[float] = None, seqlens_host=None) -> torch.Tensor:
    """Causal GQA attention over packed documents (``q [T,Hq,D]``, ``k/v [T,Hk,D]``)."""
    from . import attention as _attn
    return _attn.attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, softmax_scale, seqlens_host)


def attention_qkv_packed(qkv: torch.Tensor, cu_seqlens: torch.Tensor, num_q_heads: int, num_kv_heads: int,
                         head_dim: int, max_seqlen: Optional[int] = None, seqlens_host=None) -> torch.Tensor:
    """Causal GQA attention reading Q, K, V straight out of the fused ``[T, (hq + 2 hk) * D]``
    projection output; returns ``[T, hq * D]``."""
    from . import attention_cuda as _ac
    if qkv.dim() == 2 and _ac.kernel_supports(qkv, head_dim):
        return _ac.attention_qkv_packed(qkv, cu_seqlens, num_q_heads, num_kv_heads, head_dim)
    T = qkv.shape[0]
    nq, nk = num_q_heads * head_dim, num_kv_heads * head_dim
    q = qkv[:, :nq].reshape(T, num_q_heads, head_dim)
    k = qkv[:, nq:nq + nk].reshape(T, num_kv_heads, head_dim)
    v = qkv[:, nq + nk:].reshape(T, num_kv_heads, head_dim)
    return attention_varlen(q, k, v, cu_seqlens, max_seqlen, True, None, seqlens_host).reshape(T, nq)


# ============================================================================ fused linear + cross-entropy
CCE_BWD_CHUNK = 8192   # vocab columns whose d(logits) exist at any one time in the backward


class _LinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, smoothing, z_weight, mean):
        L = _ext.lib()
        M, K = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        n_splits = L.cb_cce_num_splits(M, V)
        part = torch.empty(3 if smoothing else 2, n_splits, M, dtype=torch.float32, device=dev)
        tgt = torch.zeros(M, dtype=torch.float32, device=dev)
        status = _ext.status_buffer(dev)
        code = L.cb_cce_forward(hidden.data_ptr(), weight.data_ptr(), labels.data_ptr(), M, V, K, hidden.stride(0),
                                weight.stride(0), 0, part[0].data_ptr(), part[1].data_ptr(),
                                part[2].data_ptr() if smoothing else None, tgt.data_ptr(), status.data_ptr(),
                                _ext.stream_ptr())
        _ext.check(code, "cce_forward")
        lse = torch.empty(M, dtype=torch.float32, device=dev)
        loss_rows = torch.empty(M, dtype=torch.float32, device=dev)
        out = torch.empty(2, dtype=torch.float32, device=dev)
        gscale = torch.empty(M, dtype=torch.float32, device=dev)
        code = L.cb_cce_combine(part[0].data_ptr(), part[1].data_ptr(), part[2].data_ptr() if smoothing else None,
                                tgt.data_ptr(), labels.data_ptr(), M, n_splits, V, smoothing, z_weight, ignore_index,
                                int(mean), lse.data_ptr(), loss_rows.data_ptr(), out.data_ptr(), gscale.data_ptr(),
                                _ext.stream_ptr())
        _ext.check(code, "cce_combine")
        ctx.save_for_backward(hidden, weight, labels, lse, gscale)
        ctx.cfg = (smoothing, z_weight)
        ctx.set_materialize_grads(False)
        return out[0], loss_rows

    @staticmethod
    def backward(ctx, gout, grows):
        hidden, weight, labels, lse, gscale = ctx.saved_tensors
        smoothing, z_weight = ctx.cfg
        L = _ext.lib()
        M, K = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        status = _ext.status_buffer(dev)
        if grows is None and gout is not None:
            g1 = gout.float().reshape(1).contiguous()     # the usual case: scalar loss, no extra kernels
        else:
            # gradient arriving through the per-row losses (reduction='none'/'sum' users)
            rows_scale = torch.zeros_like(gscale)
            if gout is not None:
                rows_scale = rows_scale + gscale * gout.float()
            if grows is not None:
                rows_scale = rows_scale + grows.float() * (labels != -100)
            gscale = rows_scale.contiguous()
            g1 = torch.ones(1, dtype=torch.float32, device=dev)
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        Vc = min(CCE_BWD_CHUNK, (V + 7) // 8 * 8)
        G = torch.empty(M, Vc, dtype=torch.bfloat16, device=dev)
        dh32 = torch.empty(M, K, dtype=torch.float32, device=dev) if need_dh else None
        dw = torch.empty_like(weight) if need_dw else None
        for c0 in range(0, V, Vc):
            vc = min(Vc, V - c0)
            wc = weight[c0:c0 + vc]
            code = L.cb_cce_dlogits(hidden.data_ptr(), wc.data_ptr(), labels.data_ptr(), lse.data_ptr(),
                                    gscale.data_ptr(), g1.data_ptr(), G.data_ptr(), M, vc, K, hidden.stride(0),
                                    weight.stride(0), G.stride(0), c0, V, smoothing, z_weight, status.data_ptr(),
                                    _ext.stream_ptr())
            _ext.check(code, "cce_dlogits")
            Gc = G[:, :vc]
            if need_dh:   # dH += G_c @ W_c
                gemm(Gc, wc, b_mn=True, out=dh32, accumulate=c0 > 0)
            if need_dw:   # dW_c = G_c^T @ H
                gemm(Gc, hidden, a_mn=True, b_mn=True, out=dw[c0:c0 + vc])
        dh = dh32.to(hidden.dtype) if need_dh else None
        return dh, dw, None, None, None, None, None


# Optional second form of the fused linear cross-entropy: with CHRONICALS_CCE_RESIDENT_GB=<n> (default 0: off) the
# [tokens, vocab] logits are kept in bf16 between forward and backward when they take at most n GB, and the
# backward pass needs no second projection onto the vocabulary (8192 tokens x 151,936 words: 2.5 GB kept,
# 2.2 TFLOP saved).  Measured inside the CUDA-graph step of the 0.5B benchmark the two forms take the same time
# (35.7 ms either way: the extra pass over 2.5 GB of logits and the long-K GEMMs cost what the recomputation did),
# so the form that never holds the logits stays the default; with eager launches the resident form saves 55
# launches per step.
CCE_RESIDENT_BYTES = int(float(os.environ.get("CHRONICALS_CCE_RESIDENT_GB", "0")) * 2 ** 30)


class _LinearCEResidentFn(torch.autograd.Function):
    """Same loss and gradients as ``_LinearCEFn`` with the logits resident in device memory:

    forward : logits = H Wᵀ (bf16, CTA-pair GEMM) -> one pass per row for log-sum-exp, target logit and loss;
    backward: d(logits) written over the logits in one pass, then dH = G W and dW = Gᵀ H as two plain GEMMs over the
              whole vocabulary.  The reference's cut cross-entropy (chronicals/kernels/cut_cross_entropy.py:252-424)
    trades this memory for recomputation; ``_LinearCEFn`` is that form."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, smoothing, z_weight, mean):
        L = _ext.lib()
        M, K = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        logits = gemm(hidden, weight)
        loss_rows = torch.empty(M, dtype=torch.float32, device=dev)
        lse = torch.empty(M, dtype=torch.float32, device=dev)
        code = L.cb_ce_logits(logits.data_ptr(), labels.data_ptr(), M, logits.stride(0), V, 1, ignore_index, smoothing,
                              z_weight, loss_rows.data_ptr(), lse.data_ptr(), _ext.stream_ptr())
        _ext.check(code, "ce_logits")
        valid = (labels != ignore_index) & (labels >= 0) & (labels < V)
        if mean:
            n = valid.sum().clamp_min(1).float()
            gscale = valid.float() / n
            loss = loss_rows.sum() / n
        else:
            gscale = valid.float()
            loss = loss_rows.sum()
        ctx.save_for_backward(hidden, weight, labels, lse, gscale, logits)
        ctx.cfg = (ignore_index, smoothing, z_weight)
        ctx.weight_ref = weakref.ref(weight) if hasattr(weight, "_cb_grad_out") else None
        ctx.set_materialize_grads(False)
        return loss, loss_rows

    @staticmethod
    def backward(ctx, gout, grows):
        hidden, weight, labels, lse, gscale, logits = ctx.saved_tensors
        ignore_index, smoothing, z_weight = ctx.cfg
        M, K = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        if grows is None and gout is not None:
            g1 = gout.float().reshape(1).contiguous()
        else:
            rows_scale = torch.zeros_like(gscale)
            if gout is not None:
                rows_scale = rows_scale + gscale * gout.float()
            if grows is not None:
                rows_scale = rows_scale + grows.float() * (labels != ignore_index)
            gscale = rows_scale.contiguous()
            g1 = torch.ones(1, dtype=torch.float32, device=dev)
        # in place: the logits are not needed again (a second backward through this node is not supported)
        code = _ext.lib().cb_ce_logits_grad(logits.data_ptr(), logits.data_ptr(), labels.data_ptr(), lse.data_ptr(),
                                            gscale.data_ptr(), g1.data_ptr(), M, logits.stride(0), V, 1, ignore_index,
                                            smoothing, z_weight, _ext.stream_ptr())
        _ext.check(code, "ce_logits_grad")
        dh = gemm(logits, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dest = grad_destination(ctx.weight_ref()) if ctx.weight_ref is not None else None
            dw = gemm(logits, hidden, a_mn=True, b_mn=True, out=dest)
        return dh, dw, None, None, None, None, None


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                         bias: Optional[torch.Tensor] = None, ignore_index: int = -100,
                         label_smoothing: float = 0.0, z_loss_weight: float = 0.0, reduction: str = "mean",
                         chunk_size: int = 8192) -> torch.Tensor:
    """Cross-entropy of ``hidden @ weight.T`` against ``labels`` (already shifted) without ever holding the
    ``[tokens, vocab]`` logits: online log-sum-exp in the GEMM epilogue, d(logits) recomputed in chunks.  Products of
    at most ``CCE_RESIDENT_BYTES`` (0 unless ``CHRONICALS_CCE_RESIDENT_GB`` is set) keep bf16 logits instead."""
    h = hidden.reshape(-1, hidden.shape[-1])
    y = labels.reshape(-1)
    if (_fast(h, weight) and bias is None and y.is_cuda and h.shape[1] % 8 == 0 and weight.stride(1) == 1
            and weight.stride(0) % 8 == 0 and ignore_index == -100):
        if not h.is_contiguous():
            h = h.contiguous()
        y = y.long().contiguous()
        fn = _LinearCEFn
        if (h.shape[0] * weight.shape[0] * 2 <= CCE_RESIDENT_BYTES and weight.shape[0] % 8 == 0 and _gemm_ok(h)
                and _gemm_ok(weight)):
            fn = _LinearCEResidentFn
        loss, rows = fn.apply(h, weight, y, ignore_index, float(label_smoothing), float(z_loss_weight),
                              reduction == "mean")
        if reduction == "none":
            return rows
        if reduction == "sum":
            return rows.sum()
        return loss
    return ref.linear_cross_entropy_chunked(h, weight, y, bias, ignore_index, label_smoothing, z_loss_weight,
                                            reduction, chunk_size)


# ============================================================================ CE on materialised logits
class _CELogitsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index, smoothing, z_weight):
        L = _ext.lib()
        rows, V = logits.shape
        dev = logits.device
        loss_rows = torch.empty(rows, dtype=torch.float32, device=dev)
        lse = torch.empty(rows, dtype=torch.float32, device=dev)
        code = L.cb_ce_logits(logits.data_ptr(), labels.data_ptr(), rows, logits.stride(0), V,
                              int(logits.dtype == torch.bfloat16), ignore_index, smoothing, z_weight,
                              loss_rows.data_ptr(), lse.data_ptr(), _ext.stream_ptr())
        _ext.check(code, "ce_logits")
        ctx.save_for_backward(logits, labels, lse)
        ctx.cfg = (ignore_index, smoothing, z_weight)
        return loss_rows

    @staticmethod
    def backward(ctx, grows):
        logits, labels, lse = ctx.saved_tensors
        ignore_index, smoothing, z_weight = ctx.cfg
        rows, V = logits.shape
        dl = torch.empty_like(logits)
        one = torch.ones(1, dtype=torch.float32, device=logits.device)
        gs = grows.float().contiguous()
        code = _ext.lib().cb_ce_logits_grad(logits.data_ptr(), dl.data_ptr(), labels.data_ptr(), lse.data_ptr(),
                                            gs.data_ptr(), one.data_ptr(), rows, logits.stride(0), V,
                                            int(logits.dtype == torch.bfloat16), ignore_index, smoothing, z_weight,
                                            _ext.stream_ptr())
        _ext.check(code, "ce_logits_grad")
        return dl, None, None, None, None


def cross_entropy_logits(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         label_smoothing: float = 0.0, z_loss_weight: float = 0.0,
                         reduction: str = "mean") -> torch.Tensor:
    lg = logits.reshape(-1, logits.shape[-1])
    y = labels.reshape(-1)
    if lg.is_cuda and not _ext.reference_forced() and lg.dtype in (torch.bfloat16, torch.float32) and lg.stride(1) == 1:
        rows = _CELogitsFn.apply(lg, y.long().contiguous(), ignore_index, float(label_smoothing), float(z_loss_weight))
        if reduction == "none":
            return rows
        if reduction == "sum":
            return rows.sum()
        return rows.sum() / (y != ignore_index).sum().clamp_min(1)
    return ref.cross_entropy_logits(lg, y, ignore_index, label_smoothing, z_loss_weight, reduction)
