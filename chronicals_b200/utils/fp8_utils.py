"""Basic FP8 helpers: formats, a quantise/dequantise handler with loss-scale bookkeeping, a linear
layer with FP8 operands, and a memory estimate.

Reference: chronicals/utils/fp8_utils.py:16-21 ``FP8Format``, :24-269 ``FP8Handler`` (per-block(128)
or per-tensor scaling, overflow back-off, amax history), :272-339 ``FP8Linear``, :342-366
``compute_fp8_memory_savings``.  The reference simulates FP8 (quantise → dequantise → bf16 matmul with
rounding done by hand); here conversions are the hardware's (``torch.float8_*`` / ``cvt.*.satfinite``)
and block scaling follows the OCP MX convention (32-element blocks, power-of-two scales) unless a
per-tensor scale is asked for.
"""
from __future__ import annotations

from collections import deque
from enum import Enum
from typing import Deque, Dict, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import _ext, ref


class FP8Format(Enum):
    E4M3 = "e4m3"
    E5M2 = "e5m2"

    @property
    def max_value(self) -> float:
        return ref.E4M3_MAX if self is FP8Format.E4M3 else ref.E5M2_MAX

    @property
    def torch_dtype(self) -> torch.dtype:
        return torch.float8_e4m3fn if self is FP8Format.E4M3 else torch.float8_e5m2


def mxfp8_quantize(x: torch.Tensor, fmt: str = "e4m3", want_dequantized: bool = False):
    """``(q_fp8, scales_e8m0[, x_dequantized_bf16])`` along the last dim in 32-element blocks.
    CUDA bf16 inputs run the quantisation kernel; everything else the PyTorch formula."""
    K = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16 and K % 32 == 0 and _ext.available() and _ext.has_symbol("cb_mxfp8_quant"):
        x2 = x.reshape(-1, K)
        if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
            x2 = x2.contiguous()
        M = x2.shape[0]
        q = torch.empty(M, K, dtype=torch.uint8, device=x.device)
        s = torch.empty(M, K // 32, dtype=torch.uint8, device=x.device)
        d = torch.empty(M, K, dtype=torch.bfloat16, device=x.device) if want_dequantized else None
        fn = _ext.lib().cb_mxfp8_quant
        fn.argtypes = [_ext.P, _ext.P, _ext.P, _ext.P, _ext.L, _ext.I, _ext.L, _ext.I, _ext.P]
        _ext.check(fn(x2.data_ptr(), q.data_ptr(), s.data_ptr(), _ext.ptr(d), M, K, x2.stride(0), int(fmt == "e5m2"),
                      _ext.stream_ptr()), "mxfp8_quant")
        qv = q.view(torch.float8_e5m2 if fmt == "e5m2" else torch.float8_e4m3fn).view(*x.shape)
        sv = s.view(*x.shape[:-1], K // 32)
        return (qv, sv, d.view(x.shape)) if want_dequantized else (qv, sv)
    pad = (-K) % 32
    xp = torch.nn.functional.pad(x, (0, pad)) if pad else x          # a ragged last block is zero-extended
    q, s = ref.mxfp8_quantize(xp, fmt)
    if want_dequantized:
        d = ref.mxfp8_dequantize(q, s, x.dtype)
        return q[..., :K], s, d[..., :K]
    return q[..., :K], s


def mxfp8_dequantize(q: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return ref.mxfp8_dequantize(q, scales, dtype)


# --------------------------------------------------------------------------- block-scaled tensor-core GEMM
def pack_mx_scales(scales: torch.Tensor) -> torch.Tensor:
    """Row-major e8m0 scales ``[R, KB]`` → the 512-byte atoms the block-scaled MMA reads: for every
    128 rows × 4 blocks one atom with byte ``(r % 32) * 16 + (r // 32 % 4) * 4 + kb % 4``, atoms ordered
    ``[row block][kb // 4]``.  Rows and blocks beyond the matrix hold 127 (scale 1.0)."""
    R, KB = scales.shape
    rb, kb4 = (R + 127) // 128, (KB + 3) // 4
    full = torch.full((rb * 128, kb4 * 4), 127, dtype=torch.uint8, device=scales.device)
    full[:R, :KB] = scales
    # [rb, r//32%4, r%32, kb4, kb%4] -> [rb, kb4, r%32, r//32%4, kb%4]
    return full.view(rb, 4, 32, kb4, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def unpack_mx_scales(packed: torch.Tensor, R: int, KB: int) -> torch.Tensor:
    """Inverse of :func:`pack_mx_scales`."""
    rb, kb4 = (R + 127) // 128, (KB + 3) // 4
    full = packed.view(rb, kb4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(rb * 128, kb4 * 4)
    return full[:R, :KB].contiguous()


def block_scaled_available() -> bool:
    return _ext.available() and not _ext.reference_forced() and _ext.has_symbol("cb_mxgemm")


def mxfp8_quantize_packed(x: torch.Tensor, fmt: str = "e4m3"):
    """``(q_uint8 [M, K], packed_scales)`` for the block-scaled GEMM; K a multiple of 32."""
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    if x2.is_cuda and x2.dtype == torch.bfloat16 and K % 32 == 0 and block_scaled_available() \
            and _ext.has_symbol("cb_mxfp8_quant_packed"):
        if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
            x2 = x2.contiguous()
        q = torch.empty(M, K, dtype=torch.uint8, device=x2.device)
        nbytes = ((M + 127) // 128) * ((K + 127) // 128) * 512
        if M % 128 or K % 128:
            sf = torch.full((nbytes,), 127, dtype=torch.uint8, device=x2.device)
        else:
            sf = torch.empty(nbytes, dtype=torch.uint8, device=x2.device)
        fn = _ext.lib().cb_mxfp8_quant_packed
        fn.argtypes = [_ext.P, _ext.P, _ext.P, _ext.L, _ext.I, _ext.L, _ext.I, _ext.P]
        _ext.check(fn(x2.data_ptr(), q.data_ptr(), sf.data_ptr(), M, K, x2.stride(0), int(fmt == "e5m2"),
                      _ext.stream_ptr()), "mxfp8_quant_packed")
        return q, sf
    q, s = ref.mxfp8_quantize(x2, fmt)
    return q.view(torch.uint8), pack_mx_scales(s)


def mxfp8_block_scaled_matmul(aq: torch.Tensor, sfa: torch.Tensor, bq: torch.Tensor, sfb: torch.Tensor,
                              bias: Optional[torch.Tensor] = None, a_fmt: str = "e4m3", b_fmt: str = "e4m3") -> torch.Tensor:
    """``C[M, N] = Σ_k (aq·2^sfa)[m, k] (bq·2^sfb)[n, k] + bias`` in bf16; ``aq [M, K]``, ``bq [N, K]`` fp8 bytes,
    scales packed by :func:`pack_mx_scales`.  On a GPU this is one ``tcgen05.mma.kind::mxf8f6f4.block_scale``
    GEMM (the tensor core applies the scales); elsewhere the operands are dequantised and multiplied in fp32."""
    M, K = aq.shape
    N = bq.shape[0]
    if aq.is_cuda and block_scaled_available() and K % 32 == 0 and not (a_fmt == "e5m2" and b_fmt == "e5m2"):
        out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
        fn = _ext.lib().cb_mxgemm
        fn.argtypes = [_ext.P, _ext.P, _ext.P, _ext.P, _ext.P, _ext.P, _ext.I, _ext.I, _ext.I, _ext.L, _ext.L, _ext.L,
                       _ext.I, _ext.I, _ext.P, _ext.P]
        code = fn(aq.data_ptr(), bq.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), out.data_ptr(), _ext.ptr(bias), M, N, K,
                  aq.stride(0), bq.stride(0), out.stride(0), int(a_fmt == "e5m2"), int(b_fmt == "e5m2"),
                  _ext.status_buffer(aq.device).data_ptr(), _ext.stream_ptr())
        _ext.check(code, "mxgemm")
        return out
    fa = torch.float8_e5m2 if a_fmt == "e5m2" else torch.float8_e4m3fn
    fb = torch.float8_e5m2 if b_fmt == "e5m2" else torch.float8_e4m3fn
    a = ref.mxfp8_dequantize(aq.view(fa), unpack_mx_scales(sfa, M, K // 32))
    b = ref.mxfp8_dequantize(bq.view(fb), unpack_mx_scales(sfb, N, K // 32))
    y = a @ b.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(torch.bfloat16 if aq.is_cuda else torch.float32)


class FP8Handler:
    """Quantise / dequantise with either MX block scaling or one delayed per-tensor scale, plus the
    dynamic loss-scale bookkeeping the reference keeps next to it."""

    def __init__(self, fmt: FP8Format = FP8Format.E4M3, block_size: int = 32, per_tensor: bool = False,
                 amax_history_len: int = 32, margin: float = 1.0, init_loss_scale: float = 2.0 ** 15,
                 growth_interval: int = 1000):
        self.fmt, self.block_size, self.per_tensor, self.margin = fmt, block_size, per_tensor, margin
        self.amax_history: Deque[float] = deque(maxlen=amax_history_len)
        self.loss_scale, self.growth_interval = init_loss_scale, growth_interval
        self._good_steps = 0
        self.overflow_count = 0

    # -- scaling -------------------------------------------------------------------------------------------
    def update_amax(self, x: torch.Tensor) -> float:
        a = float(x.detach().abs().max().item()) if x.numel() else 0.0
        self.amax_history.append(a)
        return a

    def get_scale(self) -> float:
        """Delayed scaling: the largest recent amax maps to the format's maximum."""
        amax = max(self.amax_history) if self.amax_history else 0.0
        return (self.fmt.max_value / self.margin) / amax if amax > 0 else 1.0

    def quantize(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.per_tensor:
            self.update_amax(x)
            s = self.get_scale()
            q = (x.float() * s).clamp(-self.fmt.max_value, self.fmt.max_value).to(self.fmt.torch_dtype)
            return q, torch.tensor(1.0 / s, device=x.device)
        return mxfp8_quantize(x, self.fmt.value)

    def dequantize(self, q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        if scale.dtype == torch.uint8:
            return mxfp8_dequantize(q, scale, dtype)
        return (q.float() * scale).to(dtype)

    # -- loss scaling --------------------------------------------------------------------------------------
    def check_overflow(self, grads) -> bool:
        for g in grads:
            if g is not None and not torch.isfinite(g).all():
                return True
        return False

    def update_loss_scale(self, overflow: bool) -> float:
        if overflow:
            self.loss_scale = max(1.0, self.loss_scale / 2)
            self._good_steps = 0
            self.overflow_count += 1
        else:
            self._good_steps += 1
            if self._good_steps >= self.growth_interval:
                self.loss_scale *= 2
                self._good_steps = 0
        return self.loss_scale


def _block_scaled_ok(x2: torch.Tensor, w: torch.Tensor) -> bool:
    return (x2.is_cuda and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and block_scaled_available()
            and x2.shape[1] % 32 == 0 and w.shape[0] % 8 == 0)


class _MXFP8LinearFn(torch.autograd.Function):
    """Linear layer on MXFP8 operands: inputs and weights are rounded to e4m3 with 32-element MX
    scales along K; the gradient of the output is rounded to e5m2 the same way.  The products are
    accumulated in fp32 on the tensor cores.

    On a GPU all three GEMMs (forward, dX, dW) are block-scaled ``tcgen05.mma.kind::mxf8f6f4`` products:
    the tensor core reads the fp8 bytes and applies the e8m0 scales itself.  Where that kernel does not
    apply (CPU, shapes with K not a multiple of 32) the exactly dequantised operands — an fp8 value times a
    power of two is representable in bf16 — go through the bf16 GEMM, which gives the same products."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if _block_scaled_ok(x2, w):
            aq, sa = mxfp8_quantize_packed(x2, "e4m3")
            bq, sb = mxfp8_quantize_packed(w, "e4m3")
            y = mxfp8_block_scaled_matmul(aq, sa, bq, sb, bias)
        else:
            _, _, xd = mxfp8_quantize(x2, "e4m3", True)
            _, _, wd = mxfp8_quantize(w, "e4m3", True)
            y = ops.gemm(xd, wd, bias=bias) if ops._fast(xd, wd) else torch.nn.functional.linear(xd, wd, bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        # a 2-D input gets the GEMM output itself (not a view of it), so in-place ops on it stay legal
        return y if x.dim() == 2 else y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        T, n_out = dy2.shape
        fast = ops._fast(dy2, w)
        hw = _block_scaled_ok(x2, w) and dy2.dtype == torch.bfloat16
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dX = dY W : K runs over the output features -> quantise dY along its last dim, W along dim 0
            if hw and n_out % 32 == 0 and w.shape[1] % 8 == 0:
                gq, gs = mxfp8_quantize_packed(dy2, "e5m2")
                wq, ws = mxfp8_quantize_packed(w.t().contiguous(), "e4m3")              # [in, out], scales along out
                dx = mxfp8_block_scaled_matmul(gq, gs, wq, ws, None, "e5m2", "e4m3").view(ctx.shape)
            else:
                _, _, gd = mxfp8_quantize(dy2, "e5m2", True)
                _, _, wtd = mxfp8_quantize(w.t().contiguous(), "e4m3", True)
                dx = (ops.gemm(gd, wtd) if fast else gd @ wtd.t()).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            # dW = dY^T X : K runs over tokens -> both operands quantised along the token dimension
            if hw and T % 32 == 0:
                gq, gs = mxfp8_quantize_packed(dy2.t().contiguous(), "e5m2")            # [out, T]
                xq, xs = mxfp8_quantize_packed(x2.t().contiguous(), "e4m3")             # [in, T]
                dw = mxfp8_block_scaled_matmul(gq, gs, xq, xs, None, "e5m2", "e4m3")
            else:
                _, _, gtd = mxfp8_quantize(dy2.t().contiguous(), "e5m2", True)
                _, _, xtd = mxfp8_quantize(x2.t().contiguous(), "e4m3", True)
                dw = ops.gemm(gtd, xtd) if fast and gtd.shape[1] % 8 == 0 else (gtd.float() @ xtd.float().t()).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops.colsum(dy2)
        return dx, dw, db


def rowwise_quantize_e4m3(x: torch.Tensor):
    """``(q_uint8 [M, K], scale_fp32 [M])`` with ``scale = amax(row) / 448`` and ``q = e4m3(x / scale)``.
    CUDA bf16 inputs run ``rowquant_e4m3_kernel``; everything else the PyTorch formula (same rounding)."""
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    if x2.is_cuda and x2.dtype == torch.bfloat16 and K % 16 == 0 and _ext.available() and not _ext.reference_forced() \
            and _ext.has_symbol("cb_rowquant_e4m3"):
        if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
            x2 = x2.contiguous()
        q = torch.empty(M, K, dtype=torch.uint8, device=x2.device)
        sc = torch.empty(M, dtype=torch.float32, device=x2.device)
        _ext.check(_ext.lib().cb_rowquant_e4m3(x2.data_ptr(), q.data_ptr(), sc.data_ptr(), M, K, x2.stride(0), q.stride(0),
                                              _ext.stream_ptr()), "rowquant_e4m3")
        return q, sc
    xf = x2.float()
    sc = xf.abs().amax(-1).clamp_min(1e-30) / 448.0
    q = (xf / sc[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    return q, sc


def fp8_rowwise_matmul(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor,
                       bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``(xq ⊙ xs) @ (wq ⊙ ws)ᵀ + bias`` in bf16 from e4m3 operands.  On a GPU this is one
    ``tcgen05.mma.kind::f8f6f4`` GEMM on CTA pairs with the two scale vectors applied in the epilogue."""
    M, K = xq.shape
    N = wq.shape[0]
    if xq.is_cuda and _ext.available() and not _ext.reference_forced() and _ext.has_symbol("cb_gemm2sm_fp8") and K % 16 == 0 \
            and N % 8 == 0:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
        code = _ext.lib().cb_gemm2sm_fp8(xq.data_ptr(), wq.data_ptr(), out.data_ptr(), xs.data_ptr(), ws.data_ptr(),
                                         _ext.ptr(bias), M, N, K, xq.stride(0), wq.stride(0), out.stride(0),
                                         _ext.status_buffer(xq.device).data_ptr(), _ext.stream_ptr())
        _ext.check(code, "gemm2sm_fp8")
        return out
    a = xq.view(torch.float8_e4m3fn).float() * xs[:, None]
    b = wq.view(torch.float8_e4m3fn).float() * ws[:, None]
    y = a @ b.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(torch.bfloat16 if xq.is_cuda else torch.float32)


class _FP8RowwiseLinearFn(torch.autograd.Function):
    """Forward on the FP8 tensor cores (activations quantised per token, weights per output channel, e4m3);
    backward in bf16 from the saved high-precision operands."""

    @staticmethod
    def forward(ctx, x2, w, bias):
        # 2-D in, 2-D out: the output is a fresh tensor (never a view), so in-place ops on it stay legal
        xq, xs = rowwise_quantize_e4m3(x2)
        wq, ws = rowwise_quantize_e4m3(w)
        y = fp8_rowwise_matmul(xq, xs, wq, ws, bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        return y if y.dtype == x2.dtype else y.to(x2.dtype)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = ops.gemm(dy2, w, b_mn=True) if ops._fast(dy2, w) else dy2 @ w
        if ctx.needs_input_grad[1]:
            dw = ops.gemm(dy2, x2, a_mn=True, b_mn=True) if ops._fast(dy2, x2) else dy2.t() @ x2
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops.colsum(dy2)
        return dx, dw, db


def fp8_rowwise_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _FP8RowwiseLinearFn.apply(x2, w, bias)
    return y if x.dim() == 2 else y.view(*x.shape[:-1], w.shape[0])


class FP8RowwiseLinear(nn.Module):
    """``nn.Linear`` whose forward product runs in e4m3 on the tensor cores (per-token / per-channel scales)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] % 16 != 0:
            return torch.nn.functional.linear(x, self.weight, self.bias)
        return fp8_rowwise_linear(x, self.weight, self.bias)


class FP8Linear(nn.Module):
    """``nn.Linear`` replacement computing with MXFP8 operands and a bf16 master weight."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    @classmethod
    def from_linear(cls, lin: nn.Linear) -> "FP8Linear":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, lin.weight.device, lin.weight.dtype)
        with torch.no_grad():
            m.weight.copy_(lin.weight)
            if lin.bias is not None:
                m.bias.copy_(lin.bias)
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] % 32 != 0:
            return torch.nn.functional.linear(x, self.weight, self.bias)
        return _MXFP8LinearFn.apply(x, self.weight, self.bias)


def compute_fp8_memory_savings(num_params: int, activation_elems: int = 0) -> Dict[str, float]:
    """Bytes with bf16 everywhere vs MXFP8 copies (1 byte + 1/32 byte of scale per element)."""
    bf16 = 2.0 * (num_params + activation_elems)
    fp8 = (1.0 + 1.0 / 32) * (num_params + activation_elems)
    return {"bf16_gb": bf16 / 2**30, "mxfp8_gb": fp8 / 2**30, "saved_fraction": 1 - fp8 / bf16 if bf16 else 0.0}
