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
PAIR_TILE_ROWS = 192   # rows of B per tile of the CTA-pair block-scaled kernel (``cb_mxgemm_pair_tile_rows``)


def _padded_tile_rows(tile_rows: int) -> int:
    return (tile_rows + 127) // 128 * 128


def pack_mx_scales(scales: torch.Tensor, tile_rows: int = 128) -> torch.Tensor:
    """Row-major e8m0 scales ``[R, KB]`` → the 512-byte atoms the block-scaled MMA reads: for every
    128 rows × 4 blocks one atom with byte ``(r % 32) * 16 + (r // 32 % 4) * 4 + kb % 4``, atoms ordered
    ``[row block][kb // 4]``.  Rows and blocks beyond the matrix hold 127 (scale 1.0).  With ``tile_rows``
    other than 128 the rows are first grouped in tiles of that many rows, each padded to a multiple of
    128 (the CTA-pair kernel reads the B scales per 192-row tile)."""
    R, KB = scales.shape
    P = _padded_tile_rows(tile_rows)
    tiles, kb4 = (R + tile_rows - 1) // tile_rows, (KB + 3) // 4
    full = torch.full((tiles, P, kb4 * 4), 127, dtype=torch.uint8, device=scales.device)
    body = torch.full((tiles * tile_rows, kb4 * 4), 127, dtype=torch.uint8, device=scales.device)
    body[:R, :KB] = scales
    full[:, :tile_rows] = body.view(tiles, tile_rows, kb4 * 4)
    rb = tiles * P // 128
    # [rb, r//32%4, r%32, kb4, kb%4] -> [rb, kb4, r%32, r//32%4, kb%4]
    return full.view(rb, 4, 32, kb4, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def unpack_mx_scales(packed: torch.Tensor, R: int, KB: int, tile_rows: int = 128) -> torch.Tensor:
    """Inverse of :func:`pack_mx_scales`."""
    P = _padded_tile_rows(tile_rows)
    tiles, kb4 = (R + tile_rows - 1) // tile_rows, (KB + 3) // 4
    rb = tiles * P // 128
    full = packed.view(rb, kb4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(tiles, P, kb4 * 4)
    return full[:, :tile_rows].reshape(tiles * tile_rows, kb4 * 4)[:R, :KB].contiguous()


def block_scaled_available() -> bool:
    return _ext.available() and not _ext.reference_forced() and _ext.has_symbol("cb_mxgemm")


def mxfp8_quantize_packed(x: torch.Tensor, fmt: str = "e4m3", tile_rows: int = 128):
    """``(q_uint8 [M, K], packed_scales)`` for the block-scaled GEMM; K a multiple of 32.  ``tile_rows`` as in
    :func:`pack_mx_scales` (``PAIR_TILE_ROWS`` for the B operand of the CTA-pair kernel)."""
    x2 = x.reshape(-1, x.shape[-1])
    M, K = x2.shape
    if x2.is_cuda and x2.dtype == torch.bfloat16 and K % 32 == 0 and block_scaled_available() \
            and _ext.has_symbol("cb_mxfp8_quant_packed"):
        if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
            x2 = x2.contiguous()
        q = torch.empty(M, K, dtype=torch.uint8, device=x2.device)
        tiles = (M + tile_rows - 1) // tile_rows
        nbytes = tiles * (_padded_tile_rows(tile_rows) // 128) * ((K + 127) // 128) * 512
        if M % tile_rows or tile_rows % 128 or K % 128:
            sf = torch.full((nbytes,), 127, dtype=torch.uint8, device=x2.device)
        else:
            sf = torch.empty(nbytes, dtype=torch.uint8, device=x2.device)
        fn = _ext.lib().cb_mxfp8_quant_packed
        fn.argtypes = [_ext.P, _ext.P, _ext.P, _ext.L, _ext.I, _ext.L, _ext.I, _ext.I, _ext.P]
        _ext.check(fn(x2.data_ptr(), q.data_ptr(), sf.data_ptr(), M, K, x2.stride(0), int(fmt == "e5m2"), tile_rows,
                      _ext.stream_ptr()), "mxfp8_quant_packed")
        return q, sf
    q, s = ref.mxfp8_quantize(x2, fmt)
    return q.view(torch.uint8), pack_mx_scales(s, tile_rows)


def _sf_buffer(rows: int, K: int, tile_rows: int, device) -> torch.Tensor:
    tiles = (rows + tile_rows - 1) // tile_rows
    nbytes = tiles * (_padded_tile_rows(tile_rows) // 128) * ((K + 127) // 128) * 512
    if rows % tile_rows or tile_rows % 128 or K % 128:
        return torch.full((nbytes,), 127, dtype=torch.uint8, device=device)       # padding must hold a finite scale
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def mxfp8_quantize_dual(x: torch.Tensor, fmt: str = "e4m3", row_tile: int = 128, col_tile: int = 128,
                        want_row: bool = True, want_col: bool = True):
    """``(q_row [R, C], sf_row, q_col [C, R], sf_col)``: the MXFP8 copy of ``x`` with blocks along its last
    dimension and the MXFP8 copy of ``xᵀ`` with blocks along the first — what the forward GEMM and the gradient GEMM over the
    other dimension consume; the transposed copy is written by a kernel that transposes in registers, so no
    bf16 transpose of ``x`` is ever materialised.  Scales are packed per ``row_tile`` /
    ``col_tile`` rows (:func:`pack_mx_scales`).  Outputs not asked for are ``None``."""
    R, C = x.shape
    if x.is_cuda and x.dtype == torch.bfloat16 and R % 32 == 0 and C % 32 == 0 and x.stride(0) % 8 == 0 and block_scaled_available() \
            and _ext.has_symbol("cb_mxfp8_quant_transposed") and R // 32 <= 65535:
        if x.stride(1) != 1:
            x = x.contiguous()
        dev = x.device
        q_row = sf_row = q_col = sf_col = None
        if want_row:
            q_row, sf_row = mxfp8_quantize_packed(x, fmt, row_tile)
        if want_col:
            q_col = torch.empty(C, R, dtype=torch.uint8, device=dev)
            sf_col = _sf_buffer(C, R, col_tile, dev)
            fn = _ext.lib().cb_mxfp8_quant_transposed
            fn.argtypes = [_ext.P, _ext.L, _ext.I, _ext.L, _ext.P, _ext.P, _ext.I, _ext.I, _ext.P]
            _ext.check(fn(x.data_ptr(), R, C, x.stride(0), q_col.data_ptr(), sf_col.data_ptr(), col_tile,
                          int(fmt == "e5m2"), _ext.stream_ptr()), "mxfp8_quant_transposed")
        return q_row, sf_row, q_col, sf_col
    q_row = sf_row = q_col = sf_col = None
    if want_row:
        q_row, sf_row = mxfp8_quantize_packed(x, fmt, row_tile)
    if want_col:
        q_col, sf_col = mxfp8_quantize_packed(x.t().contiguous(), fmt, col_tile)
    return q_row, sf_row, q_col, sf_col


def mxfp8_block_scaled_matmul(aq: torch.Tensor, sfa: torch.Tensor, bq: torch.Tensor, sfb: torch.Tensor,
                              bias: Optional[torch.Tensor] = None, a_fmt: str = "e4m3", b_fmt: str = "e4m3",
                              b_tile_rows: int = 128) -> torch.Tensor:
    """``C[M, N] = Σ_k (aq·2^sfa)[m, k] (bq·2^sfb)[n, k] + bias`` in bf16; ``aq [M, K]``, ``bq [N, K]`` fp8 bytes,
    scales packed by :func:`pack_mx_scales`.  On a GPU this is one ``tcgen05.mma.kind::mxf8f6f4.block_scale``
    GEMM (the tensor core applies the scales): the single-CTA kernel (128 × 128 tiles) when the B scales are
    packed per 128 rows, the CTA-pair kernel (256 × 192 tiles) when they are packed per ``PAIR_TILE_ROWS``.
    Elsewhere the operands are dequantised and multiplied in fp32."""
    M, K = aq.shape
    N = bq.shape[0]
    if aq.is_cuda and block_scaled_available() and K % 32 == 0 and not (a_fmt == "e5m2" and b_fmt == "e5m2"):
        out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
        if b_tile_rows == 128:
            fn = _ext.lib().cb_mxgemm
        elif b_tile_rows == PAIR_TILE_ROWS and N % 8 == 0:
            fn = _ext.lib().cb_mxgemm_pair
        else:
            raise ValueError(f"B scales packed for tiles of {b_tile_rows} rows: no kernel reads that layout (N = {N})")
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
    b = ref.mxfp8_dequantize(bq.view(fb), unpack_mx_scales(sfb, N, K // 32, b_tile_rows))
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


def _block_scaled_product(a: torch.Tensor, a_fmt: str, b: torch.Tensor, b_fmt: str,
                          bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] · b [N, K]ᵀ`` with both operands quantised to MXFP8 along K on the fly; the CTA-pair kernel
    whenever its TMA-store epilogue applies (N a multiple of 8), the single-CTA kernel otherwise."""
    tile = PAIR_TILE_ROWS if b.shape[0] % 8 == 0 and _ext.has_symbol("cb_mxgemm_pair") else 128
    aq, sa = mxfp8_quantize_packed(a, a_fmt)
    bq, sb = mxfp8_quantize_packed(b, b_fmt, tile_rows=tile)
    return mxfp8_block_scaled_matmul(aq, sa, bq, sb, bias, a_fmt, b_fmt, b_tile_rows=tile)


class _MXFP8LinearFn(torch.autograd.Function):
    """Linear layer on MXFP8 operands: inputs and weights are rounded to e4m3 with 32-element MX
    scales along the contraction dimension; the gradient of the output is rounded to e5m2 the same way.
    The products are accumulated in fp32 on the tensor cores.

    On a GPU all three GEMMs (forward, dX, dW) are block-scaled ``tcgen05.mma.kind::mxf8f6f4`` products:
    the tensor core reads the fp8 bytes and applies the e8m0 scales itself.  Each of ``x``, ``W`` and ``dY``
    is read once by a kernel that writes both copies the step needs (blocks along the last dimension for one
    GEMM, the transposed matrix with blocks along the first dimension for the other); the backward pass keeps
    the fp8 copies of ``xᵀ`` and ``Wᵀ`` instead of the bf16 tensors.  Where that path does not apply (CPU,
    dimensions that are not multiples of 32) the exactly dequantised operands — an fp8 value times a power of
    two is representable in bf16 — go through the bf16 GEMM, which gives the same products."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        T, n_in = x2.shape
        n_out = w.shape[0]
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        ctx.fused = (_block_scaled_ok(x2, w) and T % 32 == 0 and n_out % 32 == 0 and _ext.has_symbol("cb_mxgemm_pair")
                     and _ext.has_symbol("cb_mxfp8_quant_transposed"))
        if ctx.fused:
            need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
            xq, xs, xtq, xts = mxfp8_quantize_dual(x2, "e4m3", 128, PAIR_TILE_ROWS, True, need_dw)
            wq, ws, wtq, wts = mxfp8_quantize_dual(w, "e4m3", PAIR_TILE_ROWS, PAIR_TILE_ROWS, True, need_dx)
            y = mxfp8_block_scaled_matmul(xq, xs, wq, ws, bias, b_tile_rows=PAIR_TILE_ROWS)
            ctx.save_for_backward(xtq, xts, wtq, wts)
            ctx.dims = (T, n_in, n_out)
        else:
            if _block_scaled_ok(x2, w):
                y = _block_scaled_product(x2, "e4m3", w, "e4m3", bias)
            else:
                _, _, xd = mxfp8_quantize(x2, "e4m3", True)
                _, _, wd = mxfp8_quantize(w, "e4m3", True)
                y = ops.gemm(xd, wd, bias=bias) if ops._fast(xd, wd) else torch.nn.functional.linear(xd, wd, bias)
            ctx.save_for_backward(x2, w)
        # a 2-D input gets the GEMM output itself (not a view of it), so in-place ops on it stay legal
        return y if x.dim() == 2 else y.view(*x.shape[:-1], n_out)

    @staticmethod
    def backward(ctx, dy):
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = db = None
        if ctx.fused:
            xtq, xts, wtq, wts = ctx.saved_tensors
            need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
            gq, gs, gtq, gts = mxfp8_quantize_dual(dy2, "e5m2", 128, 128, need_dx, need_dw)
            if need_dx:       # dX [T, in] = dY [T, out] · (Wᵀ [in, out])ᵀ
                dx = mxfp8_block_scaled_matmul(gq, gs, wtq, wts, None, "e5m2", "e4m3", PAIR_TILE_ROWS).view(ctx.shape)
            if need_dw:       # dW [out, in] = dYᵀ [out, T] · (Xᵀ [in, T])ᵀ
                dw = mxfp8_block_scaled_matmul(gtq, gts, xtq, xts, None, "e5m2", "e4m3", PAIR_TILE_ROWS)
            if ctx.has_bias and ctx.needs_input_grad[2]:
                db = ops.colsum(dy2)
            return dx, dw, db
        x2, w = ctx.saved_tensors
        T, n_out = dy2.shape
        fast = ops._fast(dy2, w)
        hw = _block_scaled_ok(x2, w) and dy2.dtype == torch.bfloat16
        if ctx.needs_input_grad[0]:
            # dX = dY W : K runs over the output features -> quantise dY along its last dim, W along dim 0
            if hw and n_out % 32 == 0 and w.shape[1] % 8 == 0:
                dx = _block_scaled_product(dy2, "e5m2", w.t().contiguous(), "e4m3").view(ctx.shape)   # W^T: [in, out]
            else:
                _, _, gd = mxfp8_quantize(dy2, "e5m2", True)
                _, _, wtd = mxfp8_quantize(w.t().contiguous(), "e4m3", True)
                dx = (ops.gemm(gd, wtd) if fast else gd @ wtd.t()).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            # dW = dY^T X : K runs over tokens -> both operands quantised along the token dimension
            if hw and T % 32 == 0:
                dw = _block_scaled_product(dy2.t().contiguous(), "e5m2", x2.t().contiguous(), "e4m3")  # [out, T] x [in, T]
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
