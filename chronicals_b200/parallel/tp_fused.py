"""Fused tensor/sequence-parallel operators over peer memory (the ``"fused"`` back-end of
``parallel.tensor_parallel``).  No counterpart in the reference (single GPU).

Three building blocks, all in ``csrc``:

* ``cb_rmsnorm_push``   — RMSNorm of this rank's ``T/W`` rows whose output rows are stored into every
  rank's gather buffer (the all-gather) and signalled with one epoch flag per source rank;
* ``cb_gemm_bf16_tp``   — the tcgen05 GEMM (a) consuming such a buffer panel by panel, waiting on the
  source's flag only when it reaches that panel (own panel first), and/or (b) storing each output tile
  into the staging buffer of the rank that owns those rows (the reduce-scatter's transfer);
* ``cb_reduce_partials`` — sum of the W staged partials (+ residual) on the owner.

Buffer discipline (why nothing is overwritten while a peer still reads it): the gather buffers
alternate between two channels — channel 0 for normalised activations entering a column-parallel
GEMM, channel 1 for gradients entering a row-parallel GEMM's backward — and every reduce-scatter ends
with a group barrier.  A rank can only push into channel c again after a dependency chain through
flags or a barrier that the slowest reader of the previous contents has already passed.

Every device-side wait is bounded (``TPState.wait_budget_us``); on expiry the kernel records error 201
in the status word and all later kernels return immediately (``ops._ext.check_status`` raises).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from ..ops import _ext
from . import symm

_P, _I, _L, _F, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_ulonglong
_PROTOS = {
    "cb_gemm_bf16_tp": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _I, _P, _P, _I, _P, _I, _I, _I, _U, _P, _P],
    "cb_gemm2sm_bf16_tp": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _P, _P, _I, _P, _I, _I, _I, _U, _P, _P],
    "cb_rmsnorm_push": [_P, _P, _P, _P, _I, _I, _I, _I, _L, _F, _F, _P, _P, _P, _P, _P],
    "cb_reduce_partials": [_P, _P, _P, _I, _L, _P, _P],
    "cb_vp_combine": [_P, _I, _I, _P, _P, _P, _P],
}
_BOUND = False


def _lib():
    global _BOUND
    lib = symm._lib()
    if not _BOUND:
        for name, args in _PROTOS.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int
        _BOUND = True
    return lib


class FusedTP:
    """Symmetric buffers and launch helpers for one tensor-parallel group."""

    PANEL_ALIGN = 128          # rows per rank must be a multiple of the GEMM's M tile

    def __init__(self, tp, tokens: int, hidden: int, device):
        if not symm.peer_access_available(tp.group):
            raise RuntimeError("peer access between the local GPUs is not available")
        self.tp = tp
        self.rank, self.world = tp.rank, tp.world
        self.device = torch.device(device)
        self.ctx = symm.SymmetricContext(tp.group, tp.wait_budget_us)
        self.wait_ns = int(tp.wait_budget_us) * 1000
        self.status = self.ctx.status
        self.cap_elems = 0
        self.cap_tokens = 0
        self.flags = [symm.SymmetricBuffer(16, torch.int64, tp.group) for _ in range(2)]
        self.epoch = [torch.zeros(1, dtype=torch.int64, device=self.device) for _ in range(2)]
        self.done_ctr = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.xf = [None, None]
        self.stage = None
        self.ex = None
        # CTA-pair kernels for the two fused GEMMs where the shape fits their tiles (rows per rank a multiple of
        # 256 for the panel wait, N a multiple of 64 for the push epilogue); ``pair_gemm = False`` keeps the
        # single-CTA kernel everywhere
        self.pair_gemm = bool(getattr(tp, "pair_gemm", True))
        self.pair_min_dim = int(getattr(tp, "pair_min_dim", 1024))      # below this K and N the single-CTA kernel is quicker
        self.ensure(tokens, hidden)

    def ensure(self, tokens: int, hidden: int) -> None:
        need = tokens * hidden
        if need > self.cap_elems:
            # (re)allocation is collective: every rank reaches this with the same sizes
            for b in [*self.xf, self.stage]:
                if b is not None:
                    b.close()
            self.xf = [symm.SymmetricBuffer(need, torch.bfloat16, self.tp.group, zero=False) for _ in range(2)]
            self.stage = symm.SymmetricBuffer(need, torch.bfloat16, self.tp.group, zero=False)
            self.cap_elems = need
        if tokens > self.cap_tokens:
            if self.ex is not None:
                self.ex.close()
            self.ex = symm.SymmetricBuffer(2 * tokens, torch.float32, self.tp.group, zero=False)
            self.cap_tokens = tokens

    # ------------------------------------------------------------------------------------------ primitives
    def push(self, x: torch.Tensor, norm_w: Optional[torch.Tensor], eps: float, offset: float, channel: int
             ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """All-gather ``x`` (after RMSNorm when ``norm_w`` is given) into channel ``channel``; returns the
        local ``[T, N]`` gather buffer (complete only panel by panel, see the flags) and ``rstd``."""
        rows, N = x.shape
        if rows % self.PANEL_ALIGN:
            raise ValueError(f"rows per rank ({rows}) must be a multiple of {self.PANEL_ALIGN} for the fused path")
        self.ensure(rows * self.world, N)
        x = x.contiguous()
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if norm_w is not None else None
        buf = self.xf[channel]
        code = _lib().cb_rmsnorm_push(x.data_ptr(), _ext.ptr(norm_w), buf.ptrs, self.flags[channel].ptrs, self.world,
                                      self.rank, rows, N, N, float(eps), float(offset), _ext.ptr(rstd),
                                      self.epoch[channel].data_ptr(), self.done_ctr.data_ptr(), self.status.data_ptr(),
                                      _ext.stream_ptr())
        _ext.check(code, "rmsnorm_push")
        return buf.local[: rows * self.world * N].view(rows * self.world, N), rstd

    def gemm_wait(self, a_full: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], channel: int,
                  b_mn: bool = False) -> torch.Tensor:
        """``a_full @ op(b)ᵀ`` where ``a_full`` is the gather buffer of ``channel`` (waits per panel)."""
        M, K = a_full.shape
        N = b.shape[1] if b_mn else b.shape[0]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a_full.device)
        if self.pair_gemm and (M // self.world) % 256 == 0 and max(K, N) >= self.pair_min_dim:
            code = _lib().cb_gemm2sm_bf16_tp(a_full.data_ptr(), b.data_ptr(), out.data_ptr(), _ext.ptr(bias), M, N, K,
                                             a_full.stride(0), b.stride(0), out.stride(0), int(b_mn),
                                             self.flags[channel].local.data_ptr(), self.epoch[channel].data_ptr(),
                                             M // self.world, None, 0, self.world, self.rank, self.wait_ns,
                                             self.status.data_ptr(), _ext.stream_ptr())
            if code != -5:
                _ext.check(code, "gemm2sm_tp(wait)")
                _ext.count_launch()
                return out
        code = _lib().cb_gemm_bf16_tp(a_full.data_ptr(), b.data_ptr(), out.data_ptr(), _ext.ptr(bias), M, N, K,
                                      a_full.stride(0), b.stride(0), out.stride(0), 0, int(b_mn), 0,
                                      self.flags[channel].local.data_ptr(), self.epoch[channel].data_ptr(),
                                      M // self.world, None, 0, self.world, self.rank, self.wait_ns,
                                      self.status.data_ptr(), _ext.stream_ptr())
        _ext.check(code, "gemm_tp(wait)")
        return out

    def gemm_push_reduce(self, a: torch.Tensor, b: torch.Tensor, residual: Optional[torch.Tensor], b_mn: bool = False
                         ) -> torch.Tensor:
        """Reduce-scatter of ``a @ op(b)ᵀ`` over the group: returns my ``[T/W, N]`` rows of the sum (+ residual)."""
        M, K = a.shape
        N = b.shape[1] if b_mn else b.shape[0]
        rows = M // self.world
        if M % self.world or rows % self.PANEL_ALIGN:
            raise ValueError(f"rows per rank ({rows}) must be a multiple of {self.PANEL_ALIGN} for the fused path")
        self.ensure(M, N)
        a = a.contiguous() if a.stride(1) != 1 else a
        # owner o receives my tile rows at stage_o[my_rank][row - o * rows]: pre-offset so the global row indexes it
        ptrs = (ctypes.c_ulonglong * self.world)()
        for o in range(self.world):
            off_rows = self.rank * rows - o * rows
            ptrs[o] = (self.stage.ptrs[o] + off_rows * N * 2) & 0xFFFFFFFFFFFFFFFF
        code = -5
        if self.pair_gemm and N % 64 == 0 and max(K, N) >= self.pair_min_dim:
            code = _lib().cb_gemm2sm_bf16_tp(a.data_ptr(), b.data_ptr(), None, None, M, N, K, a.stride(0), b.stride(0), N,
                                             int(b_mn), None, None, 0, ptrs, rows, self.world, self.rank, self.wait_ns,
                                             self.status.data_ptr(), _ext.stream_ptr())
            if code != -5:
                _ext.count_launch()
        if code == -5:
            code = _lib().cb_gemm_bf16_tp(a.data_ptr(), b.data_ptr(), None, None, M, N, K, a.stride(0), b.stride(0), N, 0,
                                          int(b_mn), 0, None, None, 0, ptrs, rows, self.world, self.rank, self.wait_ns,
                                          self.status.data_ptr(), _ext.stream_ptr())
        _ext.check(code, "gemm_tp(push)")
        self.ctx.barrier()                                   # all ranks' tiles have landed in my staging buffer
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=a.device)
        code = _lib().cb_reduce_partials(self.stage.local.data_ptr(), _ext.ptr(residual), out.data_ptr(), self.world,
                                         rows * N, self.status.data_ptr(), _ext.stream_ptr())
        _ext.check(code, "reduce_partials")
        return out

    def combine_lse_tgt(self, lse_local: torch.Tensor, tgt_local: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        T = lse_local.numel()
        self.ensure(T, 0)
        mine = self.ex.local[: 2 * T].view(2, T)
        mine[0].copy_(lse_local)
        mine[1].copy_(tgt_local)
        self.ctx.barrier()
        lse, tgt = torch.empty_like(lse_local), torch.empty_like(tgt_local)
        code = _lib().cb_vp_combine(self.ex.ptrs, self.world, T, lse.data_ptr(), tgt.data_ptr(), self.status.data_ptr(),
                                    _ext.stream_ptr())
        _ext.check(code, "vp_combine")
        self.ctx.barrier()                                   # nobody refills its buffer while a peer still reads it
        return lse, tgt

    # ------------------------------------------------------------------------------------------ autograd ops
    def norm_gather_linear(self, x, norm_w, eps, offset, weight, bias):
        return _NormGatherLinear.apply(x, norm_w, weight, bias, self, float(eps), float(offset))

    def norm_gather(self, x, norm_w, eps, offset):
        return _NormGather.apply(x, norm_w, self, float(eps), float(offset))

    def linear_scatter_add(self, a, weight, x):
        return _LinearScatterAdd.apply(a, weight, x, self)


def _rmsnorm_bwd(dh: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor, offset: float):
    L = _ext.lib()
    M, N = x.shape
    part = torch.empty(L.cb_rmsnorm_bwd_blocks(M, N) * N, dtype=torch.float32, device=x.device)
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    _ext.check(L.cb_rmsnorm_bwd(dh.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(),
                                dw.data_ptr(), part.data_ptr(), M, N, offset, 0, _ext.stream_ptr()), "rmsnorm_bwd")
    return dx, dw


class _NormGatherLinear(torch.autograd.Function):
    """``y[T, N_shard] = all_gather(rmsnorm(x)) @ Wᵀ + b`` with the gather overlapped panel by panel."""

    @staticmethod
    def forward(ctx, x, norm_w, weight, bias, ft: FusedTP, eps, offset):
        x = x.contiguous()
        hf, rstd = ft.push(x, norm_w, eps, offset, 0)
        y = ft.gemm_wait(hf, weight, bias, 0)
        ctx.save_for_backward(x, norm_w, weight, rstd)
        ctx.ft, ctx.cfg, ctx.has_bias = ft, (eps, offset), bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        from .. import ops
        x, norm_w, weight, rstd = ctx.saved_tensors
        ft: FusedTP = ctx.ft
        eps, offset = ctx.cfg
        dy = dy.contiguous()
        hf, _ = ft.push(x, norm_w, eps, offset, 0)                         # re-gather the normalised activations
        dh = ft.gemm_push_reduce(dy, weight, None, b_mn=True)               # my rows of sum_r dy_r @ W_r (barrier inside)
        dx, dnw = _rmsnorm_bwd(dh, x, norm_w, rstd, offset)
        dw = ops.gemm(dy, hf, a_mn=True, b_mn=True)                         # dyᵀ @ hf; every panel has landed by now
        db = ops.colsum(dy) if ctx.has_bias else None
        return dx, dnw, dw, db, None, None, None


class _NormGather(torch.autograd.Function):
    """``all_gather(rmsnorm(x))`` as a complete tensor (used in front of the vocab-parallel loss)."""

    @staticmethod
    def forward(ctx, x, norm_w, ft: FusedTP, eps, offset):
        x = x.contiguous()
        hf, rstd = ft.push(x, norm_w, eps, offset, 0)
        ft.ctx.barrier()                                                    # all panels are in place
        ctx.save_for_backward(x, norm_w, rstd)
        ctx.ft, ctx.offset = ft, offset
        return hf.clone()

    @staticmethod
    def backward(ctx, dhf):
        x, norm_w, rstd = ctx.saved_tensors
        ft: FusedTP = ctx.ft
        rows, N = x.shape
        # reduce-scatter by pull: publish my partial gradient, then sum my rows over all ranks' copies
        W = ft.world
        mine = ft.xf[1].local[: W * rows * N].view(W * rows, N)
        mine.copy_(dhf)
        ft.ctx.barrier()
        ptrs = (ctypes.c_ulonglong * W)(*[ft.xf[1].ptrs[r] + ft.rank * rows * N * 2 for r in range(W)])
        dh = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
        _ext.check(symm._lib().cb_allreduce_pull(ptrs, W, rows * N, 1.0, dh.data_ptr(), ft.status.data_ptr(),
                                                 _ext.stream_ptr()), "allreduce_pull")
        ft.ctx.barrier()                                                    # channel 1 may be refilled from here on
        dx, dnw = _rmsnorm_bwd(dh, x, norm_w, rstd, ctx.offset)
        return dx, dnw, None, None, None


class _LinearScatterAdd(torch.autograd.Function):
    """``x + reduce_scatter(a @ Wᵀ)`` — the row-parallel GEMM whose epilogue stores each tile at its owner."""

    @staticmethod
    def forward(ctx, a, weight, x, ft: FusedTP):
        out = ft.gemm_push_reduce(a, weight, x.contiguous())
        ctx.save_for_backward(a, weight)
        ctx.ft = ft
        return out

    @staticmethod
    def backward(ctx, dout):
        from .. import ops
        a, weight = ctx.saved_tensors
        ft: FusedTP = ctx.ft
        dout = dout.contiguous()
        df, _ = ft.push(dout, None, 0.0, 0.0, 1)                             # all-gather of the output gradient
        da = ft.gemm_wait(df, weight, None, 1, b_mn=True)                    # dA = dY_full @ W   (waits per panel)
        dw = ops.gemm(df, a, a_mn=True, b_mn=True)                           # dW = dY_fullᵀ @ A  (after da: all panels in)
        return da, dw, dout, None
