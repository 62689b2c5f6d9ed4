"""LoRA forward for fused projections.

``y = x W^T + b (+ residual) + sum_s scale_s * (drop(x) A_s^T) B_s^T`` placed in split ``s``'s
output columns.  All adapted splits of a fused projection share two extra GEMMs: one against the
row-concatenated ``A`` (``[sum r, in]``) and one against a block-diagonal ``B`` (``[out, sum r]``)
whose epilogue adds the base output, so q/k/v adapters cost the same launches as one.
The frozen base weight needs no weight-gradient GEMM.  Reference formula:
chronicals/kernels/fused_lora_kernels.py:166-302, :580-666.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import _ext


def lora_cat_matrices(fl):
    """(A_cat [R, in], B_big [out, R]) for the adapted splits of a ``FusedLinear``."""
    names = [s for s in fl.splits if s in fl.lora_A]
    a_cat = torch.cat([fl.lora_A[s] for s in names], dim=0) if len(names) > 1 else fl.lora_A[names[0]]
    R = a_cat.shape[0]
    sl = fl.split_slices()
    if len(fl.splits) == 1 and len(names) == 1:
        return a_cat, fl.lora_B[names[0]] * fl.lora_scaling[names[0]]
    b_big = torch.zeros(fl.out_features, R, dtype=a_cat.dtype, device=a_cat.device)
    r0 = 0
    for s in names:
        r = fl.lora_A[s].shape[0]
        b_big[sl[s], r0:r0 + r] = fl.lora_B[s] * fl.lora_scaling[s]
        r0 += r
    return a_cat, b_big


_USE_PACK = True      # False: assemble A_cat / B_big and split their gradients with PyTorch operators (for comparison)


class _FusedLoRAFn(torch.autograd.Function):
    """One autograd node for a frozen fused projection with per-split adapters (CUDA bf16 path).

    With ``A_cat = [A_1; A_2; …]`` (``[R, in]``) and the block-diagonal ``B_big = diag(s_1 B_1, s_2 B_2, …)``
    (``[out, R]``):

    forward : ``hs = x A_catᵀ``; ``y = x Wᵀ + hs B_bigᵀ + b (+ res)`` in one dual-product GEMM;
    backward: ``dhs = dy B_big``; ``dx = dy W + dhs A_cat`` (again one dual-product GEMM); ``dA_cat = dhsᵀ x`` and ``dB_big = dyᵀ hs`` by the
              split-K GEMM (skinny outputs, K = tokens); the frozen ``W`` gets no weight-gradient GEMM.
    ``ab`` is ``A_1, B_1, A_2, B_2, …`` in split order; ``meta`` carries the output slices and scalings.
    """

    @staticmethod
    def forward(ctx, x2, w, bias, res2, meta, *ab):
        slices, scalings, drop_p, bufs = meta
        As, Bs = ab[0::2], ab[1::2]
        ranks = [b.shape[1] for b in Bs]
        R = sum(ranks)
        n_in, n_out = w.shape[1], w.shape[0]
        packed = _pack_desc(bufs, slices, ranks, scalings, As, Bs)
        if packed is not None:
            # one launch builds A_cat (the A matrices stacked, unscaled) and the block-diagonal, scaled B_big
            a_cat = torch.empty(R, n_in, dtype=w.dtype, device=w.device)
            b_big = torch.empty(n_out, R, dtype=w.dtype, device=w.device)
            a_ptrs, b_ptrs, c_rank, c_row0, c_nrows, c_scale = packed
            code = _ext.lib().cb_lora_pack(a_ptrs, b_ptrs, c_rank, c_row0, c_nrows, c_scale, len(As), n_in, n_out,
                                           a_cat.data_ptr(), b_big.data_ptr(), _ext.stream_ptr())
            _ext.check(code, "lora_pack")
        else:
            # A_cat: one concatenation, unscaled.  B_big: the adapters' B matrices copied (one multi-tensor copy) onto
            # the diagonal blocks of a persistent zero matrix, times the per-column scaling vector - the scalings live
            # on the B side, so hs = x A_catᵀ needs no scaling pass and dA no rescaling.
            a_cat = torch.cat(As, dim=0) if len(As) > 1 else As[0]
            if ("b_zero" not in bufs or bufs["b_zero"].shape != (n_out, R) or bufs["b_zero"].device != w.device
                    or bufs.get("scalings") != tuple(scalings)):
                bufs["scalings"] = tuple(scalings)
                bufs["b_zero"] = torch.zeros(n_out, R, dtype=w.dtype, device=w.device)
                bufs["colscale"] = torch.cat([torch.full((r,), float(sc)) for r, sc in zip(ranks, scalings)]).to(
                    device=w.device, dtype=w.dtype)
                r0 = 0
                bufs["views"] = []
                for sl, r in zip(slices, ranks):
                    bufs["views"].append(bufs["b_zero"][sl, r0:r0 + r])
                    r0 += r
            torch._foreach_copy_(bufs["views"], [b.detach() for b in Bs])
            b_big = bufs["b_zero"] * bufs["colscale"]                 # [out, R], scaled; off-diagonal blocks stay zero
        # adapter-branch dropout (reference fused_lora_kernels.py:63-155 draws it inside its down-projection
        # kernel): the keep mask, scaled by 1 / (1 - p), multiplies the adapter's input only
        keep = None
        xa = x2
        if drop_p > 0.0:
            keep = (torch.rand_like(x2, dtype=torch.float32) >= drop_p).to(x2.dtype) * (1.0 / (1.0 - drop_p))
            xa = x2 * keep
        hs = ops.gemm(xa, a_cat)                                      # [T, R]
        # one kernel for  x Wᵀ + hs B_bigᵀ + b (+ res): the adapter's k-block follows the projection's in the
        # same accumulators, so the output is written once
        y = ops.gemm_dual(x2, w, hs, b_big, bias=bias, addend=res2)
        ctx.save_for_backward(x2, w, a_cat, hs, b_big, keep)
        ctx.meta = (slices, ranks, scalings, bias is not None, res2 is not None, packed)
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w, a_cat, hs, b_big, keep = ctx.saved_tensors
        slices, ranks, scalings, has_bias, has_res, packed = ctx.meta
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dhs = ops.gemm(dy2, b_big, b_mn=True)                               # [T, R], carries the scalings
        dx = None
        if ctx.needs_input_grad[0]:
            if keep is None:
                dx = ops.gemm_dual(dy2, w, dhs, a_cat, b_mn=True)           # dX = dY W + dhs A_cat, one kernel
            else:
                dx = ops.gemm(dy2, w, b_mn=True)
                dx.addcmul_(ops.gemm(dhs, a_cat, b_mn=True), keep)          # the adapter's share passes the same mask
        xa = x2 if keep is None else x2 * keep
        da32 = ops.gemm_splitk(dhs, xa, a_mn=True, b_mn=True)               # fp32 [R, in]
        db32 = ops.gemm_splitk(dy2, hs, a_mn=True, b_mn=True)               # fp32 [out, R]
        n_in = x2.shape[1]
        grads = []
        if packed is not None:
            # one launch rounds both to bf16, applies the scalings to the B blocks and lays the per-adapter gradients
            # out back to back in one buffer; the returned gradients are contiguous views of it
            _, _, c_rank, c_row0, c_nrows, c_scale = packed
            sizes = [(r * n_in, (sl.stop - sl.start) * r) for sl, r in zip(slices, ranks)]
            flat = torch.empty(sum(a + b for a, b in sizes), dtype=dy2.dtype, device=dy2.device)
            code = _ext.lib().cb_lora_unpack(c_rank, c_row0, c_nrows, c_scale, len(ranks), n_in, w.shape[0],
                                             da32.data_ptr(), db32.data_ptr(), flat.data_ptr(), _ext.stream_ptr())
            _ext.check(code, "lora_unpack")
            off = 0
            for (na, nb), sl, r in zip(sizes, slices, ranks):
                grads.append(flat[off:off + na].view(r, n_in))
                grads.append(flat[off + na:off + na + nb].view(sl.stop - sl.start, r))
                off += na + nb
        else:
            colscale = torch.cat([torch.full((r,), float(sc)) for r, sc in zip(ranks, scalings)]).to(dy2.device)
            da_cat = da32.to(dy2.dtype)
            db_big = (db32 * colscale).to(dy2.dtype)
            r0 = 0
            for sl, r in zip(slices, ranks):
                grads.append(da_cat[r0:r0 + r])                             # row blocks: contiguous views
                grads.append(db_big[sl, r0:r0 + r])
                r0 += r
        db = ops.colsum(dy2) if (has_bias and ctx.needs_input_grad[2]) else None
        dw = None
        if ctx.needs_input_grad[1]:                                         # base weight left trainable on purpose
            dw = ops.gemm(dy2, x2, a_mn=True, b_mn=True)
        return (dx, dw, db, dy2 if has_res else None, None, *grads)


def _pack_desc(bufs, slices, ranks, scalings, As, Bs):
    """ctypes arrays describing up to four adapters for ``cb_lora_pack`` / ``cb_lora_unpack`` (kept per projection,
    pointers refreshed every call), or None when the kernels do not apply."""
    import ctypes
    if not _USE_PACK or len(As) > 4 or not _ext.has_symbol("cb_lora_pack") or As[0].dtype != torch.bfloat16:
        return None
    if any(not a.is_contiguous() for a in As) or any(not b.is_contiguous() for b in Bs):
        return None
    d = bufs.get("pack")
    key = (tuple((sl.start, sl.stop) for sl in slices), tuple(ranks), tuple(scalings))
    if d is None or d[0] != key:
        n = len(As)
        c_rank = (ctypes.c_int * 4)(*ranks, *([0] * (4 - n)))
        c_row0 = (ctypes.c_int * 4)(*[sl.start for sl in slices], *([0] * (4 - n)))
        c_nrows = (ctypes.c_int * 4)(*[sl.stop - sl.start for sl in slices], *([0] * (4 - n)))
        c_scale = (ctypes.c_float * 4)(*[float(s) for s in scalings], *([0.0] * (4 - n)))
        d = (key, (ctypes.c_uint64 * 4)(), (ctypes.c_uint64 * 4)(), c_rank, c_row0, c_nrows, c_scale)
        bufs["pack"] = d
    for i, (a, b) in enumerate(zip(As, Bs)):
        d[1][i] = a.data_ptr()
        d[2][i] = b.data_ptr()
    return d[1:]


def _fused_path_ok(fl, x: torch.Tensor) -> bool:
    if not ops._fast(x, fl.weight):
        return False
    sl = fl.split_slices()
    for s in fl.lora_A:
        r = fl.lora_A[s].shape[0]
        if r % 8 or sl[s].start % 8 or (sl[s].stop - sl[s].start) % 8:
            return False
    return x.shape[-1] % 8 == 0


def fused_lora_forward(fl, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    names = [s for s in fl.splits if s in fl.lora_A]
    if names and _fused_path_ok(fl, x):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        res2 = residual.reshape(-1, fl.out_features) if residual is not None else None
        sl = fl.split_slices()
        drop_p = float(fl.lora_dropout_p) if (fl.training and fl.lora_dropout_p > 0) else 0.0
        if not hasattr(fl, "_lora_bufs"):
            fl._lora_bufs = {}                      # persistent block-diagonal B buffer and column scalings
        meta = ([sl[s] for s in names], [float(fl.lora_scaling[s]) for s in names], drop_p, fl._lora_bufs)
        ab = [t for s in names for t in (fl.lora_A[s], fl.lora_B[s])]
        y = _FusedLoRAFn.apply(x2, fl.weight, fl.bias, res2, meta, *ab)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], fl.out_features)
    base = ops.linear(x, fl.weight, fl.bias, residual)
    xd = F.dropout(x, fl.lora_dropout_p, training=True) if (fl.lora_dropout_p > 0 and fl.training) else x
    a_cat, b_big = lora_cat_matrices(fl)
    h = ops.linear(xd, a_cat)
    return ops.linear(h, b_big, None, base)


def lora_linear_reference(x, w, a, b, bias=None, scaling: float = 1.0):
    """Plain formula for tests: ``x W^T + b + scaling * (x A^T) B^T``."""
    y = F.linear(x, w, bias)
    return y + scaling * F.linear(F.linear(x, a), b)
