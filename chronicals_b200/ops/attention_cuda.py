"""autograd wrappers of the tcgen05 varlen attention kernels (``csrc/attention.cu``)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _ext


def _cu32(cu_seqlens: torch.Tensor) -> torch.Tensor:
    cu = cu_seqlens
    if cu.dtype != torch.int32:
        cu = cu.to(torch.int32)
    return cu.contiguous()


class _AttnPackedFn(torch.autograd.Function):
    """Attention on a fused ``[T, (hq + 2 hk) * D]`` QKV buffer; the gradient comes back as one
    fused buffer too, so autograd never has to stitch three slice gradients together."""

    @staticmethod
    def forward(ctx, qkv, cu, hq, hk, d, scale):
        T, ld = qkv.shape[0], qkv.stride(0)
        nq, nk = hq * d, hk * d
        o = torch.empty(T, nq, dtype=qkv.dtype, device=qkv.device)     # the kernel writes the zeros of the padding rows
        lse = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
        esz = qkv.element_size()
        code = _ext.lib().cb_attn_fwd(qkv.data_ptr(), qkv.data_ptr() + nq * esz, qkv.data_ptr() + (nq + nk) * esz,
                                      o.data_ptr(), lse.data_ptr(), cu.data_ptr(), cu.numel() - 1, T, hq, hk, d,
                                      ld, ld, ld, nq, scale, _ext.status_buffer(qkv.device).data_ptr(),
                                      _ext.stream_ptr())
        _ext.check(code, "attn_fwd")
        ctx.save_for_backward(qkv, o, lse, cu)
        ctx.cfg = (hq, hk, d, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cu = ctx.saved_tensors
        hq, hk, d, scale = ctx.cfg
        T, ld = qkv.shape[0], qkv.stride(0)
        nq, nk = hq * d, hk * d
        if not do.is_contiguous():
            do = do.contiguous()
        dev = qkv.device
        # the kernels use 16-byte vector accesses on dq_acc / dk_acc / dv_acc: every region must start on a
        # 16-byte boundary whatever T is (T * nq and T * nk are multiples of 4 because D is 64 or 128)
        n_delta = (hq * T + 63) // 64 * 64
        # The accumulators are cleared by the entry point right before the kernel.  Keeping them between calls and
        # letting the finalize kernel write the zeros back (``scratch_is_zero``) was measured slower (forward +
        # backward 0.191 -> 0.229 ms on 8 x 1024 tokens, 1.53 -> 1.94 ms on the 7B shape): the clears leave the lines
        # in L2, where the TMA reduce-adds of dQ then land without fetching them from memory first.
        scratch = torch.empty(n_delta + T * nq + 2 * T * nk, dtype=torch.float32, device=dev)
        delta = scratch[:hq * T]
        dq_acc = scratch[n_delta: n_delta + T * nq]
        dk_part = scratch[n_delta + T * nq: n_delta + T * nq + T * nk]        # per kv head, accumulated by the kernel
        dv_part = scratch[n_delta + T * nq + T * nk:]
        dqkv = torch.empty(T, nq + 2 * nk, dtype=qkv.dtype, device=dev)
        esz = qkv.element_size()
        code = _ext.lib().cb_attn_bwd(qkv.data_ptr(), qkv.data_ptr() + nq * esz, qkv.data_ptr() + (nq + nk) * esz,
                                      o.data_ptr(), do.data_ptr(), lse.data_ptr(), cu.data_ptr(), cu.numel() - 1, T,
                                      hq, hk, d, ld, ld, ld, nq, do.stride(0), scale, delta.data_ptr(),
                                      dq_acc.data_ptr(), dk_part.data_ptr(), dv_part.data_ptr(), dqkv.data_ptr(),
                                      dqkv.stride(0), _ext.status_buffer(dev).data_ptr(), _ext.stream_ptr(), 0)
        _ext.check(code, "attn_bwd")
        return dqkv, None, None, None, None, None


def kernel_supports(t: torch.Tensor, d: int) -> bool:
    return (t.is_cuda and not _ext.reference_forced() and t.dtype == torch.bfloat16 and d in (64, 128) and _ext.available()
            and _ext.has_symbol("cb_attn_fwd"))


def attention_qkv_packed(qkv: torch.Tensor, cu_seqlens: torch.Tensor, num_q_heads: int, num_kv_heads: int,
                         head_dim: int, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Causal GQA attention over packed documents; ``qkv [T, (hq + 2 hk) * D]`` → ``[T, hq * D]``."""
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.stride(0) % 8 == 0
    return _AttnPackedFn.apply(qkv, _cu32(cu_seqlens), num_q_heads, num_kv_heads, head_dim, scale)


def attention_varlen_cuda(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                          max_seqlen: Optional[int], scale: float) -> torch.Tensor:
    """Separate q / k / v tensors: packed into one buffer (a copy) and run through the fused-buffer path."""
    T, hq, d = q.shape
    hk = k.shape[1]
    qkv = torch.cat((q.reshape(T, hq * d), k.reshape(T, hk * d), v.reshape(T, hk * d)), dim=1)
    return attention_qkv_packed(qkv, cu_seqlens, hq, hk, d, scale).view(T, hq, d)
