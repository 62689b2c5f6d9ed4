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


def fused_lora_forward(fl, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    base = ops.linear(x, fl.weight, fl.bias, residual)
    xd = F.dropout(x, fl.lora_dropout_p, training=True) if (fl.lora_dropout_p > 0 and fl.training) else x
    a_cat, b_big = lora_cat_matrices(fl)
    h = ops.linear(xd, a_cat)
    return ops.linear(h, b_big, None, base)


def lora_linear_reference(x, w, a, b, bias=None, scaling: float = 1.0):
    """Plain formula for tests: ``x W^T + b + scaling * (x A^T) B^T``."""
    y = F.linear(x, w, bias)
    return y + scaling * F.linear(F.linear(x, a), b)
