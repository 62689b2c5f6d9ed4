"""Kernel front-ends.  ``from chronicals_b200.kernels import fused_rmsnorm, fused_swiglu,
fused_cross_entropy, fused_qk_rope`` are the README-documented names."""
from .cut_cross_entropy import CutCrossEntropyLoss, cut_cross_entropy, get_optimal_chunk_size
from .fused_kernels import (FusedRMSNorm, FusedSwiGLU, fused_cross_entropy, fused_geglu, fused_gqa_attention,
                            fused_linear_cross_entropy, fused_qk_rope, fused_rmsnorm, fused_rope, fused_swiglu,
                            precompute_rope_cache, rmsnorm)

__all__ = ["CutCrossEntropyLoss", "cut_cross_entropy", "get_optimal_chunk_size", "FusedRMSNorm", "FusedSwiGLU",
           "fused_cross_entropy", "fused_geglu", "fused_gqa_attention", "fused_linear_cross_entropy", "fused_qk_rope",
           "fused_rmsnorm", "fused_rope", "fused_swiglu", "precompute_rope_cache", "rmsnorm"]
