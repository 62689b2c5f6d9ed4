"""Selective activation checkpointing.

Reference: chronicals/training/gradient_checkpointing.py:44-241
``GradientCheckpointer`` (sqrt(n) layer selection), :244-310 wrappers, :313-373
``apply_gradient_checkpointing`` (marks layers), :376-462 memory estimate.  The
decoder layers of this framework honour the ``_use_checkpoint`` mark by
recomputing their body in the backward pass.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as _checkpoint


def select_checkpoint_layers(num_layers: int, checkpoint_ratio: float = 0.177) -> List[int]:
    """Evenly spaced layer indices.  ``ratio <= 0`` → none, ``>= 1`` → all; the default
    0.177 ≈ 1/sqrt(32) reproduces the sqrt(n) rule for 32-layer models."""
    if checkpoint_ratio <= 0 or num_layers <= 0:
        return []
    if checkpoint_ratio >= 1:
        return list(range(num_layers))
    k = max(1, int(round(num_layers * checkpoint_ratio)))
    return sorted({min(num_layers - 1, int((i + 0.5) * num_layers / k)) for i in range(k)})


class GradientCheckpointer:
    def __init__(self, num_layers: int, checkpoint_ratio: float = 0.177, use_reentrant: bool = False,
                 use_activation_offloading: bool = False, offload_config: Optional[Any] = None):
        self.num_layers = num_layers
        self.checkpoint_ratio = checkpoint_ratio
        self.use_reentrant = use_reentrant
        self.use_activation_offloading = use_activation_offloading
        self.offload_config = offload_config
        self.checkpoint_layers = set(select_checkpoint_layers(num_layers, checkpoint_ratio))

    def should_checkpoint(self, layer_idx: int) -> bool:
        return layer_idx in self.checkpoint_layers

    def checkpoint(self, fn: Callable, *args, layer_idx: Optional[int] = None, **kwargs):
        if layer_idx is not None and not self.should_checkpoint(layer_idx):
            return fn(*args, **kwargs)
        if self.use_activation_offloading:
            from .async_activation_offload import OffloadActivations
            with OffloadActivations(self.offload_config):
                return _checkpoint(fn, *args, use_reentrant=self.use_reentrant, **kwargs)
        return _checkpoint(fn, *args, use_reentrant=self.use_reentrant, **kwargs)

    def memory_savings(self, activation_bytes_per_layer: float) -> Dict[str, float]:
        full = activation_bytes_per_layer * self.num_layers
        kept = activation_bytes_per_layer * (self.num_layers - len(self.checkpoint_layers))
        return {"full_gb": full / 2**30, "with_checkpointing_gb": kept / 2**30,
                "saved_fraction": 1 - kept / full if full else 0.0}


class CheckpointedLayer(nn.Module):
    """Wraps any module so its forward is recomputed in the backward pass."""

    def __init__(self, layer: nn.Module, use_reentrant: bool = False):
        super().__init__()
        self.layer = layer
        self.use_reentrant = use_reentrant

    def forward(self, *args, **kwargs):
        if self.training and torch.is_grad_enabled():
            return _checkpoint(self.layer, *args, use_reentrant=self.use_reentrant, **kwargs)
        return self.layer(*args, **kwargs)


class SelectiveCheckpointing:
    """Context-free helper: ``wrap(model.layers)`` replaces the selected layers by ``CheckpointedLayer``."""

    def __init__(self, checkpoint_ratio: float = 0.177):
        self.checkpoint_ratio = checkpoint_ratio

    def wrap(self, layers: nn.ModuleList) -> nn.ModuleList:
        chosen = set(select_checkpoint_layers(len(layers), self.checkpoint_ratio))
        for i in range(len(layers)):
            if i in chosen and not isinstance(layers[i], CheckpointedLayer):
                layers[i] = CheckpointedLayer(layers[i])
        return layers


def _find_layers(model: nn.Module, layers_attr: str = "layers") -> Optional[nn.ModuleList]:
    for cand in (model, getattr(model, "model", None), getattr(getattr(model, "model", None), "model", None),
                 getattr(model, "base_model", None)):
        if cand is not None and isinstance(getattr(cand, layers_attr, None), nn.ModuleList):
            return getattr(cand, layers_attr)
    for m in model.modules():
        if isinstance(getattr(m, layers_attr, None), nn.ModuleList):
            return getattr(m, layers_attr)
    return None


def apply_gradient_checkpointing(model: nn.Module, checkpoint_ratio: float = 0.177, layers_attr: str = "layers",
                                 wrap_foreign_layers: bool = True) -> List[int]:
    """Mark (native layers) or wrap (foreign layers) the selected decoder layers; returns their indices."""
    layers = _find_layers(model, layers_attr)
    if layers is None:
        return []
    chosen = select_checkpoint_layers(len(layers), checkpoint_ratio)
    for i, layer in enumerate(layers):
        on = i in chosen
        if hasattr(layer, "_use_checkpoint"):
            layer._use_checkpoint = on
        elif on and wrap_foreign_layers and not isinstance(layer, CheckpointedLayer):
            layers[i] = CheckpointedLayer(layer)
    return chosen


def enable_gradient_checkpointing(model: nn.Module, checkpoint_ratio: float = 1.0) -> List[int]:
    """README-documented name."""
    return apply_gradient_checkpointing(model, checkpoint_ratio)


def estimate_activation_memory(hidden_size: int, intermediate_size: int, num_layers: int, num_heads: int,
                               num_kv_heads: int, head_dim: int, tokens: int, bytes_per_el: int = 2,
                               checkpoint_ratio: float = 0.0) -> Dict[str, float]:
    """Bytes of activations this framework's decoder saves for backward, per micro-batch.

    Per layer and token: block input h (H), normed x (H), QKV ((hq+2hk)·d), attention out (hq·d),
    post-attention h (H), normed (H), gate|up (2I), SwiGLU out (I), plus fp32 rstd ×2 and LSE (hq)."""
    q, kv = num_heads * head_dim, num_kv_heads * head_dim
    per_tok = (4 * hidden_size + (q + 2 * kv) + q + 3 * intermediate_size) * bytes_per_el + (2 + num_heads) * 4
    per_layer = per_tok * tokens
    ck = len(select_checkpoint_layers(num_layers, checkpoint_ratio))
    kept = per_layer * (num_layers - ck) + ck * hidden_size * tokens * bytes_per_el
    return {"per_layer_gb": per_layer / 2**30, "total_gb": per_layer * num_layers / 2**30,
            "with_checkpointing_gb": kept / 2**30, "checkpointed_layers": float(ck)}
