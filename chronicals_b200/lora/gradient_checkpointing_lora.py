"""Activation checkpointing tuned for adapter training.

Reference: chronicals/lora/gradient_checkpointing_lora.py:95-142 ``LoRACheckpointConfig`` (modes
``standard`` / ``lora_fa`` / ``unsloth``), :149-286 helpers, :293-593 ``LoRAGradientCheckpointer``
(sqrt(n) layer selection, frozen layers without adapters are skipped), :600-653
``UnslothCheckpointing``, :660-759 ``apply_lora_checkpointing`` and the savings estimate.

With a frozen base only the adapters need weight gradients, but activation gradients still flow
through every layer, so a layer's inputs must be kept or recomputed.  Layers are selected evenly
(sqrt(n) by default); ``offload`` additionally parks the kept layer inputs in pinned host memory.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from ..training.gradient_checkpointing import _find_layers, apply_gradient_checkpointing, select_checkpoint_layers


@dataclass
class LoRACheckpointConfig:
    mode: str = "standard"               # standard | lora_fa | unsloth
    checkpoint_ratio: Optional[float] = None     # None → sqrt(n) layers
    skip_frozen_layers: bool = True
    offload: bool = False                # "unsloth" mode turns this on
    use_reentrant: bool = False

    def __post_init__(self):
        if self.mode not in ("standard", "lora_fa", "unsloth"):
            raise ValueError(f"unknown checkpoint mode {self.mode!r}")
        if self.mode == "unsloth":
            self.offload = True


def layer_has_trainable_params(layer: nn.Module) -> bool:
    return any(p.requires_grad for p in layer.parameters())


def sqrt_n_ratio(num_layers: int) -> float:
    return min(1.0, math.sqrt(max(1, num_layers)) / max(1, num_layers))


class LoRAGradientCheckpointer:
    def __init__(self, model: nn.Module, config: Optional[LoRACheckpointConfig] = None, layers_attr: str = "layers"):
        self.model = model
        self.config = config or LoRACheckpointConfig()
        self.layers = _find_layers(model, layers_attr)
        self.selected: List[int] = []

    def select_layers(self) -> List[int]:
        if self.layers is None:
            return []
        n = len(self.layers)
        ratio = self.config.checkpoint_ratio if self.config.checkpoint_ratio is not None else sqrt_n_ratio(n)
        chosen = select_checkpoint_layers(n, ratio)
        if self.config.skip_frozen_layers:
            # a frozen layer without adapters still needs its input for dX; recomputing it is cheap only
            # if the layer is cheap, so it is never preferred over a layer that has adapters
            with_adapters = [i for i in range(n) if layer_has_trainable_params(self.layers[i])]
            if with_adapters and len(with_adapters) < n:
                chosen = [i for i in chosen if i in with_adapters] or chosen
        return chosen

    def apply(self) -> List[int]:
        self.selected = self.select_layers()
        if self.layers is None:
            return []
        for i, layer in enumerate(self.layers):
            if hasattr(layer, "_use_checkpoint"):
                layer._use_checkpoint = i in self.selected
        if not any(hasattr(l, "_use_checkpoint") for l in self.layers):
            ratio = len(self.selected) / max(1, len(self.layers))
            apply_gradient_checkpointing(self.model, ratio)
        if self.config.offload:
            self.model._activation_offload = True
        return self.selected

    def remove(self) -> None:
        if self.layers is not None:
            for layer in self.layers:
                if hasattr(layer, "_use_checkpoint"):
                    layer._use_checkpoint = False


class UnslothCheckpointing(LoRAGradientCheckpointer):
    """Checkpoint every layer and keep the layer inputs in pinned host memory."""

    def __init__(self, model: nn.Module, layers_attr: str = "layers"):
        super().__init__(model, LoRACheckpointConfig(mode="unsloth", checkpoint_ratio=1.0), layers_attr)


def apply_lora_checkpointing(model: nn.Module, mode: str = "standard", checkpoint_ratio: Optional[float] = None
                             ) -> List[int]:
    return LoRAGradientCheckpointer(model, LoRACheckpointConfig(mode=mode, checkpoint_ratio=checkpoint_ratio)).apply()


def estimate_checkpointing_savings(num_layers: int, activation_gb_per_layer: float, checkpoint_ratio: Optional[float] = None
                                   ) -> Dict[str, float]:
    ratio = checkpoint_ratio if checkpoint_ratio is not None else sqrt_n_ratio(num_layers)
    k = len(select_checkpoint_layers(num_layers, ratio))
    full = num_layers * activation_gb_per_layer
    kept = (num_layers - k) * activation_gb_per_layer
    return {"checkpointed_layers": float(k), "full_gb": full, "with_checkpointing_gb": kept,
            "saved_gb": full - kept, "recompute_overhead": k / max(1, num_layers) / 3.0}


class SelectiveCheckpoint:
    """Callable that runs ``function(*args, **kwargs)`` under activation checkpointing according to a
    :class:`LoRACheckpointConfig` (reference gradient_checkpointing_lora.py:149-300): ``standard`` and ``lora_fa``
    recompute the block in backward, ``unsloth`` additionally parks the saved inputs in pinned host memory.
    With ``enabled=False`` the function is simply called."""

    def __init__(self, config: Optional[LoRACheckpointConfig] = None, enabled: bool = True):
        self.config = config or LoRACheckpointConfig()
        self.enabled = enabled
        self._offload = None

    def __call__(self, function, *args, use_reentrant: Optional[bool] = None, **kwargs):
        if not self.enabled:
            return function(*args, **kwargs)
        reentrant = self.config.use_reentrant if use_reentrant is None else use_reentrant
        if self.config.offload:
            if self._offload is None:
                from ..training.async_activation_offload import CheckpointWithOffload
                self._offload = CheckpointWithOffload(use_reentrant=reentrant)
            return self._offload(function, *args, **kwargs)
        from torch.utils.checkpoint import checkpoint
        return checkpoint(function, *args, use_reentrant=reentrant, **kwargs)
