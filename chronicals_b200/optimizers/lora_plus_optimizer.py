"""LoRA+ : different learning rates for the A and B adapter matrices.

API follows the reference (chronicals/optimizers/lora_plus_optimizer.py:55-189
``LoRAPlusParameterGroups``, :196-429 ``LoRAPlusAdamW`` = ``LoRAPlusOptimizer``,
:435-546 helpers): parameters are classified by name into ``lora_A`` / ``lora_B``
/ ``other``; the B group trains at ``lr * lr_ratio`` (16 by default), adapter
weight decay is separate.  The optimizer itself is this framework's
multi-tensor ``FusedAdamW`` — per-group rates live in its device-side group
table, so the A/B split costs nothing at step time.
"""
from __future__ import annotations

import re
from typing import Any, Dict, Iterable, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from .fused_adamw import FusedAdamW

# PEFT names ("…lora_A.default.weight"), this framework's ("…lora_A.q_proj"), and bare conventions
_A_PATTERNS = [r"(^|\.)lora_A($|\.)", r"lora_A_", r"\.A$", r"_A$", r"lora_down"]
_B_PATTERNS = [r"(^|\.)lora_B($|\.)", r"lora_B_", r"\.B$", r"_B$", r"lora_up"]


class LoRAPlusParameterGroups:
    """Splits trainable parameters into A / B / other groups by name."""

    def __init__(self, a_patterns: Optional[List[str]] = None, b_patterns: Optional[List[str]] = None):
        self.a_re = [re.compile(p) for p in (a_patterns or _A_PATTERNS)]
        self.b_re = [re.compile(p) for p in (b_patterns or _B_PATTERNS)]

    def classify(self, name: str) -> str:
        if any(r.search(name) for r in self.a_re):
            return "lora_A"
        if any(r.search(name) for r in self.b_re):
            return "lora_B"
        return "other"

    def split(self, named_params: Iterable[Tuple[str, nn.Parameter]]) -> Dict[str, List[nn.Parameter]]:
        out: Dict[str, List[nn.Parameter]] = {"lora_A": [], "lora_B": [], "other": []}
        for name, p in named_params:
            if p.requires_grad:
                out[self.classify(name)].append(p)
        return out

    def get_param_groups(self, model_or_named, base_lr: float = 1e-4, lr_ratio: float = 16.0,
                         weight_decay: float = 0.0, weight_decay_lora: Optional[float] = None) -> List[Dict[str, Any]]:
        if lr_ratio < 1.0:
            raise ValueError(f"lr_ratio must be >= 1 (got {lr_ratio}): LoRA+ trains B faster than A")
        named = model_or_named.named_parameters() if hasattr(model_or_named, "named_parameters") else model_or_named
        parts = self.split(named)
        wd_lora = weight_decay if weight_decay_lora is None else weight_decay_lora
        groups = []
        if parts["lora_A"]:
            groups.append({"params": parts["lora_A"], "lr": base_lr, "weight_decay": wd_lora,
                           "name": "lora_A", "_group_name": "lora_A"})
        if parts["lora_B"]:
            groups.append({"params": parts["lora_B"], "lr": base_lr * lr_ratio, "weight_decay": wd_lora,
                           "name": "lora_B", "_group_name": "lora_B"})
        if parts["other"]:
            groups.append({"params": parts["other"], "lr": base_lr, "weight_decay": weight_decay,
                           "name": "other", "_group_name": "other"})
        return groups


class LoRAPlusAdamW(FusedAdamW):
    """AdamW whose ``lora_B`` group runs at ``lr * lr_ratio``.

    ``params`` may be a module (parameters are classified by name), an iterable of
    ``(name, parameter)`` pairs, ready-made groups, or plain parameters (then all share ``lr``).
    """

    def __init__(self, params, lr: float = 1e-4, lr_ratio: float = 16.0, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, weight_decay_lora: float = 0.0, auto_detect_lora: bool = True,
                 max_grad_norm: float = 0.0, **kw):
        if lr_ratio < 1.0:
            raise ValueError(f"lr_ratio must be >= 1 (got {lr_ratio})")
        self.lr_ratio = lr_ratio
        self.base_lr = lr
        groups: Any
        if isinstance(params, nn.Module):
            groups = LoRAPlusParameterGroups().get_param_groups(params, lr, lr_ratio, weight_decay, weight_decay_lora) \
                if auto_detect_lora else [p for p in params.parameters() if p.requires_grad]
        else:
            items = list(params)
            if items and isinstance(items[0], tuple) and isinstance(items[0][0], str):
                groups = LoRAPlusParameterGroups().get_param_groups(items, lr, lr_ratio, weight_decay, weight_decay_lora)
            else:
                groups = items
        if not groups:
            raise ValueError("no trainable parameters")
        super().__init__(groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         max_grad_norm=max_grad_norm, **kw)

    def get_lr_by_group(self) -> Dict[str, float]:
        return {g.get("name", f"group{i}"): g["lr"] for i, g in enumerate(self.param_groups)}

    def scale_lora_lr(self, factor: float) -> None:
        for g in self.param_groups:
            if g.get("name") in ("lora_A", "lora_B"):
                g["lr"] *= factor
                if "initial_lr" in g:
                    g["initial_lr"] *= factor


LoRAPlusOptimizer = LoRAPlusAdamW


def get_lora_plus_param_groups(model: nn.Module, base_lr: float = 1e-4, lr_ratio: float = 16.0,
                               weight_decay: float = 0.0, weight_decay_lora: Optional[float] = None):
    return LoRAPlusParameterGroups().get_param_groups(model, base_lr, lr_ratio, weight_decay, weight_decay_lora)


def create_lora_plus_optimizer(model: nn.Module, base_lr: float = 1e-4, lr_ratio: float = 16.0, betas=(0.9, 0.999),
                               eps: float = 1e-8, weight_decay: float = 0.0, optimizer_class=None,
                               max_grad_norm: float = 0.0, **kw):
    """LoRA+ groups on ``optimizer_class`` (default: the fused multi-tensor AdamW)."""
    groups = get_lora_plus_param_groups(model, base_lr, lr_ratio, weight_decay, kw.pop("weight_decay_lora", 0.0))
    if optimizer_class is None:
        return LoRAPlusAdamW(groups, lr=base_lr, lr_ratio=lr_ratio, betas=betas, eps=eps, weight_decay=weight_decay,
                             max_grad_norm=max_grad_norm, **kw)
    return optimizer_class(groups, lr=base_lr, betas=betas, eps=eps, **kw)


def wrap_optimizer_with_lora_plus(optimizer: torch.optim.Optimizer, model: nn.Module, lr_ratio: float = 16.0):
    """Re-group an existing optimizer's parameters in place so adapter B matrices get ``lr * lr_ratio``."""
    names = {id(p): n for n, p in model.named_parameters()}
    cls = LoRAPlusParameterGroups()
    new_groups = []
    for g in optimizer.param_groups:
        buckets: Dict[str, List[nn.Parameter]] = {"lora_A": [], "lora_B": [], "other": []}
        for p in g["params"]:
            buckets[cls.classify(names.get(id(p), ""))].append(p)
        for kind, ps in buckets.items():
            if not ps:
                continue
            ng = {k: v for k, v in g.items() if k != "params"}
            ng["params"] = ps
            ng["name"] = ng["_group_name"] = kind
            if kind == "lora_B":
                ng["lr"] = g["lr"] * lr_ratio
            new_groups.append(ng)
    optimizer.param_groups = new_groups
    return optimizer
