"""LoRA adapters: a wrapper for plain ``nn.Linear`` modules, a model-level helper
that also understands this framework's fused projections, and initialisers.

API follows the reference (chronicals/lora/lora_optimized.py:40-358
``OptimizedLoRALinear`` with kaiming / PiSSA / OLoRA / zeros init and
merge/unmerge, :365-490 ``LoRAModel``, :497-549 helpers).  Naming follows PEFT —
``lora_A [r, in]`` (Kaiming), ``lora_B [out, r]`` (zeros) — which is also what the
LoRA+ name patterns expect; the reference's own module has the two names
swapped, which would send the 16x learning rate to the wrong matrix.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops

DEFAULT_TARGET_MODULES = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


@dataclass
class LoRAConfig:
    """README-documented configuration object (``from chronicals.lora import LoRAConfig, apply_lora``)."""
    rank: int = 16
    alpha: float = 32.0
    dropout: float = 0.0
    target_modules: List[str] = field(default_factory=lambda: list(DEFAULT_TARGET_MODULES))
    init_method: str = "kaiming"
    use_lora_plus: bool = True
    lora_plus_ratio: float = 16.0

    # aliases used by PEFT-style code
    @property
    def r(self) -> int:
        return self.rank

    @property
    def lora_alpha(self) -> float:
        return self.alpha

    def to_peft_config(self) -> Dict[str, Any]:
        return {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": self.rank, "lora_alpha": self.alpha,
                "lora_dropout": self.dropout, "target_modules": list(self.target_modules), "bias": "none"}


def _randomized_svd(w: torch.Tensor, rank: int, n_iter: int = 4, oversample: int = 8
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Top-``rank`` SVD by randomized range finding (Halko et al.); exact for small matrices."""
    m, n = w.shape
    k = min(rank + oversample, min(m, n))
    if min(m, n) <= 4 * k:
        u, s, vh = torch.linalg.svd(w.float(), full_matrices=False)
        return u[:, :rank], s[:rank], vh[:rank]
    g = torch.randn(n, k, device=w.device, dtype=torch.float32)
    y = w.float() @ g
    for _ in range(n_iter):
        y, _ = torch.linalg.qr(y)
        y = w.float() @ (w.float().t() @ y)
    q, _ = torch.linalg.qr(y)
    b = q.t() @ w.float()
    ub, s, vh = torch.linalg.svd(b, full_matrices=False)
    return (q @ ub)[:, :rank], s[:rank], vh[:rank]


class OptimizedLoRALinear(nn.Module):
    """``y = base(x) + (alpha / r) * (drop(x) A^T) B^T`` around a frozen ``nn.Linear``.

    The low-rank path is evaluated in the cheap bracketing (rank-sized intermediate first)."""

    def __init__(self, base_layer: nn.Linear, rank: int = 8, alpha: float = 16.0, dropout: float = 0.0,
                 init_method: str = "kaiming", merge_weights: bool = False):
        super().__init__()
        self.base_layer = base_layer
        self.in_features, self.out_features = base_layer.in_features, base_layer.out_features
        self.rank, self.alpha, self.scaling = rank, alpha, alpha / rank
        self.dropout_p = dropout
        self.merged = False
        for p in base_layer.parameters():
            p.requires_grad_(False)
        dev, dt = base_layer.weight.device, base_layer.weight.dtype
        self.lora_A = nn.Parameter(torch.zeros(rank, self.in_features, device=dev, dtype=dt))
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, rank, device=dev, dtype=dt))
        self.reset_lora_parameters(init_method)
        if merge_weights:
            self.merge()

    @property
    def weight(self) -> torch.Tensor:
        return self.base_layer.weight

    @property
    def bias(self):
        return self.base_layer.bias

    @torch.no_grad()
    def reset_lora_parameters(self, init_method: str = "kaiming") -> None:
        if init_method == "kaiming":
            a = torch.empty(self.rank, self.in_features, dtype=torch.float32, device=self.lora_A.device)
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
            self.lora_A.copy_(a)
            self.lora_B.zero_()
        elif init_method == "zeros":
            self.lora_A.zero_()
            self.lora_B.zero_()
        elif init_method == "pissa":
            self.init_pissa()
        elif init_method == "olora":
            self.init_olora()
        else:
            raise ValueError(f"unknown init_method {init_method!r}")

    @torch.no_grad()
    def init_pissa(self) -> None:
        """Principal singular directions go into the adapter; the base keeps the residual, so the
        wrapped layer's function is unchanged at initialisation."""
        w = self.base_layer.weight.float()
        u, s, vh = _randomized_svd(w, self.rank)
        rs = torch.sqrt(s / self.scaling)
        b = u * rs[None, :]
        a = rs[:, None] * vh
        self.lora_B.copy_(b)
        self.lora_A.copy_(a)
        self.base_layer.weight.copy_((w - self.scaling * (b @ a)).to(self.base_layer.weight.dtype))

    @torch.no_grad()
    def init_olora(self) -> None:
        """Orthonormal initialisation from a QR factorisation of the weight (residual kept in the base)."""
        w = self.base_layer.weight.float()
        q, r = torch.linalg.qr(w)
        b = q[:, : self.rank]
        a = r[: self.rank]
        self.lora_B.copy_(b)
        self.lora_A.copy_(a)
        self.base_layer.weight.copy_((w - self.scaling * (b @ a)).to(self.base_layer.weight.dtype))

    def delta_weight(self) -> torch.Tensor:
        return self.scaling * (self.lora_B.float() @ self.lora_A.float())

    @torch.no_grad()
    def merge(self) -> None:
        if not self.merged:
            self.base_layer.weight.add_(self.delta_weight().to(self.base_layer.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self) -> None:
        if self.merged:
            self.base_layer.weight.sub_(self.delta_weight().to(self.base_layer.weight.dtype))
            self.merged = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        base = ops.linear(x, self.base_layer.weight, self.base_layer.bias)
        if self.merged:
            return base
        xd = F.dropout(x, self.dropout_p, self.training) if self.dropout_p > 0 else x
        h = ops.linear(xd, self.lora_A)
        return ops.linear(h, self.lora_B * self.scaling, None, base)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, rank={self.rank}, alpha={self.alpha}"


def _is_native(model: nn.Module) -> bool:
    return hasattr(model, "hf_state_dict")


def apply_lora_to_model(model: nn.Module, rank: int = 16, alpha: float = 32.0,
                        target_modules: Optional[Iterable[str]] = None, init_method: str = "kaiming",
                        dropout: float = 0.0, freeze_base: bool = True) -> nn.Module:
    """Attach adapters to every target projection and freeze everything else.

    Native models: adapters are added per split of the fused projections.  Other models: matching
    ``nn.Linear`` modules are wrapped by ``OptimizedLoRALinear``."""
    targets = list(target_modules) if target_modules is not None else list(DEFAULT_TARGET_MODULES)
    if freeze_base:
        for p in model.parameters():
            p.requires_grad_(False)
    n = 0
    if _is_native(model):
        from ..models.decoder import FusedLinear
        for mod in model.modules():
            if isinstance(mod, FusedLinear):
                for split in mod.splits:
                    if split in targets and split not in mod.lora_A:
                        mod.add_lora(split, rank, alpha, dropout, "zeros" if init_method == "zeros" else "kaiming")
                        n += 1
        model.lora_config = {"rank": rank, "alpha": alpha, "dropout": dropout, "target_modules": targets}
    else:
        for parent in list(model.modules()):
            for name, child in list(parent.named_children()):
                if isinstance(child, nn.Linear) and any(name == t or name.endswith(t) for t in targets):
                    setattr(parent, name, OptimizedLoRALinear(child, rank, alpha, dropout, init_method))
                    n += 1
        model.lora_config = {"rank": rank, "alpha": alpha, "dropout": dropout, "target_modules": targets}
    if n == 0:
        raise ValueError(f"no module matched target_modules={targets}")
    return model


def apply_lora(model: nn.Module, config: Optional[LoRAConfig] = None, **kw) -> nn.Module:
    """README-documented entry point."""
    c = config or LoRAConfig(**kw)
    return apply_lora_to_model(model, c.rank, c.alpha, c.target_modules, c.init_method, c.dropout)


def get_lora_parameters(model: nn.Module) -> List[nn.Parameter]:
    return [p for n, p in model.named_parameters() if "lora_" in n]


def get_lora_params(model: nn.Module) -> List[nn.Parameter]:
    return get_lora_parameters(model)


def count_lora_params(model: nn.Module) -> Tuple[int, int]:
    lora = sum(p.numel() for p in get_lora_parameters(model))
    return lora, sum(p.numel() for p in model.parameters())


def get_lora_optimizer_groups(model: nn.Module, lr: float = 2e-4, lr_ratio: float = 16.0, weight_decay: float = 0.0):
    from ..optimizers.lora_plus_optimizer import get_lora_plus_param_groups
    return get_lora_plus_param_groups(model, lr, lr_ratio, weight_decay)


class LoRAModel(nn.Module):
    """Wraps a model, applies adapters, and exposes adapter-level utilities."""

    def __init__(self, model: nn.Module, rank: int = 16, alpha: float = 32.0,
                 target_modules: Optional[Iterable[str]] = None, init_method: str = "kaiming", dropout: float = 0.0):
        super().__init__()
        self.model = apply_lora_to_model(model, rank, alpha, target_modules, init_method, dropout)
        self.rank, self.alpha = rank, alpha

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def get_lora_parameters(self) -> List[nn.Parameter]:
        return get_lora_parameters(self.model)

    def get_lora_state_dict(self) -> Dict[str, torch.Tensor]:
        from ..checkpoint.io import lora_state_dict
        return {k: v.detach().clone() for k, v in lora_state_dict(self.model).items()}

    def load_lora_state_dict(self, sd: Dict[str, torch.Tensor]) -> int:
        sd = {k[len("base_model.model."):] if k.startswith("base_model.model.") else k: v for k, v in sd.items()}
        if _is_native(self.model):
            own = self.model.hf_state_dict(include_lora=True)
        else:
            own = dict(self.model.state_dict())
        n = 0
        with torch.no_grad():
            for k, v in sd.items():
                if k in own:
                    own[k].copy_(v.to(own[k].dtype))
                    n += 1
        return n

    def _adapted(self):
        from ..models.decoder import FusedLinear
        for m in self.model.modules():
            if isinstance(m, OptimizedLoRALinear) or (isinstance(m, FusedLinear) and m.has_lora):
                yield m

    def merge_lora(self) -> None:
        for m in self._adapted():
            m.merge() if isinstance(m, OptimizedLoRALinear) else m.merge_lora()

    def unmerge_lora(self) -> None:
        for m in self._adapted():
            m.unmerge() if isinstance(m, OptimizedLoRALinear) else m.unmerge_lora()

    def print_trainable_parameters(self) -> Tuple[int, int]:
        tr = sum(p.numel() for p in self.model.parameters() if p.requires_grad)
        tot = sum(p.numel() for p in self.model.parameters())
        print(f"trainable params: {tr:,} || all params: {tot:,} || trainable%: {100 * tr / max(1, tot):.4f}")
        return tr, tot


def benchmark_bracketing(in_features: int = 4096, out_features: int = 4096, rank: int = 16, tokens: int = 4096,
                         device: Optional[str] = None) -> Dict[str, float]:
    """FLOPs of the two evaluation orders of ``x A^T B^T`` (the low-rank-first order is what runs)."""
    low_rank_first = 2.0 * tokens * rank * (in_features + out_features)
    weight_first = 2.0 * out_features * rank * in_features + 2.0 * tokens * in_features * out_features
    return {"low_rank_first_gflop": low_rank_first / 1e9, "weight_first_gflop": weight_first / 1e9,
            "ratio": weight_first / low_rank_first}
