"""DoRA: weight-decomposed low-rank adaptation.

``W' = m * (W + s B A) / ||W + s B A||`` with the norm taken per output row over the input
dimension and ``m`` a trainable magnitude vector initialised to ``||W||`` (so the layer starts
unchanged).  Reference: chronicals/lora/dora_adapter.py:58-298 ``DoRALinear`` (incl.
``forward_optimized``, merge/unmerge), :305-427 ``DoRAModel``, :434-578 helpers.

``forward`` never materialises ``W + s B A`` for the matmul: it evaluates the base and low-rank
products separately and rescales the output columns, which needs only the row norms.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Iterable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .lora_optimized import DEFAULT_TARGET_MODULES, OptimizedLoRALinear


class DoRALinear(nn.Module):
    def __init__(self, base_layer: nn.Linear, rank: int = 8, alpha: float = 16.0, dropout: float = 0.0,
                 detach_norm: bool = True):
        super().__init__()
        self.base_layer = base_layer
        self.in_features, self.out_features = base_layer.in_features, base_layer.out_features
        self.rank, self.alpha, self.scaling, self.dropout_p = rank, alpha, alpha / rank, dropout
        self.detach_norm = detach_norm          # treat the norm as a constant in backward (DoRA paper, sec. 4.3)
        self.merged = False
        for p in base_layer.parameters():
            p.requires_grad_(False)
        dev, dt = base_layer.weight.device, base_layer.weight.dtype
        a = torch.empty(rank, self.in_features, dtype=torch.float32, device=dev)
        nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        self.lora_A = nn.Parameter(a.to(dt))
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, rank, device=dev, dtype=dt))
        self.magnitude = nn.Parameter(base_layer.weight.detach().float().norm(dim=1).to(dt))

    def _row_norm(self) -> torch.Tensor:
        """``||W + s B A||`` per output row, computed without forming the sum:
        ``||W||² + 2 s <W, BA> + s² ||BA||²`` row-wise."""
        W = self.base_layer.weight.float()
        A, B = self.lora_A.float(), self.lora_B.float()
        w2 = W.pow(2).sum(1)
        WA = W @ A.t()                                  # [out, r]
        cross = (WA * B).sum(1)
        AA = A @ A.t()                                  # [r, r]
        ba2 = ((B @ AA) * B).sum(1)
        return (w2 + 2 * self.scaling * cross + self.scaling ** 2 * ba2).clamp_min(1e-12).sqrt()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.merged:
            return ops.linear(x, self.base_layer.weight, self.base_layer.bias)
        xd = F.dropout(x, self.dropout_p, self.training) if self.dropout_p > 0 else x
        base = ops.linear(x, self.base_layer.weight)
        low = ops.linear(ops.linear(xd, self.lora_A), self.lora_B * self.scaling)
        norm = self._row_norm()
        if self.detach_norm:
            norm = norm.detach()
        y = (base + low) * (self.magnitude.float() / norm).to(base.dtype)
        return y if self.base_layer.bias is None else y + self.base_layer.bias

    forward_optimized = forward

    def forward_reference(self, x: torch.Tensor) -> torch.Tensor:
        """Literal formula (materialises the adapted weight); used by tests."""
        W = self.base_layer.weight.float() + self.scaling * (self.lora_B.float() @ self.lora_A.float())
        Wn = self.magnitude.float()[:, None] * W / W.norm(dim=1, keepdim=True)
        return F.linear(x.float(), Wn, None if self.base_layer.bias is None else self.base_layer.bias.float()).to(x.dtype)

    @torch.no_grad()
    def merge(self) -> None:
        if self.merged:
            return
        self._saved_weight = self.base_layer.weight.detach().clone()
        W = self.base_layer.weight.float() + self.scaling * (self.lora_B.float() @ self.lora_A.float())
        W = self.magnitude.float()[:, None] * W / W.norm(dim=1, keepdim=True)
        self.base_layer.weight.copy_(W.to(self.base_layer.weight.dtype))
        self.merged = True

    @torch.no_grad()
    def unmerge(self) -> None:
        if self.merged:
            self.base_layer.weight.copy_(self._saved_weight)
            del self._saved_weight
            self.merged = False


def apply_dora_to_model(model: nn.Module, rank: int = 8, alpha: float = 16.0,
                        target_modules: Optional[Iterable[str]] = None, dropout: float = 0.0) -> nn.Module:
    targets = list(target_modules) if target_modules is not None else list(DEFAULT_TARGET_MODULES)
    for p in model.parameters():
        p.requires_grad_(False)
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear) and any(name == t or name.endswith(t) for t in targets):
                setattr(parent, name, DoRALinear(child, rank, alpha, dropout))
                n += 1
    if n == 0:
        raise ValueError(f"no nn.Linear matched target_modules={targets}; DoRA wraps plain nn.Linear modules "
                         "(for this framework's fused projections use LoRA)")
    model.dora_config = {"rank": rank, "alpha": alpha, "target_modules": targets}
    return model


def convert_lora_to_dora(module: OptimizedLoRALinear) -> DoRALinear:
    """Keeps the trained A/B; the magnitude starts at the current adapted row norm (function preserved)."""
    d = DoRALinear(module.base_layer, module.rank, module.alpha, module.dropout_p)
    with torch.no_grad():
        d.lora_A.copy_(module.lora_A)
        d.lora_B.copy_(module.lora_B)
        d.magnitude.copy_(d._row_norm().to(d.magnitude.dtype))
    return d


def get_dora_plus_param_groups(model: nn.Module, base_lr: float = 1e-4, lr_ratio: float = 16.0,
                               magnitude_lr_scale: float = 1.0, weight_decay: float = 0.0) -> List[Dict[str, Any]]:
    a, b, m, other = [], [], [], []
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        (a if "lora_A" in n else b if "lora_B" in n else m if "magnitude" in n else other).append(p)
    groups = []
    for name, ps, lr, wd in (("lora_A", a, base_lr, 0.0), ("lora_B", b, base_lr * lr_ratio, 0.0),
                             ("magnitude", m, base_lr * magnitude_lr_scale, 0.0), ("other", other, base_lr, weight_decay)):
        if ps:
            groups.append({"params": ps, "lr": lr, "weight_decay": wd, "name": name, "_group_name": name})
    return groups


class DoRAModel(nn.Module):
    def __init__(self, model: nn.Module, rank: int = 8, alpha: float = 16.0,
                 target_modules: Optional[Iterable[str]] = None, dropout: float = 0.0):
        super().__init__()
        self.model = apply_dora_to_model(model, rank, alpha, target_modules, dropout)

    def forward(self, *a, **kw):
        return self.model(*a, **kw)

    def _layers(self):
        return [m for m in self.model.modules() if isinstance(m, DoRALinear)]

    def get_dora_parameters(self) -> List[nn.Parameter]:
        return [p for n, p in self.model.named_parameters() if p.requires_grad]

    def get_dora_state_dict(self) -> Dict[str, torch.Tensor]:
        return {n: p.detach().clone() for n, p in self.model.named_parameters()
                if any(k in n for k in ("lora_A", "lora_B", "magnitude"))}

    def merge_dora(self) -> None:
        for m in self._layers():
            m.merge()

    def unmerge_dora(self) -> None:
        for m in self._layers():
            m.unmerge()

    def print_trainable_parameters(self):
        tr = sum(p.numel() for p in self.model.parameters() if p.requires_grad)
        tot = sum(p.numel() for p in self.model.parameters())
        print(f"trainable params: {tr:,} || all params: {tot:,} || trainable%: {100 * tr / max(1, tot):.4f}")
        return tr, tot
