"""Alternative optimizers, learning-rate schedules and factories.

Same classes and update rules as the reference module
(chronicals/optimizers/optimizers.py:24-155 ``ScheduleFreeAdamW``, :162-267
``Muon``, :336-417 ``AdamAtan2``, :424-523 ``HybridMuonAdamW``, :530-602
``WSDScheduler``, :605-677 ``OneCycleLR``, :684-803 factories).  One deliberate
difference: ``OneCycleLR`` here scales each parameter group's own base rate, so
a LoRA+ A/B ratio survives the schedule (the reference writes one rate to all
groups).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Iterable, List, Optional

import torch
from torch.optim import Optimizer
from torch.optim.lr_scheduler import LRScheduler


# ------------------------------------------------------------------------------------------- ScheduleFreeAdamW
class ScheduleFreeAdamW(Optimizer):
    """Schedule-free AdamW: the optimizer iterates on ``z`` and the model holds the running
    average ``x``; ``eval_mode()`` / ``train_mode()`` swap the parameters between the two."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 warmup_steps: int = 0):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                                      warmup_steps=warmup_steps))
        self._mode = "train"

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["z"] = p.detach().clone().float()
                    st["exp_avg"] = torch.zeros_like(st["z"])
                    st["exp_avg_sq"] = torch.zeros_like(st["z"])
                st["step"] += 1
                t = st["step"]
                grad = p.grad.float()
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                denom = st["exp_avg_sq"].sqrt() / math.sqrt(1 - b2 ** t) + g["eps"]
                warm = min(1.0, t / g["warmup_steps"]) if g["warmup_steps"] > 0 else 1.0
                x = p.detach().float()
                if g["weight_decay"]:
                    x.mul_(1 - g["lr"] * g["weight_decay"])
                st["z"].addcdiv_(st["exp_avg"], denom, value=-g["lr"] * warm / (1 - b1 ** t))
                x.mul_(1 - 1.0 / t).add_(st["z"], alpha=1.0 / t)
                p.copy_(x)
        return loss

    @torch.no_grad()
    def eval_mode(self) -> None:
        if self._mode == "eval":
            return
        for g in self.param_groups:
            for p in g["params"]:
                st = self.state.get(p)
                if st and "z" in st:
                    st["x_backup"] = p.detach().clone()
                    p.copy_(st["z"])
        self._mode = "eval"

    @torch.no_grad()
    def train_mode(self) -> None:
        if self._mode == "train":
            return
        for g in self.param_groups:
            for p in g["params"]:
                st = self.state.get(p)
                if st and "x_backup" in st:
                    p.copy_(st.pop("x_backup"))
        self._mode = "train"


# ------------------------------------------------------------------------------------------- Muon
def newton_schulz_orthogonalize(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate orthogonalisation ``X <- 1.5 X - 0.5 (X X^T) X`` of a matrix scaled so its
    singular values start below sqrt(3).  CUDA bf16 matrices run the two products of every iteration on the
    tcgen05 GEMM (``X X^T`` is the NT form, ``(X X^T) X`` the NN form, no transposed copies); everything
    else uses fp32 matmuls."""
    transposed = G.shape[0] > G.shape[1]
    if (G.is_cuda and G.dtype == torch.bfloat16 and G.dim() == 2 and G.shape[0] % 8 == 0 and G.shape[1] % 8 == 0):
        from .. import ops
        if ops._fast(G):
            X = (G.t() if transposed else G).contiguous()
            X = (X.float() / (X.float().norm() + 1e-7)).to(torch.bfloat16)
            for _ in range(steps):
                A = ops.gemm(X, X)                                         # X X^T      [m, m]
                AX = ops.gemm(A, X, b_mn=True, out_dtype=torch.float32)    # (X X^T) X  [m, n], fp32 out
                X = (1.5 * X.float() - 0.5 * AX).to(torch.bfloat16)
            return (X.t() if transposed else X).contiguous().to(G.dtype)
    X = G.float()
    if transposed:
        X = X.t()
    X = X / (X.norm() + 1e-7)
    for _ in range(steps):
        X = 1.5 * X - 0.5 * (X @ X.t()) @ X
    if transposed:
        X = X.t()
    return X.to(G.dtype)


class Muon(Optimizer):
    """Momentum with orthogonalised updates for 2-D parameters; SGD-momentum for the rest."""

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5,
                 weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(grad)
                buf = st["momentum_buffer"]
                buf.mul_(g["momentum"]).add_(grad)
                u = grad.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                if p.dim() >= 2:
                    u2 = u.reshape(u.shape[0], -1)
                    o = newton_schulz_orthogonalize(u2, g["ns_steps"])
                    o = o * math.sqrt(max(1.0, u2.shape[0] / u2.shape[1]))
                    u = o.reshape(u.shape)
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(u.to(p.dtype), alpha=-g["lr"])
        return loss


# ------------------------------------------------------------------------------------------- AdamAtan2
class AdamAtan2(Optimizer):
    """Adam whose update is ``a * atan2(m_hat, sqrt(v_hat))`` — bounded, scale-invariant, no epsilon."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.99), weight_decay: float = 0.0, a: float = 1.27):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), weight_decay=weight_decay, a=a))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                t = st["step"]
                grad = p.grad.float()
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                m_hat = st["exp_avg"] / (1 - b1 ** t)
                v_hat = st["exp_avg_sq"] / (1 - b2 ** t)
                x = p.detach().float()
                if g["weight_decay"]:
                    x.mul_(1 - g["lr"] * g["weight_decay"])
                x.add_(torch.atan2(m_hat, v_hat.sqrt()), alpha=-g["lr"] * g["a"])
                p.copy_(x)
        return loss


# ------------------------------------------------------------------------------------------- Hybrid Muon + AdamW
_MUON_NAME_HINTS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "qkv_proj",
                    "gate_up_proj", "attention", "mlp", "self_attn", "feed_forward")


class HybridMuonAdamW(Optimizer):
    """Muon on the hidden 2-D weight matrices, AdamW on everything else (embeddings, norms, biases, head)."""

    def __init__(self, model_or_named_params, lr: float = 1e-3, muon_lr: Optional[float] = None, betas=(0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.01, momentum: float = 0.95):
        named = list(model_or_named_params.named_parameters()) if hasattr(model_or_named_params, "named_parameters") \
            else list(model_or_named_params)
        muon_p, adam_p = [], []
        for name, p in named:
            if not p.requires_grad:
                continue
            if p.dim() >= 2 and any(h in name for h in _MUON_NAME_HINTS) and "embed" not in name and "lm_head" not in name:
                muon_p.append(p)
            else:
                adam_p.append(p)
        self.muon = Muon(muon_p, lr=muon_lr if muon_lr is not None else lr * 10, momentum=momentum) if muon_p else None
        from .fused_adamw import FusedAdamW
        self.adamw = FusedAdamW(adam_p, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                max_grad_norm=0.0) if adam_p else None
        groups = (self.muon.param_groups if self.muon else []) + (self.adamw.param_groups if self.adamw else [])
        super().__init__([{"params": [p for g in groups for p in g["params"]]}], {"lr": lr})
        self.param_groups = groups

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.muon:
            self.muon.step()
        if self.adamw:
            self.adamw.step()
        return loss

    def zero_grad(self, set_to_none: bool = True):
        for o in (self.muon, self.adamw):
            if o:
                o.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {"muon": self.muon.state_dict() if self.muon else None,
                "adamw": self.adamw.state_dict() if self.adamw else None}

    def load_state_dict(self, sd):
        if self.muon and sd.get("muon"):
            self.muon.load_state_dict(sd["muon"])
        if self.adamw and sd.get("adamw"):
            self.adamw.load_state_dict(sd["adamw"])


# ------------------------------------------------------------------------------------------- 8-bit passthrough
class Adam8bit:
    """Constructor-compatible wrapper: returns the block-wise 8-bit AdamW of ``optimizers_8bit``."""

    def __new__(cls, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, **kw):
        from .optimizers_8bit import AdamW8bit
        return AdamW8bit(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)


# ------------------------------------------------------------------------------------------- schedulers
class WSDScheduler(LRScheduler):
    """Warm-up, stable, decay: ``step/warmup`` → 1.0 for ``stable_ratio`` of training → cosine or
    linear decay to ``min_lr_ratio``.  Per-group base rates are preserved."""

    def __init__(self, optimizer, total_steps: int, warmup_ratio: float = 0.05, stable_ratio: float = 0.80,
                 min_lr_ratio: float = 0.1, decay_type: str = "cosine", warmup_steps: Optional[int] = None,
                 last_epoch: int = -1):
        self.total_steps = max(1, int(total_steps))
        self.warmup_steps = int(warmup_steps) if warmup_steps is not None and warmup_steps >= 0 \
            else int(self.total_steps * warmup_ratio)
        self.stable_steps = int(self.total_steps * stable_ratio)
        self.decay_steps = max(1, self.total_steps - self.warmup_steps - self.stable_steps)
        self.min_lr_ratio = min_lr_ratio
        self.decay_type = decay_type
        super().__init__(optimizer, last_epoch)

    def multiplier(self, step: int) -> float:
        if self.warmup_steps > 0 and step < self.warmup_steps:
            return (step + 1) / self.warmup_steps
        if step < self.warmup_steps + self.stable_steps:
            return 1.0
        prog = min(1.0, (step - self.warmup_steps - self.stable_steps) / self.decay_steps)
        if self.decay_type == "linear":
            return 1.0 - (1.0 - self.min_lr_ratio) * prog
        return self.min_lr_ratio + (1.0 - self.min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * prog))

    def get_lr(self) -> List[float]:
        m = self.multiplier(max(self.last_epoch, 0))
        return [b * m for b in self.base_lrs]


class OneCycleLR(LRScheduler):
    """One-cycle: ramp ``base/25 → base`` over ``pct_start`` of training, then anneal to ``base/25/1e4``."""

    def __init__(self, optimizer, total_steps: int, max_lr: Optional[float] = None, pct_start: float = 0.3,
                 anneal_strategy: str = "cos", div_factor: float = 25.0, final_div_factor: float = 1e4,
                 last_epoch: int = -1):
        self.total_steps = max(1, int(total_steps))
        self.pct_start, self.anneal = pct_start, anneal_strategy
        self.div_factor, self.final_div_factor = div_factor, final_div_factor
        self._max_lr_scale: Optional[float] = None
        if max_lr is not None:
            ref_lr = max(g["lr"] for g in optimizer.param_groups)
            self._max_lr_scale = max_lr / ref_lr if ref_lr > 0 else 1.0
        super().__init__(optimizer, last_epoch)

    def _interp(self, a: float, b: float, pct: float) -> float:
        if self.anneal == "linear":
            return a + (b - a) * pct
        return b + (a - b) * 0.5 * (1.0 + math.cos(math.pi * pct))

    def multiplier(self, step: int) -> float:
        up = max(1.0, self.pct_start * self.total_steps)
        lo, hi, end = 1.0 / self.div_factor, 1.0, 1.0 / (self.div_factor * self.final_div_factor)
        if step <= up:
            return self._interp(lo, hi, step / up)
        return self._interp(hi, end, min(1.0, (step - up) / max(1.0, self.total_steps - up)))

    def get_lr(self) -> List[float]:
        m = self.multiplier(max(self.last_epoch, 0)) * (self._max_lr_scale or 1.0)
        return [b * m for b in self.base_lrs]


class WarmupCosineScheduler(LRScheduler):
    """Linear warm-up from ``start_factor`` then cosine to ``min_lr_ratio`` (the trainer's ``cosine``);
    with ``cosine=False`` the rate stays constant after warm-up (``constant``)."""

    def __init__(self, optimizer, total_steps: int, warmup_steps: int, min_lr_ratio: float = 0.1,
                 start_factor: float = 0.1, cosine: bool = True, last_epoch: int = -1):
        self.total_steps, self.warmup_steps = max(1, int(total_steps)), max(0, int(warmup_steps))
        self.min_lr_ratio, self.start_factor, self.cosine = min_lr_ratio, start_factor, cosine
        super().__init__(optimizer, last_epoch)

    def multiplier(self, step: int) -> float:
        if step < self.warmup_steps:
            return self.start_factor + (1 - self.start_factor) * step / max(1, self.warmup_steps)
        if not self.cosine:
            return 1.0
        prog = min(1.0, (step - self.warmup_steps) / max(1, self.total_steps - self.warmup_steps))
        return self.min_lr_ratio + (1 - self.min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * prog))

    def get_lr(self) -> List[float]:
        m = self.multiplier(max(self.last_epoch, 0))
        return [b * m for b in self.base_lrs]


# ------------------------------------------------------------------------------------------- factories
def _trainable(model_or_params) -> List[torch.nn.Parameter]:
    if hasattr(model_or_params, "parameters"):
        return [p for p in model_or_params.parameters() if p.requires_grad]
    return [p for p in model_or_params if p.requires_grad]


def create_optimizer(model, optimizer_type: str = "fused_adamw", lr: float = 2e-5, weight_decay: float = 0.01,
                     betas=(0.9, 0.95), eps: float = 1e-8, max_grad_norm: float = 1.0, **kw) -> Optimizer:
    from .fused_adamw import FusedAdamW
    t = optimizer_type.lower()
    if t in ("fused_adamw", "adamw_fused"):
        return FusedAdamW(_trainable(model), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                          max_grad_norm=max_grad_norm, **kw)
    if t == "adamw":
        return torch.optim.AdamW(_trainable(model), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if t == "schedule_free":
        return ScheduleFreeAdamW(_trainable(model), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                 warmup_steps=kw.get("warmup_steps", 0))
    if t == "muon":
        return Muon(_trainable(model), lr=lr * 10, weight_decay=weight_decay)
    if t == "hybrid_muon":
        return HybridMuonAdamW(model, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if t in ("8bit_adam", "adamw8bit", "adam8bit"):
        from .optimizers_8bit import AdamW8bit
        return AdamW8bit(_trainable(model), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if t == "paged_adamw":
        from .optimizers_8bit import PagedAdamW
        return PagedAdamW(_trainable(model), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if t == "adam_atan2":
        return AdamAtan2(_trainable(model), lr=lr, betas=(betas[0], 0.99), weight_decay=weight_decay)
    if t in ("lora_plus", "loraplus"):
        from .lora_plus_optimizer import create_lora_plus_optimizer
        return create_lora_plus_optimizer(model, base_lr=lr, lr_ratio=kw.get("lr_ratio", 16.0), betas=betas, eps=eps,
                                          weight_decay=weight_decay)
    raise ValueError(f"unknown optimizer_type {optimizer_type!r}")


def create_scheduler(optimizer, scheduler_type: str = "wsd", total_steps: int = 1000, warmup_ratio: float = 0.03,
                     min_lr_ratio: float = 0.1, stable_ratio: float = 0.80, warmup_steps: Optional[int] = None,
                     **kw) -> Optional[LRScheduler]:
    t = (scheduler_type or "constant").lower()
    ws = int(warmup_steps) if warmup_steps is not None and warmup_steps >= 0 else int(total_steps * warmup_ratio)
    target = optimizer.adamw if isinstance(optimizer, HybridMuonAdamW) and optimizer.adamw else optimizer
    if t == "wsd":
        return WSDScheduler(target, total_steps, warmup_ratio, stable_ratio, min_lr_ratio,
                            kw.get("decay_type", "cosine"), warmup_steps=warmup_steps)
    if t == "one_cycle":
        return OneCycleLR(target, total_steps, max_lr=kw.get("max_lr"), pct_start=kw.get("pct_start", 0.3))
    if t == "cosine":
        return WarmupCosineScheduler(target, total_steps, ws, min_lr_ratio, 0.1, True)
    if t == "constant":
        return WarmupCosineScheduler(target, total_steps, ws, 1.0, 0.1, False)
    if t in ("none", ""):
        return None
    raise ValueError(f"unknown lr_scheduler_type {scheduler_type!r}")
