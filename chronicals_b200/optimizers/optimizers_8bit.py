"""8-bit and paged optimizers.

The reference wraps bitsandbytes (chronicals/optimizers/optimizers_8bit.py:88-110
probe, :117-336 ``AdamW8bit`` / ``Adam8bit``, :343-426 ``PagedAdamW``, :433-550
``OptimizerStateConverter``, :557-666 ``HybridPrecisionOptimizer``, :673-748
factory).  bitsandbytes is not a dependency here: the moments are stored with
this framework's own block-wise quantisation (256-element blocks, one fp32
absmax per block; signed linear code for the first moment, unsigned for the
square-rooted second moment) and de/re-quantised around an fp32 AdamW update.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch.optim import Optimizer

from ..ops import ref

BLOCK = 256


def get_bnb_info() -> Dict[str, Any]:
    try:
        import bitsandbytes as bnb  # noqa: F401
        return {"available": True, "version": getattr(bnb, "__version__", "?")}
    except Exception:
        return {"available": False, "version": None, "note": "using the built-in block-wise 8-bit states"}


class AdamW8bit(Optimizer):
    """AdamW with 8-bit block-quantised moments (≈ 2 bytes of state per parameter instead of 8).

    Tensors smaller than ``min_8bit_size`` keep fp32 states (quantisation noise matters most there)."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 min_8bit_size: int = 4096, block_size: int = BLOCK, is_paged: bool = False):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))
        self.min_8bit_size, self.block_size, self.is_paged = min_8bit_size, block_size, is_paged

    def _kernel_ok(self, p, st) -> bool:
        """The fused kernel handles contiguous CUDA parameters (bf16 or fp32) whose moments are 8-bit, resident
        on the device (not paged) and quantised in blocks of 256."""
        if not (p.is_cuda and p.is_contiguous() and p.dtype in (torch.bfloat16, torch.float32)):
            return False
        if self.block_size != 256 or self.is_paged or st["exp_avg"].dtype != torch.int8 or not st["exp_avg"].is_cuda:
            return False
        if p.grad.dtype != p.dtype:
            return False
        from ..ops import _ext
        return _ext.available() and not _ext.reference_forced() and _ext.has_symbol("cb_adamw8bit")

    def _load(self, st, name, shape, signed):
        q = st[name]
        if q.dtype in (torch.int8, torch.uint8):
            x = ref.dequantize_blockwise_8bit(q.to(st[name + "_absmax"].device), st[name + "_absmax"], shape,
                                              self.block_size, signed)
            return x if signed else x * x          # second moment is stored as its square root
        return q

    def _store(self, st, name, x, signed):
        if st[name].dtype in (torch.int8, torch.uint8):
            y = x if signed else x.sqrt()
            q, a = ref.quantize_blockwise_8bit(y, self.block_size, signed)
            st[name] = q[: x.numel()] if q.numel() >= x.numel() else q
            st[name + "_absmax"] = a
            if self.is_paged:
                st[name] = st[name].to("cpu", non_blocking=True) if x.is_cuda else st[name]
        else:
            st[name] = x

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
                    if p.numel() >= self.min_8bit_size:
                        nb = (p.numel() + self.block_size - 1) // self.block_size
                        st["exp_avg"] = torch.zeros(p.numel(), dtype=torch.int8, device=p.device)
                        st["exp_avg_sq"] = torch.zeros(p.numel(), dtype=torch.uint8, device=p.device)
                        st["exp_avg_absmax"] = torch.zeros(nb, device=p.device)
                        st["exp_avg_sq_absmax"] = torch.zeros(nb, device=p.device)
                    else:
                        st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                        st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                t = st["step"]
                if self._kernel_ok(p, st):
                    from ..ops import _ext
                    gr = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                    code = _ext.lib().cb_adamw8bit(p.data_ptr(), gr.data_ptr(), st["exp_avg"].data_ptr(),
                                                   st["exp_avg_sq"].data_ptr(), st["exp_avg_absmax"].data_ptr(),
                                                   st["exp_avg_sq_absmax"].data_ptr(), p.numel(),
                                                   int(p.dtype == torch.bfloat16), float(g["lr"]), b1, b2, float(g["eps"]),
                                                   float(g["weight_decay"]), 1.0 - b1 ** t, 1.0 - b2 ** t, _ext.stream_ptr())
                    _ext.check(code, "adamw8bit")
                    continue
                grad = p.grad.float()
                m = self._load(st, "exp_avg", p.shape, True).to(p.device)
                v = self._load(st, "exp_avg_sq", p.shape, False).to(p.device)
                m = m * b1 + grad * (1 - b1)
                v = v * b2 + grad * grad * (1 - b2)
                x = p.detach().float()
                if g["weight_decay"]:
                    x.mul_(1 - g["lr"] * g["weight_decay"])
                denom = (v / (1 - b2 ** t)).sqrt_().add_(g["eps"])
                x.addcdiv_(m, denom, value=-g["lr"] / (1 - b1 ** t))
                p.copy_(x)
                self._store(st, "exp_avg", m, True)
                self._store(st, "exp_avg_sq", v, False)
        return loss

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        """``torch.optim.Optimizer.load_state_dict`` casts every state tensor to the parameter dtype, which would
        turn the int8 / uint8 codes and the fp32 block maxima into bf16.  The saved tensors are put back with
        their own dtypes (on the parameter's device, or on the host for the paged variant)."""
        super().load_state_dict(state_dict)
        saved = state_dict["state"]
        ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for pid, p in zip(ids, params):
            src = saved.get(pid)
            if src is None:
                continue
            st = self.state[p]
            for name, val in src.items():
                if torch.is_tensor(val):
                    on_host = self.is_paged and val.dtype in (torch.int8, torch.uint8)
                    st[name] = val.detach().clone().to("cpu" if on_host else p.device)
                else:
                    st[name] = val

    def state_bytes(self) -> int:
        n = 0
        for st in self.state.values():
            for v in st.values():
                if isinstance(v, torch.Tensor):
                    n += v.numel() * v.element_size()
        return n


class Adam8bit(AdamW8bit):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, **kw):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)


class PagedAdamW(AdamW8bit):
    """8-bit AdamW whose quantised moments live in host memory between steps (frees device memory
    at the cost of PCIe traffic per step)."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01, **kw):
        kw.pop("is_paged", None)
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, is_paged=True, **kw)


class OptimizerStateConverter:
    """Converts AdamW states between fp32 (``torch.optim.AdamW`` / ``FusedAdamW``) and the 8-bit layout."""

    @staticmethod
    def to_8bit(state: Dict[str, torch.Tensor], block_size: int = BLOCK) -> Dict[str, torch.Tensor]:
        m, v = state["exp_avg"].float(), state["exp_avg_sq"].float()
        qm, am = ref.quantize_blockwise_8bit(m, block_size, True)
        qv, av = ref.quantize_blockwise_8bit(v.sqrt(), block_size, False)
        return {"exp_avg": qm[: m.numel()], "exp_avg_absmax": am, "exp_avg_sq": qv[: v.numel()],
                "exp_avg_sq_absmax": av, "step": int(state.get("step", 0))}

    @staticmethod
    def to_fp32(state: Dict[str, torch.Tensor], shape, block_size: int = BLOCK) -> Dict[str, torch.Tensor]:
        m = ref.dequantize_blockwise_8bit(state["exp_avg"], state["exp_avg_absmax"], shape, block_size, True)
        r = ref.dequantize_blockwise_8bit(state["exp_avg_sq"], state["exp_avg_sq_absmax"], shape, block_size, False)
        return {"exp_avg": m, "exp_avg_sq": r * r, "step": int(state.get("step", 0))}


class HybridPrecisionOptimizer(Optimizer):
    """8-bit states for the large matrices, full-precision fused AdamW for everything small
    (norms, biases, adapters)."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 size_threshold: int = 1 << 20):
        plist = [p for p in params if p.requires_grad]
        big = [p for p in plist if p.numel() >= size_threshold]
        small = [p for p in plist if p.numel() < size_threshold]
        from .fused_adamw import FusedAdamW
        self.opt8 = AdamW8bit(big, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay) if big else None
        self.opt32 = FusedAdamW(small, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, max_grad_norm=0.0) \
            if small else None
        super().__init__([{"params": plist}], {"lr": lr})
        self.param_groups = (self.opt8.param_groups if self.opt8 else []) + (self.opt32.param_groups if self.opt32 else [])

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for o in (self.opt8, self.opt32):
            if o:
                o.step()
        return loss

    def zero_grad(self, set_to_none: bool = True):
        for o in (self.opt8, self.opt32):
            if o:
                o.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {"opt8": self.opt8.state_dict() if self.opt8 else None,
                "opt32": self.opt32.state_dict() if self.opt32 else None}

    def load_state_dict(self, sd):
        if self.opt8 and sd.get("opt8"):
            self.opt8.load_state_dict(sd["opt8"])
        if self.opt32 and sd.get("opt32"):
            self.opt32.load_state_dict(sd["opt32"])


def create_8bit_optimizer(model_or_params, optimizer_type: str = "adamw8bit", lr: float = 1e-3, betas=(0.9, 0.999),
                          eps: float = 1e-8, weight_decay: float = 0.01, **kw) -> Optimizer:
    params = [p for p in (model_or_params.parameters() if hasattr(model_or_params, "parameters") else model_or_params)
              if p.requires_grad]
    t = optimizer_type.lower()
    if t in ("adamw8bit", "adamw_8bit", "8bit_adam"):
        return AdamW8bit(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
    if t in ("adam8bit", "adam_8bit"):
        return Adam8bit(params, lr=lr, betas=betas, eps=eps, **kw)
    if t in ("paged_adamw", "pagedadamw"):
        return PagedAdamW(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
    if t == "hybrid":
        return HybridPrecisionOptimizer(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
    raise ValueError(f"unknown 8-bit optimizer type {optimizer_type!r}")
