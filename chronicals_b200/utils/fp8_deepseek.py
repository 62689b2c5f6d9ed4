"""Block-scaled FP8 training stack.

API follows the reference's DeepSeek-V3-style module (chronicals/utils/fp8_deepseek.py:69-108
``FP8Spec``, :115-368 ``FP8GradScaler``, :375-504 ``FP8GradientAccumulator``, :781-986 block
quantisers, :993-1067 ``AmaxHistory``, :1074-1300 ``FP8LinearFunction`` / ``FP8Linear``, :1308-1449 model
conversion, :1456-1513 ``FP8Context``, :1917-2018 ``SmoothSwiGLU``, :2025-2137
``PerTensorDynamicScaler``, :2144-2343 ``FP8TrainingConfig`` / ``FP8Trainer``).

Differences: blocks are the OCP MX ones (32 elements, e8m0 power-of-two scales) instead of 128
elements with fp32 scales; conversions are real (hardware ``cvt``) instead of hand-rolled rounding;
the exclude list no longer contains the bare word ``gate`` (which also excluded ``gate_proj``);
nothing synchronises with the host on the forward path.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import ref
from .fp8_utils import FP8Format, FP8Linear, _MXFP8LinearFn, compute_fp8_memory_savings, mxfp8_dequantize, mxfp8_quantize


@dataclass
class FP8Spec:
    name: str
    max_value: float
    min_normal: float
    mantissa_bits: int
    exponent_bits: int
    torch_dtype: torch.dtype

    @classmethod
    def e4m3(cls) -> "FP8Spec":
        return cls("e4m3", ref.E4M3_MAX, 2.0 ** -6, 3, 4, torch.float8_e4m3fn)

    @classmethod
    def e5m2(cls) -> "FP8Spec":
        return cls("e5m2", ref.E5M2_MAX, 2.0 ** -14, 2, 5, torch.float8_e5m2)


E4M3, E5M2 = FP8Spec.e4m3(), FP8Spec.e5m2()
MX_BLOCK_SIZE = ref.MX_BLOCK


# ------------------------------------------------------------------------------------------- quantisers
def quantize_block_e4m3(x: torch.Tensor, block_size: int = MX_BLOCK_SIZE) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 values + e8m0 block scales (``block_size`` is fixed at 32 by the MX format)."""
    return mxfp8_quantize(x, "e4m3")


def quantize_block_e5m2(x: torch.Tensor, block_size: int = MX_BLOCK_SIZE) -> Tuple[torch.Tensor, torch.Tensor]:
    return mxfp8_quantize(x, "e5m2")


def dequantize_block(q: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return mxfp8_dequantize(q, scales, dtype)


class AmaxHistory:
    """Ring buffer of recent absolute maxima kept on the device (no ``.item()``)."""

    def __init__(self, length: int = 32, device=None):
        self.length = length
        self.buf = torch.zeros(length, dtype=torch.float32, device=device)
        self.idx = 0
        self.count = 0

    def update(self, x: torch.Tensor) -> None:
        if self.buf.device != x.device:
            self.buf = self.buf.to(x.device)
        self.buf[self.idx] = x.detach().abs().amax().float()
        self.idx = (self.idx + 1) % self.length
        self.count = min(self.count + 1, self.length)

    def amax(self) -> torch.Tensor:
        return self.buf.max()

    def get_scale(self, fmt_max: float = ref.E4M3_MAX, margin: float = 1.0) -> torch.Tensor:
        a = self.amax()
        return torch.where(a > 0, (fmt_max / margin) / a, torch.ones_like(a))


class PerTensorDynamicScaler:
    """Per-tensor delayed scaling (COAT-style): scale from the amax history, refreshed every step."""

    def __init__(self, fmt: FP8Spec = E4M3, history_len: int = 16, margin: float = 1.0):
        self.fmt, self.margin = fmt, margin
        self.history = AmaxHistory(history_len)

    def quantize(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        self.history.update(x)
        s = self.history.get_scale(self.fmt.max_value, self.margin)
        q = (x.float() * s).clamp(-self.fmt.max_value, self.fmt.max_value).to(self.fmt.torch_dtype)
        return q, 1.0 / s

    @staticmethod
    def dequantize(q: torch.Tensor, inv_scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return (q.float() * inv_scale).to(dtype)


# ------------------------------------------------------------------------------------------- grad scaling
class FP8GradScaler:
    """Dynamic loss scaling with overflow back-off (growth ×2 every ``growth_interval`` clean steps,
    back-off ×0.5 on inf/nan), checked on the device; ``step`` skips the update after an overflow."""

    def __init__(self, init_scale: float = 2.0 ** 15, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 1000, min_scale: float = 1.0, max_scale: float = 2.0 ** 24, enabled: bool = True):
        self.scale_value, self.growth_factor, self.backoff_factor = init_scale, growth_factor, backoff_factor
        self.growth_interval, self.min_scale, self.max_scale, self.enabled = growth_interval, min_scale, max_scale, enabled
        self._good, self.num_overflows, self.num_steps = 0, 0, 0
        self._found_inf = False

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self.scale_value if self.enabled else loss

    def unscale_(self, optimizer) -> bool:
        if not self.enabled:
            return False
        inv = 1.0 / self.scale_value
        found = torch.zeros((), dtype=torch.float32)
        for g in optimizer.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    p.grad.mul_(inv)
                    found = found.to(p.grad.device) + (~torch.isfinite(p.grad)).any().float()
        self._found_inf = bool(found.item() > 0)
        return self._found_inf

    def step(self, optimizer) -> bool:
        """Returns True when the optimizer step was taken."""
        self.num_steps += 1
        if self.enabled and self._found_inf:
            optimizer.zero_grad(set_to_none=True)
            return False
        optimizer.step()
        return True

    def update(self) -> float:
        if not self.enabled:
            return self.scale_value
        if self._found_inf:
            self.scale_value = max(self.min_scale, self.scale_value * self.backoff_factor)
            self._good = 0
            self.num_overflows += 1
        else:
            self._good += 1
            if self._good >= self.growth_interval:
                self.scale_value = min(self.max_scale, self.scale_value * self.growth_factor)
                self._good = 0
        self._found_inf = False
        return self.scale_value

    def state_dict(self) -> Dict[str, Any]:
        return {"scale": self.scale_value, "good_steps": self._good, "num_overflows": self.num_overflows}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.scale_value, self._good = sd["scale"], sd.get("good_steps", 0)
        self.num_overflows = sd.get("num_overflows", 0)


class FP8GradientAccumulator:
    """Accumulates low-precision gradients of several micro-batches in fp32 and writes the mean back."""

    def __init__(self, params: Iterable[nn.Parameter], use_fp8_communication: bool = False):
        self.params = [p for p in params if p.requires_grad]
        self.buffers: Dict[int, torch.Tensor] = {}
        self.count = 0
        self.use_fp8_communication = use_fp8_communication

    def accumulate(self) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            b = self.buffers.get(id(p))
            if b is None:
                b = self.buffers[id(p)] = torch.zeros_like(p, dtype=torch.float32)
            b.add_(p.grad.float())
            p.grad = None
        self.count += 1

    def finalize(self) -> None:
        n = max(1, self.count)
        for p in self.params:
            b = self.buffers.get(id(p))
            if b is not None:
                p.grad = (b / n).to(p.dtype)
                b.zero_()
        self.count = 0


# ------------------------------------------------------------------------------------------- linear + conversion
FP8LinearFunction = _MXFP8LinearFn

DEFAULT_FP8_EXCLUDE_PATTERNS = ["embed_tokens", "embeddings", "wte", "wpe", "lm_head", "output", "classifier", "norm",
                                "layernorm", "layer_norm", "rmsnorm", "ln_", "router", "mlp.gate."]


def should_convert_to_fp8(name: str, module: nn.Module, exclude_patterns: Optional[List[str]] = None,
                          min_features: int = 32) -> bool:
    if not isinstance(module, nn.Linear):
        return False
    pats = DEFAULT_FP8_EXCLUDE_PATTERNS if exclude_patterns is None else exclude_patterns
    low = name.lower()
    if any(p in low for p in pats):
        return False
    return module.in_features % 32 == 0 and module.in_features >= min_features


def convert_linear_to_fp8(linear: nn.Linear) -> FP8Linear:
    return FP8Linear.from_linear(linear)


class _FusedFP8Mixin:
    """Marks this framework's fused projections to compute with MXFP8 operands."""


def convert_model_to_fp8(model: nn.Module, exclude_patterns: Optional[List[str]] = None, verbose: bool = False,
                         mode: str = "mxfp8") -> nn.Module:
    """Replace eligible ``nn.Linear`` modules by ``FP8Linear`` (bf16 master weights are kept); fused
    projections of native models are switched to an FP8 forward: ``mode="mxfp8"`` = MX block-scaled operands
    (32-element blocks, e8m0 scales) in forward, dX and dW, multiplied by the block-scaled tensor-core GEMM
    (``kind::mxf8f6f4.block_scale``: the tensor core applies the scales), ``mode="rowwise"`` = e4m3 operands
    with per-token / per-channel scales multiplied by the FP8 tensor-core GEMM (``kind::f8f6f4``) in the
    forward only."""
    if mode not in ("mxfp8", "rowwise"):
        raise ValueError(f"unknown fp8 mode {mode!r}")
    n = 0
    from ..models.decoder import FusedLinear
    pats = DEFAULT_FP8_EXCLUDE_PATTERNS if exclude_patterns is None else list(exclude_patterns)
    for name, mod in list(model.named_modules()):
        if isinstance(mod, FusedLinear):
            if not any(p in name.lower() for p in pats) and mod.in_features % 32 == 0:
                mod.use_mxfp8 = mode == "mxfp8"
                mod.use_fp8_rowwise = mode == "rowwise"
                n += 1
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            full = f"{parent_name}.{child_name}" if parent_name else child_name
            if should_convert_to_fp8(full, child, pats):
                setattr(parent, child_name, convert_linear_to_fp8(child))
                n += 1
    if verbose:
        print(f"[fp8] {n} projections now compute with MXFP8 operands")
    model._fp8_converted = n
    return model


def apply_fp8_to_huggingface_model(model: nn.Module, exclude_patterns: Optional[List[str]] = None) -> nn.Module:
    return convert_model_to_fp8(model, exclude_patterns)


class FP8Context:
    """Holds per-step FP8 caches (quantised weights are valid until the optimizer changes them)."""

    def __init__(self, model: nn.Module):
        self.model = model
        self.step = 0
        self._cache: Dict[int, Any] = {}

    def get_cached_weight(self, module: nn.Module):
        return self._cache.get(id(module))

    def cache_weight(self, module: nn.Module, value) -> None:
        self._cache[id(module)] = value

    def invalidate_caches(self) -> None:
        self._cache.clear()
        self.step += 1

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.invalidate_caches()
        return False


# ------------------------------------------------------------------------------------------- SmoothSwiGLU
class SmoothSwiGLU(nn.Module):
    """SwiGLU whose output is divided by a per-channel smoothing scale before FP8 quantisation
    (the scale is folded back into the consumer's weight), taming activation outliers."""

    def __init__(self, intermediate_size: int, momentum: float = 0.99):
        super().__init__()
        self.register_buffer("smooth_scale", torch.ones(intermediate_size))
        self.momentum = momentum

    def forward(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        y = ref.swiglu(gate, up)
        if self.training:
            with torch.no_grad():
                amax = y.detach().abs().reshape(-1, y.shape[-1]).amax(0).float().clamp_min(1e-6)
                self.smooth_scale.mul_(self.momentum).add_(amax.to(self.smooth_scale.device), alpha=1 - self.momentum)
        return y / self.smooth_scale.to(y.dtype)

    def fold_into(self, down_proj: nn.Linear) -> None:
        """Multiply the consumer's input columns by the scale so the product is unchanged."""
        with torch.no_grad():
            down_proj.weight.mul_(self.smooth_scale.to(down_proj.weight.dtype)[None, :])


def replace_swiglu_with_smooth(model: nn.Module) -> int:
    n = 0
    for mod in model.modules():
        if hasattr(mod, "gate_proj") and hasattr(mod, "up_proj") and not hasattr(mod, "smooth_swiglu"):
            mod.smooth_swiglu = SmoothSwiGLU(mod.gate_proj.out_features)
            n += 1
    return n


# ------------------------------------------------------------------------------------------- attention in FP8
class FP8AttentionConfig:
    """Options of the FP8 attention path (reference fp8_deepseek.py:1760-1787): which tensors are rounded to e4m3
    and with which block size.  Scores and softmax always stay in fp32 inside the attention kernel."""

    def __init__(self, use_fp8_qkv: bool = True, use_fp8_output: bool = True, qkv_block_size: int = MX_BLOCK_SIZE,
                 compute_dtype: torch.dtype = torch.float32, output_dtype: torch.dtype = torch.bfloat16):
        self.use_fp8_qkv, self.use_fp8_output, self.qkv_block_size = use_fp8_qkv, use_fp8_output, qkv_block_size
        self.compute_dtype, self.output_dtype = compute_dtype, output_dtype


def prepare_fp8_attention_inputs(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                 config: Optional[FP8AttentionConfig] = None):
    """Q, K, V → block-scaled e4m3 payloads plus their scales (``{"q_scales", "k_scales", "v_scales"}``)."""
    cfg = config or FP8AttentionConfig()
    if not cfg.use_fp8_qkv:
        return query, key, value, {}
    (q8, qs), (k8, ks), (v8, vs) = (quantize_block_e4m3(t, cfg.qkv_block_size) for t in (query, key, value))
    return q8, k8, v8, {"q_scales": qs, "k_scales": ks, "v_scales": vs}


def fp8_flash_attention_forward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                config: Optional[FP8AttentionConfig] = None, causal: bool = True,
                                softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Attention on operands rounded through block-scaled e4m3 (``[batch, seq, heads, head_dim]`` in and out;
    grouped-query K / V allowed).  The reference simulates FP8 the same way: quantise, dequantise, run the
    ordinary attention (fp8_deepseek.py:1826-1910); here the attention itself is this framework's varlen
    kernel on CUDA bf16 inputs and SDPA elsewhere."""
    cfg = config or FP8AttentionConfig()
    q8, k8, v8, sc = prepare_fp8_attention_inputs(query, key, value, cfg)
    if sc:
        q, k, v = (dequantize_block(t, sc[n], query.dtype) for t, n in
                   ((q8, "q_scales"), (k8, "k_scales"), (v8, "v_scales")))
    else:
        q, k, v = query, key, value
    B, S, H, D = q.shape
    scale = softmax_scale if softmax_scale is not None else D ** -0.5
    if q.is_cuda and q.dtype == torch.bfloat16 and causal and D in (64, 128):
        from .. import ops
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=q.device)
        out = ops.attention_varlen(q.reshape(B * S, H, D), k.reshape(B * S, -1, D), v.reshape(B * S, -1, D), cu, S,
                                   softmax_scale=scale).view(B, S, H, D)
    else:
        out = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal, scale=scale,
            enable_gqa=q.shape[2] != k.shape[2]).transpose(1, 2)
    if cfg.use_fp8_output:
        o8, os_ = quantize_block_e4m3(out.contiguous(), cfg.qkv_block_size)
        out = dequantize_block(o8, os_, cfg.output_dtype)
    return out.to(cfg.output_dtype)


# ------------------------------------------------------------------------------------------- trainer wrapper
@dataclass
class FP8TrainingConfig:
    enabled: bool = True
    forward_format: str = "e4m3"
    backward_format: str = "e5m2"
    block_size: int = MX_BLOCK_SIZE
    amax_history_len: int = 32
    use_loss_scaling: bool = False           # bf16 master weights: loss scaling is normally unnecessary
    exclude_patterns: List[str] = field(default_factory=lambda: list(DEFAULT_FP8_EXCLUDE_PATTERNS))


class FP8Trainer:
    """Minimal loop helper: converts the model, owns the grad scaler and the FP8 context."""

    def __init__(self, model: nn.Module, optimizer: torch.optim.Optimizer, config: Optional[FP8TrainingConfig] = None):
        self.config = config or FP8TrainingConfig()
        self.model = convert_model_to_fp8(model, self.config.exclude_patterns) if self.config.enabled else model
        self.optimizer = optimizer
        self.scaler = FP8GradScaler(enabled=self.config.use_loss_scaling)
        self.context = FP8Context(self.model)

    def training_step(self, loss_fn, *inputs) -> torch.Tensor:
        loss = loss_fn(self.model, *inputs)
        self.scaler.scale(loss).backward()
        self.scaler.unscale_(self.optimizer)
        self.scaler.step(self.optimizer)
        self.scaler.update()
        self.optimizer.zero_grad(set_to_none=True)
        self.context.invalidate_caches()
        return loss.detach()


__all__ = ["FP8Spec", "E4M3", "E5M2", "quantize_block_e4m3", "quantize_block_e5m2", "dequantize_block", "AmaxHistory",
           "PerTensorDynamicScaler", "FP8GradScaler", "FP8GradientAccumulator", "FP8LinearFunction", "FP8Linear",
           "DEFAULT_FP8_EXCLUDE_PATTERNS", "should_convert_to_fp8", "convert_linear_to_fp8", "convert_model_to_fp8",
           "apply_fp8_to_huggingface_model", "FP8Context", "SmoothSwiGLU", "replace_swiglu_with_smooth",
           "fp8_flash_attention_forward", "FP8TrainingConfig", "FP8Trainer", "compute_fp8_memory_savings", "FP8Format"]
