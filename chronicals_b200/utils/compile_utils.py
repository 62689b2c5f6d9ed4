"""Compilation settings and LoRA adapter hot-swapping.

Reference: chronicals/utils/compile_utils.py:83-98 ``get_compile_info``, :105-186 ``CompileConfig``,
:193-286 ``GraphBreakPrevention``, :293-473 ``LoRAHotswapManager`` (swap adapter weights in place from
``adapter_model.safetensors`` without rebuilding the model), :480-699 ``CompiledLoRAModel``, :706-779
helpers.  This framework has no tracing compiler on its hot path: "compiling" a model here means
capturing its training step in a CUDA graph, and because adapters are swapped by copying into the
existing parameter tensors, a captured graph stays valid across swaps.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.nn as nn


def get_compile_info() -> Dict[str, Any]:
    return {"torch_version": torch.__version__, "torch_compile_used": False,
            "step_capture": "CUDA graph (torch.cuda.CUDAGraph)", "cuda": torch.cuda.is_available()}


@dataclass
class CompileConfig:
    """Kept for signature compatibility; only ``use_cuda_graphs`` and ``warmup_steps`` have an effect."""
    enabled: bool = True
    mode: str = "default"
    fullgraph: bool = False
    backend: str = "cuda_graph"
    dynamic: Optional[bool] = None
    use_cuda_graphs: bool = True
    warmup_steps: int = 3
    options: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def for_training(cls) -> "CompileConfig":
        return cls(mode="default", use_cuda_graphs=True)

    @classmethod
    def for_inference(cls) -> "CompileConfig":
        return cls(mode="max-autotune", use_cuda_graphs=True, warmup_steps=1)

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.__dict__)


class GraphBreakPrevention:
    """Checks the conditions under which a training step can be replayed from one CUDA graph."""

    @staticmethod
    def check(model: nn.Module, batch: Optional[Dict[str, Any]] = None) -> List[str]:
        problems = []
        if not torch.cuda.is_available():
            problems.append("no CUDA device")
        if not hasattr(model, "hf_state_dict"):
            problems.append("model is not a native packed-layout model (host-side control flow is unknown)")
        if batch is not None and isinstance(batch.get("cu_seqlens"), torch.Tensor) and not batch["cu_seqlens"].is_cuda:
            problems.append("cu_seqlens is on the host: shapes are static only if every batch has the same document count")
        return problems

    @staticmethod
    def make_static(batch: Dict[str, Any], max_documents: int) -> Dict[str, Any]:
        """Pad ``cu_seqlens`` to ``max_documents + 1`` entries (repeating the end offset = empty
        documents) so every batch has the same tensor shapes."""
        cu = batch.get("cu_seqlens")
        if isinstance(cu, torch.Tensor) and cu.numel() < max_documents + 1:
            pad = cu[-1:].expand(max_documents + 1 - cu.numel())
            batch = dict(batch, cu_seqlens=torch.cat((cu, pad)))
        return batch


class LoRAHotswapManager:
    """Swap adapter weights in place.  ``register`` loads an adapter directory (PEFT layout) into host
    memory once; ``swap`` copies its tensors into the model's existing LoRA parameters."""

    def __init__(self, model: nn.Module):
        self.model = model
        self.adapters: Dict[str, Dict[str, torch.Tensor]] = {}
        self.active: Optional[str] = None

    def _targets(self) -> Dict[str, torch.Tensor]:
        if hasattr(self.model, "hf_state_dict"):
            return {k: v for k, v in self.model.hf_state_dict(include_lora=True).items() if "lora_" in k}
        return {k: v for k, v in self.model.state_dict().items() if "lora_" in k}

    def register(self, name: str, adapter_dir_or_state) -> int:
        if isinstance(adapter_dir_or_state, dict):
            sd = adapter_dir_or_state
        else:
            path = os.path.join(adapter_dir_or_state, "adapter_model.safetensors")
            if os.path.exists(path):
                from safetensors.torch import load_file
                sd = load_file(path)
            else:
                sd = torch.load(os.path.join(adapter_dir_or_state, "adapter_model.bin"), map_location="cpu", weights_only=True)
        clean = {}
        for k, v in sd.items():
            k = k[len("base_model.model."):] if k.startswith("base_model.model.") else k
            clean[k.replace(".default", "")] = v
        self.adapters[name] = clean
        return len(clean)

    @torch.no_grad()
    def swap(self, name: str, strict: bool = True) -> int:
        sd = self.adapters[name]
        n = 0
        for k, dst in self._targets().items():
            src = sd.get(k)
            if src is None:
                if strict:
                    raise KeyError(f"adapter {name!r} has no tensor for {k}")
                continue
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"adapter {name!r}: shape of {k} is {tuple(src.shape)}, model has {tuple(dst.shape)} "
                                 "(hot-swapping needs equal ranks)")
            dst.copy_(src.to(dst.dtype))
            n += 1
        self.active = name
        return n

    _manual_weight_swap = swap


class CompiledLoRAModel(nn.Module):
    """Model + hot-swap manager; ``forward`` is the model's, adapters change without re-capture."""

    def __init__(self, model: nn.Module, config: Optional[CompileConfig] = None):
        super().__init__()
        self.model = model
        self.config = config or CompileConfig()
        self.hotswap = LoRAHotswapManager(model)

    def forward(self, *a, **kw):
        return self.model(*a, **kw)

    def load_adapter(self, name: str, path_or_state, activate: bool = True) -> None:
        self.hotswap.register(name, path_or_state)
        if activate:
            self.hotswap.swap(name)

    def set_adapter(self, name: str) -> None:
        self.hotswap.swap(name)


def compile_model_with_lora(model: nn.Module, config: Optional[CompileConfig] = None) -> CompiledLoRAModel:
    return CompiledLoRAModel(model, config)


def get_optimal_compile_mode(model_size_b: float = 0.5, training: bool = True) -> str:
    """The reference picks a torch.compile mode; the equivalent decision here is whether to capture
    the step in a CUDA graph (yes when the step is launch-bound, i.e. for small models)."""
    return "cuda_graph" if model_size_b <= 3 else "eager"
