"""chronicals_b200: a Blackwell-native LLM fine-tuning framework.

Public surface follows the reference package (chronicals/__init__.py:29-72):
lazily exported ``ChronicalsTrainer``, ``ChronicalsConfig``, ``LoRAPlusOptimizer``,
``SequencePacker`` plus ``get_version``, ``get_device_info``, ``print_info``.
"""
from __future__ import annotations

import importlib
from typing import Any, Dict

__version__ = "0.1.0"

_LAZY = {
    "ChronicalsTrainer": ("chronicals_b200.training.chronicals_trainer", "ChronicalsTrainer"),
    "TrainerState": ("chronicals_b200.training.chronicals_trainer", "TrainerState"),
    "ChronicalsConfig": ("chronicals_b200.config.config", "ChronicalsConfig"),
    "TrainingConfig": ("chronicals_b200.config.config", "TrainingConfig"),
    "ParallelConfig": ("chronicals_b200.config.config", "ParallelConfig"),
    "LoRAPlusOptimizer": ("chronicals_b200.optimizers.lora_plus_optimizer", "LoRAPlusOptimizer"),
    "LoRAPlusAdamW": ("chronicals_b200.optimizers.lora_plus_optimizer", "LoRAPlusAdamW"),
    "FusedAdamW": ("chronicals_b200.optimizers.fused_adamw", "FusedAdamW"),
    "SequencePacker": ("chronicals_b200.data.sequence_packer", "SequencePacker"),
    "PackedBatch": ("chronicals_b200.data.sequence_packer", "PackedBatch"),
    "CausalLM": ("chronicals_b200.models.decoder", "CausalLM"),
    "build_model": ("chronicals_b200.models.decoder", "build_model"),
}

__all__ = list(_LAZY) + ["get_version", "get_device_info", "print_info", "__version__"]


def __getattr__(name: str) -> Any:
    if name in _LAZY:
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'chronicals_b200' has no attribute {name!r}")


def get_version() -> str:
    return __version__


def get_device_info() -> Dict[str, Any]:
    import torch
    from .ops import _ext
    info: Dict[str, Any] = {
        "cuda_available": torch.cuda.is_available(),
        "triton_available": False,          # this framework does not use Triton
        "kernels_built": _ext.available(),
        "torch_version": torch.__version__,
        "device_count": torch.cuda.device_count() if torch.cuda.is_available() else 0,
    }
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        info.update(device_name=p.name, compute_capability=f"{p.major}.{p.minor}",
                    total_memory_gb=p.total_memory / 2**30, sm_count=p.multi_processor_count)
    return info


def print_info() -> None:
    print(f"chronicals_b200 {__version__}")
    for k, v in get_device_info().items():
        print(f"  {k}: {v}")
