"""Hardware detection and per-GPU LoRA hyper-parameter presets.

Reference: chronicals/lora/lora_presets.py:50-224 (``GPUType``, ``GPUSpec``, detection),
:231-299 ``LoRAPreset``, :306-557 per-GPU tables and registry, :564-761 selection helpers.
The tables stop at H100 in the reference; B200 presets are added.  ``expected_tokens_per_sec``
is an expectation used to size runs, not a measurement.
"""
from __future__ import annotations

import re
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional

import torch


class GPUType(Enum):
    T4 = "t4"
    A10G = "a10g"
    L4 = "l4"
    A100_40GB = "a100_40gb"
    A100_80GB = "a100_80gb"
    H100 = "h100"
    B200 = "b200"
    UNKNOWN = "unknown"


@dataclass
class GPUSpec:
    name: str
    memory_gb: float
    bf16_tflops: float
    bandwidth_gbs: float
    supports_bf16: bool = True
    supports_fp8: bool = False


GPU_SPECS: Dict[GPUType, GPUSpec] = {
    GPUType.T4: GPUSpec("T4", 16, 65, 320, supports_bf16=False),
    GPUType.A10G: GPUSpec("A10G", 24, 125, 600),
    GPUType.L4: GPUSpec("L4", 24, 121, 300, supports_fp8=True),
    GPUType.A100_40GB: GPUSpec("A100-40GB", 40, 312, 1555),
    GPUType.A100_80GB: GPUSpec("A100-80GB", 80, 312, 2039),
    GPUType.H100: GPUSpec("H100", 80, 989, 3350, supports_fp8=True),
    GPUType.B200: GPUSpec("B200", 180, 2250, 7700, supports_fp8=True),
    GPUType.UNKNOWN: GPUSpec("unknown", 16, 50, 300),
}


def detect_gpu(name: Optional[str] = None, memory_gb: Optional[float] = None) -> GPUType:
    if name is None:
        if not torch.cuda.is_available():
            return GPUType.UNKNOWN
        p = torch.cuda.get_device_properties(0)
        name, memory_gb = p.name, p.total_memory / 2**30
    n = name.upper()
    if "B200" in n or "B100" in n or "GB200" in n:
        return GPUType.B200
    if "H100" in n or "H200" in n:
        return GPUType.H100
    if "A100" in n:
        return GPUType.A100_80GB if (memory_gb or 40) > 60 else GPUType.A100_40GB
    if "A10" in n:
        return GPUType.A10G
    if re.search(r"\bL4\b", n):
        return GPUType.L4
    if "T4" in n:
        return GPUType.T4
    return GPUType.UNKNOWN


def detect_hardware() -> Dict[str, Any]:
    t = detect_gpu()
    return {"gpu_type": t, "spec": GPU_SPECS[t], "num_gpus": torch.cuda.device_count() if torch.cuda.is_available() else 0}


@dataclass
class LoRAPreset:
    name: str = "default"
    rank: int = 16
    alpha: float = 32.0
    dropout: float = 0.0
    target_modules: List[str] = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                               "up_proj", "down_proj"])
    batch_size: int = 4
    gradient_accumulation_steps: int = 4
    max_seq_length: int = 512
    learning_rate: float = 2e-4
    use_lora_plus: bool = True
    lora_plus_ratio: float = 16.0
    use_gradient_checkpointing: bool = True
    use_sequence_packing: bool = True
    use_cuda_graphs: bool = False
    precision: str = "bf16"
    expected_tokens_per_sec: int = 0
    expected_memory_gb: float = 0.0

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def to_training_config(self):
        from ..config.config import TrainingConfig
        cfg = TrainingConfig(per_device_train_batch_size=self.batch_size,
                             gradient_accumulation_steps=self.gradient_accumulation_steps,
                             max_seq_length=self.max_seq_length, learning_rate=self.learning_rate,
                             use_gradient_checkpointing=self.use_gradient_checkpointing,
                             use_sequence_packing=self.use_sequence_packing, use_cuda_graphs=self.use_cuda_graphs,
                             bf16=self.precision == "bf16", fp8=False)
        cfg.use_lora, cfg.lora_rank, cfg.lora_alpha = True, self.rank, self.alpha
        cfg.use_lora_plus, cfg.lora_plus_ratio = self.use_lora_plus, self.lora_plus_ratio
        cfg.lora_target_modules = list(self.target_modules)
        return cfg


def _p(name, size, **kw) -> LoRAPreset:
    return LoRAPreset(name=f"{name}-{size}", **kw)


# per GPU: model-size class → preset (expected throughput figures for the older GPUs are the reference's own)
PRESETS: Dict[GPUType, Dict[str, LoRAPreset]] = {
    GPUType.T4: {
        "0.5b": _p("t4", "0.5b", rank=16, batch_size=2, max_seq_length=512, precision="fp16", expected_tokens_per_sec=8000),
        "1b": _p("t4", "1b", rank=8, batch_size=1, max_seq_length=512, precision="fp16", expected_tokens_per_sec=5000),
        "3b": _p("t4", "3b", rank=8, batch_size=1, max_seq_length=256, precision="fp16", expected_tokens_per_sec=2000),
    },
    GPUType.A10G: {
        "0.5b": _p("a10g", "0.5b", batch_size=4, expected_tokens_per_sec=15000),
        "1b": _p("a10g", "1b", batch_size=4, expected_tokens_per_sec=10000),
        "3b": _p("a10g", "3b", batch_size=2, expected_tokens_per_sec=6000),
        "7b": _p("a10g", "7b", rank=8, batch_size=1, expected_tokens_per_sec=3000),
    },
    GPUType.L4: {
        "0.5b": _p("l4", "0.5b", batch_size=4, expected_tokens_per_sec=12000),
        "3b": _p("l4", "3b", batch_size=2, expected_tokens_per_sec=5000),
    },
    GPUType.A100_40GB: {
        "0.5b": _p("a100-40", "0.5b", rank=32, batch_size=8, max_seq_length=1024, expected_tokens_per_sec=35000),
        "1b": _p("a100-40", "1b", rank=32, batch_size=8, max_seq_length=1024, expected_tokens_per_sec=25000),
        "3b": _p("a100-40", "3b", batch_size=4, max_seq_length=1024, expected_tokens_per_sec=15000),
        "7b": _p("a100-40", "7b", batch_size=2, max_seq_length=1024, expected_tokens_per_sec=8000),
    },
    GPUType.A100_80GB: {
        "0.5b": _p("a100-80", "0.5b", rank=64, batch_size=16, max_seq_length=2048, expected_tokens_per_sec=50000),
        "1b": _p("a100-80", "1b", rank=32, batch_size=16, max_seq_length=2048, expected_tokens_per_sec=35000),
        "3b": _p("a100-80", "3b", rank=32, batch_size=8, max_seq_length=2048, expected_tokens_per_sec=20000),
        "7b": _p("a100-80", "7b", batch_size=4, max_seq_length=2048, expected_tokens_per_sec=10000),
        "13b": _p("a100-80", "13b", batch_size=2, max_seq_length=1024, expected_tokens_per_sec=5000),
    },
    GPUType.H100: {
        "0.5b": _p("h100", "0.5b", rank=64, batch_size=16, max_seq_length=2048, use_gradient_checkpointing=False,
                   expected_tokens_per_sec=100000),
        "1b": _p("h100", "1b", rank=64, batch_size=16, max_seq_length=2048, expected_tokens_per_sec=70000),
        "7b": _p("h100", "7b", rank=32, batch_size=4, max_seq_length=2048, expected_tokens_per_sec=20000),
    },
    GPUType.B200: {
        "0.5b": _p("b200", "0.5b", rank=16, batch_size=8, gradient_accumulation_steps=1, max_seq_length=4096,
                   use_gradient_checkpointing=False, use_cuda_graphs=True, expected_tokens_per_sec=200000),
        "1b": _p("b200", "1b", rank=32, batch_size=8, gradient_accumulation_steps=1, max_seq_length=4096,
                 use_gradient_checkpointing=False, use_cuda_graphs=True, expected_tokens_per_sec=120000),
        "7b": _p("b200", "7b", rank=32, batch_size=4, gradient_accumulation_steps=1, max_seq_length=4096,
                 use_gradient_checkpointing=False, expected_tokens_per_sec=30000),
        "13b": _p("b200", "13b", rank=32, batch_size=2, gradient_accumulation_steps=2, max_seq_length=4096,
                  expected_tokens_per_sec=15000),
    },
}
PRESETS[GPUType.UNKNOWN] = PRESETS[GPUType.T4]
PRESET_REGISTRY: Dict[str, LoRAPreset] = {p.name: p for d in PRESETS.values() for p in d.values()}


def get_model_size(model_or_name) -> str:
    """Size class ("0.5b", "1b", "3b", "7b", "13b") from a parameter count or a model name."""
    if isinstance(model_or_name, str):
        m = re.search(r"(\d+(?:\.\d+)?)\s*b", model_or_name.lower())
        n = float(m.group(1)) * 1e9 if m else 1e9
    elif isinstance(model_or_name, (int, float)):
        n = float(model_or_name)
    else:
        n = float(sum(p.numel() for p in model_or_name.parameters()))
    for cls, lim in (("0.5b", 0.8e9), ("1b", 2e9), ("3b", 5e9), ("7b", 10e9)):
        if n < lim:
            return cls
    return "13b"


def get_preset_for_hardware(gpu_type: Optional[GPUType] = None, model_size: str = "0.5b") -> LoRAPreset:
    t = gpu_type or detect_gpu()
    table = PRESETS.get(t, PRESETS[GPUType.UNKNOWN])
    order = ["0.5b", "1b", "3b", "7b", "13b"]
    i = order.index(model_size) if model_size in order else 0
    for k in order[i:] + order[:i][::-1]:
        if k in table:
            return table[k]
    return next(iter(table.values()))


def get_optimal_preset(model_or_name=None, gpu_name: Optional[str] = None) -> LoRAPreset:
    t = detect_gpu(gpu_name) if gpu_name else detect_gpu()
    return get_preset_for_hardware(t, get_model_size(model_or_name if model_or_name is not None else "0.5b"))


def get_optimization_recommendations(gpu_type: Optional[GPUType] = None, model_size: str = "0.5b") -> List[str]:
    t = gpu_type or detect_gpu()
    spec = GPU_SPECS[t]
    rec = []
    if not spec.supports_bf16:
        rec.append("use fp16 with loss scaling (no bf16 tensor cores)")
    if spec.memory_gb >= 80 and model_size in ("0.5b", "1b", "3b"):
        rec.append("disable gradient checkpointing: activations fit")
    if t == GPUType.B200:
        rec.append("enable CUDA-graph step capture and sequence packing; MXFP8 GEMMs for 7B and larger")
    if spec.memory_gb <= 24:
        rec.append("rank 8, micro-batch 1-2, gradient checkpointing on")
    rec.append("LoRA+ with lr_ratio 16 (B matrices learn faster)")
    return rec


def compare_presets(names: List[str]) -> List[Dict[str, Any]]:
    return [PRESET_REGISTRY[n].to_dict() for n in names if n in PRESET_REGISTRY]


def list_all_presets() -> List[str]:
    return sorted(PRESET_REGISTRY)
