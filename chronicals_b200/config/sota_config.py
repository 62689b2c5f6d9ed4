"""Performance model, presets and diagnostics.

Reference: chronicals/config/sota_config.py:76-175 ``TheoreticalPerformance``, :182-223
``OPTIMIZATION_SYNERGY``, :230-504 ``MaxPerformanceConfig``, :511-786 ``OptimizationStatus`` /
``OptimizationChecklist``, :793-854 and :1104-1262 diagnostic reports, :917-962
``BENCHMARK_COMPARISON``, :969-1032 ``get_sota_config_for_gpu``, :1039-1097 ``UNSLOTH_BENCHMARKS``,
:1269-1353 synergy checks.  The reference's tables are A100 targets; here the performance model is
computed from the model architecture and the *measured* B200 peaks, and published A100 numbers of the
reference are kept only as labelled comparison constants.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from .config import ChronicalsConfig, TrainingConfig, measured_peaks, roofline_analysis

# published by the reference for 1x A100-40GB, Qwen2.5-0.5B (its README); comparison constants only
REFERENCE_PUBLISHED = {"full_ft_tok_s": 41184.0, "lora_tok_s": 11699.0, "full_ft_mfu": 0.396, "hardware": "A100-40GB"}
UNSLOTH_BENCHMARKS = {"full_ft_tok_s": 11736.0, "lora_max_tok_s": 2857.0, "hf_peft_lora_tok_s": 3420.0,
                      "plain_pytorch_tok_s": 8240.0, "hardware": "A100-40GB", "source": "reference README"}
BENCHMARK_COMPARISON = {"reference_chronicals": REFERENCE_PUBLISHED, "unsloth": UNSLOTH_BENCHMARKS}


@dataclass
class TheoreticalPerformance:
    """Step-time floor of a dense decoder from FLOPs and bytes."""
    model: ChronicalsConfig
    tokens_per_step: int = 8192
    seq_len: int = 1024
    peak_tflops: Optional[float] = None
    hbm_gbs: Optional[float] = None

    def __post_init__(self):
        p = measured_peaks()
        self.peak_tflops = self.peak_tflops or p["bf16_tflops_sustained"]
        self.hbm_gbs = self.hbm_gbs or p["hbm_gbs"]

    def flops_per_step(self) -> Dict[str, float]:
        r = roofline_analysis(self.model, self.tokens_per_step, self.seq_len, self.peak_tflops)
        return {"gemm": r["gemm_flops"], "attention": r["attn_flops"], "total": r["gemm_flops"] + r["attn_flops"]}

    def optimizer_bytes(self) -> float:
        return self.model.num_parameters() * 22.0            # p,g,m,v read + p,m,v write (bf16 params, fp32 moments)

    def floor_seconds(self) -> float:
        return self.flops_per_step()["total"] / (self.peak_tflops * 1e12) + self.optimizer_bytes() / (self.hbm_gbs * 1e9)

    def max_tokens_per_second(self) -> float:
        return self.tokens_per_step / self.floor_seconds()

    def mfu(self, tokens_per_second: float, peak_tflops: float = 2250.0) -> float:
        return 6.0 * self.model.num_parameters() * tokens_per_second / (peak_tflops * 1e12)


# which features multiply and which overlap (qualitative; kept as data so reports can print it)
OPTIMIZATION_SYNERGY: Dict[str, Dict[str, Any]] = {
    "sequence_packing+varlen_attention": {"effect": "multiplicative", "note": "no FLOPs on padding; block skipping per document"},
    "cut_cross_entropy+large_vocab": {"effect": "memory", "note": "the [T, V] logits never exist; frees ~5 GB at V=152k, T=8192"},
    "cuda_graphs+fused_optimizer": {"effect": "multiplicative", "note": "no host sync inside a step, so the whole step replays"},
    "gradient_checkpointing+small_model": {"effect": "negative", "note": "recompute costs ~30 % and 180 GB holds the activations"},
    "fused_collectives+sharded_optimizer": {"effect": "multiplicative", "note": "AdamW runs on 1/W of the parameters per rank"},
}


@dataclass
class MaxPerformanceConfig:
    """One-call preset for maximum throughput on the detected GPU."""
    model_name: str = "qwen2.5-0.5b"
    batch_size: int = 8
    seq_length: int = 1024
    gradient_accumulation_steps: int = 1
    learning_rate: float = 2e-5
    use_cuda_graphs: bool = True
    use_sequence_packing: bool = True
    use_gradient_checkpointing: bool = False
    comm_backend: str = "fused"

    def to_training_config(self) -> TrainingConfig:
        cfg = TrainingConfig(per_device_train_batch_size=self.batch_size, max_seq_length=self.seq_length,
                             gradient_accumulation_steps=self.gradient_accumulation_steps,
                             learning_rate=self.learning_rate, use_cuda_graphs=self.use_cuda_graphs,
                             use_sequence_packing=self.use_sequence_packing,
                             use_gradient_checkpointing=self.use_gradient_checkpointing, fp8=False,
                             gpu_peak_tflops=2250.0)
        cfg.parallel.comm_backend = self.comm_backend
        return cfg


@dataclass
class OptimizationStatus:
    name: str
    enabled: bool
    available: bool = True
    note: str = ""


class OptimizationChecklist:
    """What is switched on in a ``TrainingConfig`` and whether the machine can honour it."""

    def __init__(self, config: TrainingConfig):
        from ..ops import _ext
        cuda = torch.cuda.is_available()
        built = _ext.available()
        self.items: List[OptimizationStatus] = [
            OptimizationStatus("sm_100a kernel library", built, built, "python -m chronicals_b200.csrc.build"),
            OptimizationStatus("bf16", config.bf16, cuda),
            OptimizationStatus("fused AdamW + in-kernel clipping", config.use_fused_adamw and config.optimizer_type == "fused_adamw"),
            OptimizationStatus("cut cross-entropy", config.ce_implementation in ("cce", "triton_cce", "adaptive")),
            OptimizationStatus("sequence packing", config.use_sequence_packing),
            OptimizationStatus("varlen attention", config.use_flash_varlen),
            OptimizationStatus("CUDA-graph step", config.use_cuda_graphs, cuda, "needs gradient_accumulation_steps == 1"),
            OptimizationStatus("gradient checkpointing", config.use_gradient_checkpointing, True, "costs speed; for memory only"),
            OptimizationStatus("fused collectives", config.parallel.comm_backend == "fused", cuda and torch.cuda.device_count() > 1),
        ]

    def report(self) -> str:
        lines = ["optimization checklist:"]
        for it in self.items:
            mark = "x" if it.enabled and it.available else ("!" if it.enabled else " ")
            lines.append(f"  [{mark}] {it.name}" + (f"  ({it.note})" if it.note else ""))
        return "\n".join(lines)

    def as_dict(self) -> Dict[str, bool]:
        return {it.name: bool(it.enabled and it.available) for it in self.items}


def print_diagnostic_report(config: Optional[TrainingConfig] = None) -> None:
    print(OptimizationChecklist(config or TrainingConfig()).report())


def print_comprehensive_diagnostic(config: Optional[TrainingConfig] = None, model: Optional[ChronicalsConfig] = None) -> None:
    cfg = config or TrainingConfig()
    m = model or ChronicalsConfig.from_model_name("qwen2.5-0.5b")
    print_diagnostic_report(cfg)
    tp = TheoreticalPerformance(m, cfg.per_device_train_batch_size * cfg.max_seq_length, cfg.max_seq_length)
    fl = tp.flops_per_step()
    p = measured_peaks()
    print(f"model: {m.num_parameters() / 1e6:.0f} M parameters; step of {tp.tokens_per_step} tokens = "
          f"{fl['total'] / 1e12:.1f} TFLOP ({100 * fl['attention'] / fl['total']:.1f} % attention)")
    print(f"peaks ({p['source']}): bf16 {p['bf16_tflops_sustained']:.0f} TFLOP/s sustained, HBM {p['hbm_gbs']:.0f} GB/s")
    print(f"floor: {1e3 * tp.floor_seconds():.1f} ms/step = {tp.max_tokens_per_second():,.0f} tok/s per GPU")
    print(f"published reference (A100-40GB): {REFERENCE_PUBLISHED['full_ft_tok_s']:,.0f} tok/s full fine-tune")


def get_sota_config_for_gpu(gpu_name: Optional[str] = None) -> TrainingConfig:
    from .config import get_optimal_config_for_gpu
    return get_optimal_config_for_gpu(gpu_name)


def verify_optimization_synergy(config: TrainingConfig) -> List[str]:
    """Warnings about flag combinations that work against each other."""
    w = []
    if config.use_cuda_graphs and config.gradient_accumulation_steps > 1:
        w.append("use_cuda_graphs is ignored when gradient_accumulation_steps > 1")
    if config.use_gradient_checkpointing and config.use_cuda_graphs:
        w.append("gradient checkpointing inside a captured step is allowed but pointless for small models")
    if not config.use_sequence_packing and config.use_flash_varlen:
        w.append("varlen attention without packing computes on padding")
    if config.parallel.comm_backend == "fused" and config.optimizer_type != "fused_adamw":
        w.append("fused collectives are implemented for the fused AdamW / LoRA+ optimizers only")
    return w


def print_synergy_report(config: Optional[TrainingConfig] = None) -> None:
    for k, v in OPTIMIZATION_SYNERGY.items():
        print(f"  {k}: {v['effect']} — {v['note']}")
    for w in verify_optimization_synergy(config or TrainingConfig()):
        print("  warning:", w)


@dataclass
class IntegrationTestConfig:
    """Tiny settings used by smoke tests."""
    model_name: str = "tiny-qwen2"
    steps: int = 5
    batch_size: int = 2
    seq_length: int = 128
