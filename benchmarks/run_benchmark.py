"""Benchmark suite: full fine-tune and LoRA throughput of this framework against baselines.

Reference: benchmarks/run_benchmark.py (``BenchmarkResult`` :70-106, ``CUDATimer`` :155-207,
``MultiRunTimer`` :210-244, ``find_optimal_batch_size`` :246-376, ``compute_mfu`` :379-407,
``benchmark_chronicals`` :819-1260, ``benchmark_chronicals_lora`` :1878-2228, micro-benchmarks
:2611-2948, ``benchmark_with_cuda_graphs`` :2951-3091, ``print_comparison`` :3094-3195, CLI :3198-3768).

Differences by design: there is no network here, so data is a seeded synthetic instruction-length
distribution and models are random-initialised from a named architecture; baselines that need
packages which are not installed (Unsloth, Liger) are reported as ``skipped`` with the reason.
Methods: ``chronicals`` (this framework's trainer), ``chronicals_lora``, ``chronicals_eager`` (no CUDA
graph), ``huggingface`` (transformers model + torch fused AdamW), ``native_pytorch`` (this framework's
model definition executed by plain PyTorch ops in fp32-free bf16 through the oracle formulas).

Every number is device-timed with CUDA events after warm-up.  ``python benchmarks/run_benchmark.py
--methods chronicals huggingface --steps 20`` prints a table and writes JSON with a methodology block.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

B200_DENSE_BF16_TFLOPS = 2250.0          # nominal dense bf16 peak used for MFU
TARGET_TOKENS_PER_SEC = 50_000.0         # the reference's stated A100 target, kept for the gap report
PUBLISHED = {"chronicals_full_ft_a100": 41_184.0, "chronicals_lora_a100": 11_699.0, "unsloth_full_ft_a100": 11_736.0}


@dataclass
class BenchmarkResult:
    method: str
    status: str = "ok"                    # ok | skipped | failed
    reason: str = ""
    tokens_per_sec: float = 0.0
    ms_per_step: float = 0.0
    ms_per_step_std: float = 0.0
    mfu: float = 0.0
    peak_memory_gb: float = 0.0
    batch_size: int = 0
    seq_length: int = 0
    steps: int = 0
    final_loss: float = float("nan")
    n_params: int = 0
    trainable_params: int = 0
    extra: Dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


class CUDATimer:
    """Device time of a region from CUDA events (wall clock on CPU)."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        self.ms = 0.0

    def __enter__(self):
        if self.cuda:
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            self.a.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self.b.record()
            torch.cuda.synchronize()
            self.ms = self.a.elapsed_time(self.b)
        else:
            self.ms = 1e3 * (time.perf_counter() - self.t0)
        return False


class MultiRunTimer:
    """Repeat a measurement and report mean / std / min."""

    def __init__(self, num_runs: int = 3):
        self.num_runs = num_runs
        self.samples: List[float] = []

    def run(self, fn: Callable[[], float]) -> "MultiRunTimer":
        self.samples = [float(fn()) for _ in range(self.num_runs)]
        return self

    @property
    def mean(self) -> float:
        return statistics.fmean(self.samples) if self.samples else 0.0

    @property
    def std(self) -> float:
        return statistics.pstdev(self.samples) if len(self.samples) > 1 else 0.0

    @property
    def best(self) -> float:
        return min(self.samples) if self.samples else 0.0


def compute_mfu(n_params: int, tokens_per_sec: float, peak_tflops: float = B200_DENSE_BF16_TFLOPS) -> float:
    """Model FLOPs utilisation with the 6·N·tokens approximation (forward + backward)."""
    return 6.0 * n_params * tokens_per_sec / (peak_tflops * 1e12)


def find_optimal_batch_size(step_fn: Callable[[int], None], start: int = 1, limit: int = 256,
                            memory_fraction: float = 0.9) -> int:
    """Largest power-of-two micro-batch whose step fits in ``memory_fraction`` of device memory.
    ``step_fn(batch)`` must run one full training step.  Doubling stops at the first failure."""
    best, b = 0, start
    total = torch.cuda.get_device_properties(0).total_memory if torch.cuda.is_available() else 0
    while b <= limit:
        try:
            if torch.cuda.is_available():
                torch.cuda.reset_peak_memory_stats()
            step_fn(b)
            if total and torch.cuda.max_memory_allocated() > memory_fraction * total:
                break
            best = b
            b *= 2
        except RuntimeError as e:                       # out of memory ends the search
            if "out of memory" not in str(e).lower():
                raise
            torch.cuda.empty_cache()
            break
    return max(best, start)


def synthetic_instruction_lengths(n: int, seed: int = 0, mean_tokens: float = 180.0, max_len: int = 1024) -> List[int]:
    """Log-normal lengths resembling instruction-tuning corpora (median ≈ 150 tokens, long tail)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.exp(torch.randn(n, generator=g) * 0.7 + math.log(mean_tokens) - 0.245)
    return [int(v) for v in x.clamp(8, max_len).tolist()]


def load_alpaca_dataloader(vocab_size: int, batch_size: int, seq_length: int, n_batches: int, seed: int = 0,
                           packed: bool = False) -> List[Dict[str, torch.Tensor]]:
    """Batches shaped like a tokenised instruction dataset.  ``packed=False``: dense ``[B, S]`` rows of
    uniform random ids (the headline configuration); ``packed=True``: documents with synthetic lengths
    packed into rows with position ids and document boundaries."""
    g = torch.Generator().manual_seed(seed)
    out = []
    if not packed:
        for _ in range(n_batches):
            ids = torch.randint(0, vocab_size, (batch_size, seq_length), generator=g)
            out.append({"input_ids": ids, "labels": ids.clone()})
        return out
    from chronicals_b200.data.sequence_packer import SequencePacker
    need = n_batches * batch_size
    packer = SequencePacker(max_seq_length=seq_length, strategy="bfd")
    lens = synthetic_instruction_lengths(need * max(4, seq_length // 150), seed, max_len=seq_length)
    docs = [torch.randint(0, vocab_size, (L,), generator=g).tolist() for L in lens]
    rows = packer.pack_all_sequences(docs)[:need]
    for i in range(0, len(rows) - batch_size + 1, batch_size):
        chunk = rows[i:i + batch_size]
        # one flat row of B*S tokens: document boundaries are recovered from the position ids
        out.append({k: torch.cat([getattr(r, k).reshape(-1) for r in chunk]).unsqueeze(0)
                    for k in ("input_ids", "labels", "position_ids")})
    return out


# ------------------------------------------------------------------------------------------------ methods
def _device() -> torch.device:
    return torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")


def _training_config(a, **over):
    from chronicals_b200 import TrainingConfig
    kw = dict(output_dir=os.path.join("/tmp", f"cb_suite_{os.getpid()}"), per_device_train_batch_size=a.batch_size,
              max_seq_length=a.seq_length, gradient_accumulation_steps=a.grad_accum, learning_rate=2e-5,
              weight_decay=0.01, max_grad_norm=1.0, lr_scheduler_type="constant", warmup_ratio=0.0, bf16=True,
              fp8=False, use_gradient_checkpointing=False, use_sequence_packing=False, logging_steps=10 ** 9,
              save_steps=0, visual_reporting=False, use_cuda_graphs=a.use_cuda_graphs and a.grad_accum == 1, seed=0)
    kw.update(over)
    cfg = TrainingConfig(**kw)
    cfg.save_final = False
    cfg.log_jsonl = False
    return cfg


def _time_steps(step: Callable[[int], Any], a, tokens_per_step: int) -> Dict[str, float]:
    """Warm up, then time ``a.steps`` steps ``a.num_runs`` times; the best run is reported."""
    for i in range(a.warmup_steps):
        step(i)
    runs = []
    last = None
    for _ in range(a.num_runs):
        with CUDATimer() as t:
            for i in range(a.steps):
                last = step(i)
        runs.append(t.ms / a.steps)
    best = min(runs)
    loss = float(last.detach().float().item()) if isinstance(last, torch.Tensor) else float("nan")
    return {"ms": best, "std": statistics.pstdev(runs) if len(runs) > 1 else 0.0,
            "tok_s": tokens_per_step / (best / 1e3), "loss": loss}


def _finish(method: str, a, n_params: int, trainable: int, t: Dict[str, float], **extra) -> BenchmarkResult:
    mem = torch.cuda.max_memory_allocated() / 2 ** 30 if torch.cuda.is_available() else 0.0
    return BenchmarkResult(method=method, tokens_per_sec=t["tok_s"], ms_per_step=t["ms"], ms_per_step_std=t["std"],
                           mfu=compute_mfu(n_params, t["tok_s"]), peak_memory_gb=mem, batch_size=a.batch_size,
                           seq_length=a.seq_length, steps=a.steps, final_loss=t["loss"], n_params=n_params,
                           trainable_params=trainable, extra=extra)


def benchmark_chronicals(a, lora: bool = False, graphs: Optional[bool] = None, packed: bool = False) -> BenchmarkResult:
    """This framework's trainer on its own decoder (full fine-tune, or LoRA r=16 with LoRA+)."""
    from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, build_model
    dev = _device()
    cfg = ChronicalsConfig.from_model_name(a.model)
    model = build_model(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev, seed=0)
    over: Dict[str, Any] = {}
    if graphs is not None:
        over["use_cuda_graphs"] = graphs and a.grad_accum == 1
    if lora:
        from chronicals_b200.lora import apply_lora_to_model
        apply_lora_to_model(model, rank=a.lora_rank, alpha=2.0 * a.lora_rank)
        over.update(optimizer_type="lora_plus", learning_rate=2e-4, lora_plus_lr_ratio=16.0, weight_decay=0.0)
    n_params = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    targs = _training_config(a, **over)
    trainer = ChronicalsTrainer(model, targs, None)
    data = load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 4, seed=0, packed=packed)
    data = [{k: v.to(dev) for k, v in b.items()} for b in data]
    t = _time_steps(lambda i: trainer.training_step(data[i % len(data)]), a, a.batch_size * a.seq_length)
    name = "chronicals_lora" if lora else ("chronicals" if targs.use_cuda_graphs else "chronicals_eager")
    if packed:
        name += "_packed"
    return _finish(name, a, n_params, trainable, t, cuda_graph=bool(trainer.use_cuda_graphs), lora_rank=a.lora_rank if lora else 0)


def benchmark_chronicals_lora(a) -> BenchmarkResult:
    return benchmark_chronicals(a, lora=True)


def benchmark_with_cuda_graphs(a) -> BenchmarkResult:
    return benchmark_chronicals(a, graphs=True)


def benchmark_native_pytorch(a) -> BenchmarkResult:
    """The same decoder executed by stock PyTorch operators (the oracle formulas): fp32 master-free bf16
    matmuls through cuBLAS, SDPA attention, unfused elementwise ops, chunked cross-entropy, torch AdamW."""
    from chronicals_b200 import ChronicalsConfig, build_model
    from chronicals_b200.ops import _ext
    dev = _device()
    cfg = ChronicalsConfig.from_model_name(a.model)
    model = build_model(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev, seed=0)
    n_params = sum(p.numel() for p in model.parameters())
    opt = torch.optim.AdamW(model.parameters(), lr=2e-5, weight_decay=0.01, fused=dev.type == "cuda")
    data = load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 4, seed=0)
    data = [{k: v.to(dev) for k, v in b.items()} for b in data]

    def step(i):
        with _ext.force_reference():
            loss = model(data[i % len(data)]["input_ids"], labels=data[i % len(data)]["labels"]).loss
            loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss
    t = _time_steps(step, a, a.batch_size * a.seq_length)
    return _finish("native_pytorch", a, n_params, n_params, t)


def benchmark_huggingface(a) -> BenchmarkResult:
    """transformers' implementation of the same architecture (random init), SDPA attention, torch fused AdamW."""
    try:
        import transformers
        from chronicals_b200 import ChronicalsConfig
    except Exception as e:                               # pragma: no cover
        return BenchmarkResult("huggingface", status="skipped", reason=f"transformers not importable: {e}")
    dev = _device()
    cfg = ChronicalsConfig.from_model_name(a.model)
    hf_cfg = transformers.Qwen2Config(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads, max_position_embeddings=max(cfg.max_position_embeddings, a.seq_length),
        rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, tie_word_embeddings=cfg.tie_word_embeddings,
        attn_implementation="sdpa")
    torch.manual_seed(0)
    model = transformers.AutoModelForCausalLM.from_config(hf_cfg).to(dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    n_params = sum(p.numel() for p in model.parameters())
    opt = torch.optim.AdamW(model.parameters(), lr=2e-5, weight_decay=0.01, fused=dev.type == "cuda")
    data = load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 4, seed=0)
    data = [{k: v.to(dev) for k, v in b.items()} for b in data]

    def step(i):
        loss = model(**data[i % len(data)]).loss
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss
    t = _time_steps(step, a, a.batch_size * a.seq_length)
    return _finish("huggingface", a, n_params, n_params, t, transformers=transformers.__version__)


def _skipped(name: str, package: str) -> Callable[[Any], BenchmarkResult]:
    def run(a) -> BenchmarkResult:
        try:
            __import__(package)
        except Exception as e:
            return BenchmarkResult(name, status="skipped", reason=f"{package} is not installed ({type(e).__name__})")
        return BenchmarkResult(name, status="skipped", reason=f"{package} baseline needs network access for its model hub")
    return run


METHODS: Dict[str, Callable[[Any], BenchmarkResult]] = {
    "chronicals": benchmark_chronicals,
    "chronicals_eager": lambda a: benchmark_chronicals(a, graphs=False),
    "chronicals_packed": lambda a: benchmark_chronicals(a, packed=True),
    "chronicals_lora": benchmark_chronicals_lora,
    "huggingface": benchmark_huggingface,
    "native_pytorch": benchmark_native_pytorch,
    "unsloth": _skipped("unsloth", "unsloth"),
    "liger": _skipped("liger", "liger_kernel"),
}
