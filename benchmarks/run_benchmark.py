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
        over.update(optimizer_type="lora_plus", learning_rate=2e-4, weight_decay=0.0)
    n_params = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    targs = _training_config(a, **over)
    if lora:
        targs.lora_plus_ratio = 16.0
    trainer = ChronicalsTrainer(model, targs, None)
    data = load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 4, seed=0, packed=packed)
    data = [{k: v.to(dev) for k, v in b.items()} for b in data]
    t = _time_steps(lambda i: trainer.training_step(data[i % len(data)]), a, a.batch_size * a.seq_length)   # one micro-step
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


class _PlainLoRALinear(torch.nn.Module):
    """``nn.Linear`` with a frozen weight and a rank-r adapter, written with stock PyTorch operators only
    (what PEFT's ``LoraLayer`` computes): ``y = W x + (alpha / r) * B (A x)``."""

    def __init__(self, base: torch.nn.Linear, rank: int, alpha: float):
        super().__init__()
        self.base = base
        for p in self.base.parameters():
            p.requires_grad_(False)
        dev, dt = base.weight.device, base.weight.dtype
        self.lora_A = torch.nn.Parameter(torch.empty(rank, base.in_features, device=dev, dtype=dt))
        self.lora_B = torch.nn.Parameter(torch.zeros(base.out_features, rank, device=dev, dtype=dt))
        torch.nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.scaling = alpha / rank

    def forward(self, x):
        return self.base(x) + torch.nn.functional.linear(torch.nn.functional.linear(x, self.lora_A), self.lora_B) * self.scaling


def benchmark_huggingface_lora(a) -> BenchmarkResult:
    """The library baseline of the LoRA comparison that runs offline: transformers' implementation of the same
    architecture (random init, SDPA attention) with plain PyTorch LoRA modules (rank / alpha as in the other LoRA
    methods, all seven projections), frozen base, torch fused AdamW on the adapters.  It stands where the
    reference's suite puts Unsloth / PEFT, which need a model hub."""
    try:
        import transformers
        from chronicals_b200 import ChronicalsConfig
    except Exception as e:                               # pragma: no cover
        return BenchmarkResult("huggingface_lora", status="skipped", reason=f"transformers not importable: {e}")
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
    for p in model.parameters():
        p.requires_grad_(False)
    targets = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
    for module in list(model.modules()):
        for name, child in list(module.named_children()):
            if name in targets and isinstance(child, torch.nn.Linear):
                setattr(module, name, _PlainLoRALinear(child, a.lora_rank, 2.0 * a.lora_rank))
    n_params = sum(p.numel() for p in model.parameters())
    adapters = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(adapters, lr=2e-4, weight_decay=0.0, fused=dev.type == "cuda")
    data = load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 4, seed=0)
    data = [{k: v.to(dev) for k, v in b.items()} for b in data]

    def step(i):
        loss = model(**data[i % len(data)]).loss
        loss.backward()
        torch.nn.utils.clip_grad_norm_(adapters, 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss
    t = _time_steps(step, a, a.batch_size * a.seq_length)
    return _finish("huggingface_lora", a, n_params, sum(p.numel() for p in adapters), t, lora_rank=a.lora_rank,
                   transformers=transformers.__version__)


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
    "huggingface_lora": benchmark_huggingface_lora,
    "native_pytorch": benchmark_native_pytorch,
    "unsloth": _skipped("unsloth", "unsloth"),
    "liger": _skipped("liger", "liger_kernel"),
}


# ------------------------------------------------------------------------------------------------ micro-benchmarks
def micro_benchmark(a) -> Dict[str, float]:
    """Forward, backward, optimizer and full-step device times of one training step (eager, no graph)."""
    from chronicals_b200 import ChronicalsConfig, build_model
    from chronicals_b200.optimizers import FusedAdamW
    dev = _device()
    cfg = ChronicalsConfig.from_model_name(a.model)
    model = build_model(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev, seed=0)
    opt = FusedAdamW(model.parameters(), lr=2e-5, weight_decay=0.01, max_grad_norm=1.0) if dev.type == "cuda" \
        else torch.optim.AdamW(model.parameters(), lr=2e-5)
    batch = {k: v.to(dev) for k, v in load_alpaca_dataloader(cfg.vocab_size, a.batch_size, a.seq_length, 1)[0].items()}
    out: Dict[str, List[float]] = {"forward_ms": [], "backward_ms": [], "optimizer_ms": [], "full_step_ms": []}
    for it in range(a.warmup_steps + a.steps):
        with CUDATimer() as tf:
            loss = model(batch["input_ids"], labels=batch["labels"]).loss
        with CUDATimer() as tb:
            loss.backward()
        with CUDATimer() as to:
            opt.step()
            opt.zero_grad(set_to_none=True)
        if it >= a.warmup_steps:
            out["forward_ms"].append(tf.ms)
            out["backward_ms"].append(tb.ms)
            out["optimizer_ms"].append(to.ms)
            out["full_step_ms"].append(tf.ms + tb.ms + to.ms)
    return {k: statistics.fmean(v) for k, v in out.items()}


def print_gap_analysis(results: List[BenchmarkResult], a) -> None:
    """Where the measured step time sits against the roofline of the measured peaks."""
    from chronicals_b200 import ChronicalsConfig
    from chronicals_b200.config.sota_config import TheoreticalPerformance
    cfg = ChronicalsConfig.from_model_name(a.model)
    tp = TheoreticalPerformance(cfg, a.batch_size * a.seq_length, a.seq_length)
    floor_ms = 1e3 * tp.floor_seconds()
    print(f"\ngap analysis ({a.model}, {a.batch_size}x{a.seq_length} tokens/step)")
    print(f"  roofline floor: {floor_ms:.1f} ms/step = {tp.max_tokens_per_second():,.0f} tok/s "
          f"(GEMM+attention FLOPs at {tp.peak_tflops:.0f} TFLOP/s measured, optimizer bytes at {tp.hbm_gbs:.0f} GB/s measured)")
    for r in results:
        if r.status == "ok":
            print(f"  {r.method:<22} {r.ms_per_step:8.2f} ms  = {r.ms_per_step / floor_ms:5.2f}x floor, "
                  f"{100 * r.tokens_per_sec / TARGET_TOKENS_PER_SEC:6.0f} % of the reference's 50k tok/s target")


def print_comparison(results: List[BenchmarkResult]) -> None:
    ok = [r for r in results if r.status == "ok"]
    base = next((r for r in ok if r.method == "huggingface"), None)
    print(f"\n{'method':<22}{'tok/s':>12}{'ms/step':>10}{'MFU %':>8}{'mem GB':>8}{'loss':>9}{'vs HF':>8}")
    for r in results:
        if r.status != "ok":
            print(f"{r.method:<22}{r.status:>12}  {r.reason}")
            continue
        rel = f"{r.tokens_per_sec / base.tokens_per_sec:7.2f}x" if base else "      -"
        print(f"{r.method:<22}{r.tokens_per_sec:>12,.0f}{r.ms_per_step:>10.2f}{100 * r.mfu:>8.1f}{r.peak_memory_gb:>8.1f}"
              f"{r.final_loss:>9.3f}{rel:>8}")
    print(f"published by the reference on 1x A100-40GB: {PUBLISHED['chronicals_full_ft_a100']:,.0f} tok/s full fine-tune, "
          f"{PUBLISHED['chronicals_lora_a100']:,.0f} tok/s LoRA; Unsloth {PUBLISHED['unsloth_full_ft_a100']:,.0f} tok/s")


def validate_losses(results: List[BenchmarkResult], tolerance: float = 0.15) -> bool:
    """All methods start from a random model on the same data: their losses must agree closely
    (ln V at initialisation).  Guards against a method that skips work."""
    losses = [r.final_loss for r in results if r.status == "ok" and r.final_loss == r.final_loss]
    return (max(losses) - min(losses) <= tolerance * max(1.0, max(losses))) if losses else True


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="chronicals_b200 benchmark suite")
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--seq_length", type=int, default=1024)
    ap.add_argument("--grad_accum", type=int, default=1)
    ap.add_argument("--warmup_steps", type=int, default=5)
    ap.add_argument("--num_runs", type=int, default=1)
    ap.add_argument("--methods", nargs="+", default=["chronicals"], choices=sorted(METHODS))
    ap.add_argument("--output", default=None, help="write the results as JSON to this path")
    ap.add_argument("--gap-analysis", action="store_true")
    ap.add_argument("--micro-benchmark", action="store_true")
    ap.add_argument("--full-suite", action="store_true", help="run every method")
    ap.add_argument("--auto-batch", action="store_true", help="search the largest micro-batch that fits")
    ap.add_argument("--use-cuda-graphs", dest="use_cuda_graphs", action="store_true", default=True)
    ap.add_argument("--no-cuda-graphs", dest="use_cuda_graphs", action="store_false")
    ap.add_argument("--use-compile", action="store_true", help="accepted for compatibility; there is no tracing compiler here")
    ap.add_argument("--no-compile", action="store_true", help="accepted for compatibility")
    ap.add_argument("--lora_rank", type=int, default=16)
    ap.add_argument("--unsloth-lora", action="store_true", help="adds the unsloth and chronicals_lora methods")
    ap.add_argument("--unsloth-full", action="store_true", help="adds the unsloth method")
    ap.add_argument("--fair-compare", action="store_true", help="same data, same optimizer settings, loss validation")
    ap.add_argument("--target-throughput", type=float, default=TARGET_TOKENS_PER_SEC)
    ap.add_argument("--validate", action="store_true", help="check that all methods agree on the loss")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    methods = sorted(METHODS) if a.full_suite else list(a.methods)
    if a.unsloth_lora:
        methods += [m for m in ("chronicals_lora", "unsloth") if m not in methods]
    if a.unsloth_full and "unsloth" not in methods:
        methods.append("unsloth")
    if a.auto_batch and torch.cuda.is_available():
        def one(b):
            saved, a.batch_size = a.batch_size, b
            try:
                saved_steps, saved_w = a.steps, a.warmup_steps
                a.steps, a.warmup_steps = 1, 0
                benchmark_chronicals(a, graphs=False)
                a.steps, a.warmup_steps = saved_steps, saved_w
            finally:
                a.batch_size = saved
        a.batch_size = find_optimal_batch_size(one, start=a.batch_size)
        print(f"auto batch size: {a.batch_size}")
    results: List[BenchmarkResult] = []
    for m in methods:
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats()
        try:
            r = METHODS[m](a)
        except Exception as e:                          # one failing baseline must not hide the others
            r = BenchmarkResult(m, status="failed", reason=f"{type(e).__name__}: {e}"[:300])
        results.append(r)
        print(json.dumps(r.to_dict()), flush=True)
    print_comparison(results)
    if a.gap_analysis:
        print_gap_analysis(results, a)
    micro = micro_benchmark(a) if a.micro_benchmark else None
    if micro:
        print("\nmicro-benchmark (eager): " + ", ".join(f"{k} {v:.2f}" for k, v in micro.items()))
    valid = validate_losses(results) if (a.validate or a.fair_compare) else None
    if valid is not None:
        print(f"loss agreement across methods: {'ok' if valid else 'MISMATCH'}")
    if a.output:
        payload = {"results": [r.to_dict() for r in results], "micro_benchmark": micro, "loss_agreement": valid,
                   "methodology": {"timing": "CUDA events around the timed steps, after warm-up, synchronised on both sides",
                                   "data": "synthetic seeded token ids; random-initialised weights (no network)",
                                   "tokens_per_step": a.batch_size * a.seq_length * a.grad_accum, "steps": a.steps,
                                   "warmup_steps": a.warmup_steps, "num_runs": a.num_runs, "dtype": "bf16",
                                   "mfu": f"6*N*tok/s over {B200_DENSE_BF16_TFLOPS:.0f} TFLOP/s dense bf16",
                                   "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"}}
        with open(a.output, "w") as f:
            json.dump(payload, f, indent=1)
    return 0 if (valid is None or valid) else 1


if __name__ == "__main__":
    sys.exit(main())
