"""Timers, MFU, memory snapshots, throughput regression monitor and reports.

Same classes as the reference (chronicals/utils/profiling_utils.py:33-96 GPU
table and detection, :99-187 record types, :190-270 ``MFUTracker``, :273-370
``ThroughputMonitor``, :373-620 ``PerformanceProfiler``, :623-737
``MixedPrecisionManager``, :740-866 reports) with a B200 entry and NVTX ranges
around phases.  Timings are CUDA events on the current stream; nothing here
synchronises unless a result is read.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Any, Deque, Dict, List, Optional

import torch

# dense (no 2:4 sparsity) tensor-core peaks in TFLOP/s and memory bandwidth in GB/s
GPU_SPECS: Dict[str, Dict[str, float]] = {
    "B200": {"bf16_tflops": 2250.0, "fp8_tflops": 4500.0, "memory_gb": 180.0, "bandwidth_gbs": 7700.0, "sms": 148},
    "H200": {"bf16_tflops": 989.0, "fp8_tflops": 1979.0, "memory_gb": 141.0, "bandwidth_gbs": 4800.0, "sms": 132},
    "H100": {"bf16_tflops": 989.0, "fp8_tflops": 1979.0, "memory_gb": 80.0, "bandwidth_gbs": 3350.0, "sms": 132},
    "A100": {"bf16_tflops": 312.0, "fp8_tflops": 312.0, "memory_gb": 80.0, "bandwidth_gbs": 2039.0, "sms": 108},
    "L40": {"bf16_tflops": 181.0, "fp8_tflops": 362.0, "memory_gb": 48.0, "bandwidth_gbs": 864.0, "sms": 142},
    "L4": {"bf16_tflops": 121.0, "fp8_tflops": 242.0, "memory_gb": 24.0, "bandwidth_gbs": 300.0, "sms": 58},
    "A10": {"bf16_tflops": 125.0, "fp8_tflops": 125.0, "memory_gb": 24.0, "bandwidth_gbs": 600.0, "sms": 72},
    "V100": {"bf16_tflops": 125.0, "fp8_tflops": 125.0, "memory_gb": 32.0, "bandwidth_gbs": 900.0, "sms": 80},
    "T4": {"bf16_tflops": 65.0, "fp8_tflops": 65.0, "memory_gb": 16.0, "bandwidth_gbs": 320.0, "sms": 40},
}


def detect_gpu_specs(name: Optional[str] = None) -> Dict[str, Any]:
    if name is None:
        name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    up = name.upper()
    for key, spec in GPU_SPECS.items():
        if key in up:
            return {"name": name, "key": key, **spec}
    return {"name": name, "key": "unknown", "bf16_tflops": 100.0, "fp8_tflops": 100.0, "memory_gb": 0.0,
            "bandwidth_gbs": 500.0, "sms": 0}


@dataclass
class TimingBreakdown:
    data_ms: float = 0.0
    forward_ms: float = 0.0
    backward_ms: float = 0.0
    optimizer_ms: float = 0.0
    other_ms: float = 0.0

    @property
    def total_ms(self) -> float:
        return self.data_ms + self.forward_ms + self.backward_ms + self.optimizer_ms + self.other_ms


@dataclass
class MemorySnapshot:
    allocated_gb: float = 0.0
    reserved_gb: float = 0.0
    peak_allocated_gb: float = 0.0

    @classmethod
    def capture(cls, device=None) -> "MemorySnapshot":
        if not torch.cuda.is_available():
            return cls()
        return cls(torch.cuda.memory_allocated(device) / 2**30, torch.cuda.memory_reserved(device) / 2**30,
                   torch.cuda.max_memory_allocated(device) / 2**30)


@dataclass
class PerformanceMetrics:
    step: int = 0
    step_ms: float = 0.0
    tokens: int = 0
    tokens_per_sec: float = 0.0
    mfu: float = 0.0
    timing: TimingBreakdown = field(default_factory=TimingBreakdown)
    memory: MemorySnapshot = field(default_factory=MemorySnapshot)


class MFUTracker:
    """Model FLOPs utilisation with the reference's definition ``6·N·tokens/s ÷ peak``."""

    def __init__(self, num_params: int, peak_tflops: Optional[float] = None, num_gpus: int = 1,
                 attention_flops_per_token: float = 0.0):
        self.num_params = num_params
        self.peak_flops = (peak_tflops or detect_gpu_specs()["bf16_tflops"]) * 1e12 * max(1, num_gpus)
        self.flops_per_token = 6.0 * num_params + attention_flops_per_token
        self.history: List[float] = []

    def compute(self, tokens_per_sec: float) -> float:
        mfu = self.flops_per_token * tokens_per_sec / self.peak_flops
        self.history.append(mfu)
        return mfu

    def average(self) -> float:
        return sum(self.history) / len(self.history) if self.history else 0.0


class ThroughputMonitor:
    """Rolling window of throughput samples; flags a regression when the recent mean drops
    more than ``threshold_pct`` below the best window seen."""

    def __init__(self, window: int = 20, threshold_pct: float = 10.0):
        self.window: Deque[float] = deque(maxlen=window)
        self.threshold = threshold_pct / 100.0
        self.best = 0.0
        self.regressions: List[Dict[str, float]] = []

    def update(self, tokens_per_sec: float, step: int = 0) -> bool:
        self.window.append(tokens_per_sec)
        if len(self.window) < (self.window.maxlen or 1):
            return False
        mean = sum(self.window) / len(self.window)
        self.best = max(self.best, mean)
        if mean < self.best * (1 - self.threshold):
            self.regressions.append({"step": step, "mean": mean, "best": self.best})
            return True
        return False


class _EventPair:
    def __init__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.end = torch.cuda.Event(enable_timing=True)


class PerformanceProfiler:
    """``profile_step()`` / ``profile_phase(name)`` context managers → per-step records.
    Events are resolved lazily (first read synchronises)."""

    PHASES = ("data", "forward", "backward", "optimizer", "other")

    def __init__(self, enabled: bool = True, num_params: int = 0, peak_tflops: Optional[float] = None,
                 use_nvtx: bool = True):
        self.enabled = enabled
        self.cuda = torch.cuda.is_available()
        self.use_nvtx = use_nvtx and self.cuda
        self.records: List[PerformanceMetrics] = []
        self._pending: List[Dict[str, Any]] = []
        self._cur: Optional[Dict[str, Any]] = None
        self.mfu = MFUTracker(num_params, peak_tflops) if num_params else None
        self.monitor = ThroughputMonitor()

    @contextlib.contextmanager
    def profile_step(self, tokens: int = 0):
        if not self.enabled:
            yield
            return
        cur = {"tokens": tokens, "phases": {}, "t0": time.perf_counter()}
        if self.cuda:
            cur["ev"] = _EventPair()
            cur["ev"].start.record()
        if self.use_nvtx:
            torch.cuda.nvtx.range_push("step")
        self._cur = cur
        try:
            yield
        finally:
            if self.use_nvtx:
                torch.cuda.nvtx.range_pop()
            if self.cuda:
                cur["ev"].end.record()
            cur["t1"] = time.perf_counter()
            self._pending.append(cur)
            self._cur = None

    @contextlib.contextmanager
    def profile_phase(self, name: str):
        if not self.enabled or self._cur is None:
            yield
            return
        if self.use_nvtx:
            torch.cuda.nvtx.range_push(name)
        t0 = time.perf_counter()
        ev = _EventPair() if self.cuda else None
        if ev:
            ev.start.record()
        try:
            yield
        finally:
            if ev:
                ev.end.record()
            if self.use_nvtx:
                torch.cuda.nvtx.range_pop()
            self._cur["phases"].setdefault(name, []).append((ev, time.perf_counter() - t0))

    def _resolve(self) -> None:
        if not self._pending:
            return
        if self.cuda:
            torch.cuda.synchronize()
        for cur in self._pending:
            step_ms = cur["ev"].start.elapsed_time(cur["ev"].end) if self.cuda else (cur["t1"] - cur["t0"]) * 1e3
            tb = TimingBreakdown()
            for name, items in cur["phases"].items():
                ms = sum((ev.start.elapsed_time(ev.end) if ev else dt * 1e3) for ev, dt in items)
                attr = f"{name}_ms" if name in self.PHASES else "other_ms"
                setattr(tb, attr, getattr(tb, attr) + ms)
            tps = cur["tokens"] / (step_ms / 1e3) if step_ms > 0 and cur["tokens"] else 0.0
            rec = PerformanceMetrics(step=len(self.records) + 1, step_ms=step_ms, tokens=cur["tokens"],
                                     tokens_per_sec=tps, mfu=self.mfu.compute(tps) if self.mfu and tps else 0.0,
                                     timing=tb, memory=MemorySnapshot.capture())
            self.records.append(rec)
            if tps:
                self.monitor.update(tps, rec.step)
        self._pending = []

    def record_step(self, tokens: int, step_ms: float) -> PerformanceMetrics:
        tps = tokens / (step_ms / 1e3) if step_ms > 0 else 0.0
        rec = PerformanceMetrics(step=len(self.records) + 1, step_ms=step_ms, tokens=tokens, tokens_per_sec=tps,
                                 mfu=self.mfu.compute(tps) if self.mfu else 0.0, memory=MemorySnapshot.capture())
        self.records.append(rec)
        return rec

    def summary(self) -> Dict[str, Any]:
        self._resolve()
        if not self.records:
            return {"steps": 0}
        ms = [r.step_ms for r in self.records]
        return {"steps": len(ms), "mean_step_ms": sum(ms) / len(ms), "min_step_ms": min(ms), "max_step_ms": max(ms),
                "mean_tokens_per_sec": sum(r.tokens_per_sec for r in self.records) / len(ms),
                "peak_memory_gb": max(r.memory.peak_allocated_gb for r in self.records),
                "regressions": self.monitor.regressions}

    def save_report(self, path: str) -> str:
        self._resolve()
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump({"summary": self.summary(), "records": [asdict(r) for r in self.records],
                       "gpu": detect_gpu_specs()}, f, indent=2)
        return path


class MixedPrecisionManager:
    """Chooses compute dtype and (for fp16) owns the loss scaler."""

    def __init__(self, bf16: bool = True, fp16: bool = False, init_scale: float = 65536.0):
        self.dtype = torch.bfloat16 if bf16 else (torch.float16 if fp16 else torch.float32)
        self.scaler = torch.amp.GradScaler("cuda", init_scale=init_scale) if (fp16 and torch.cuda.is_available()) else None

    def autocast(self, device_type: str = "cuda"):
        if self.dtype == torch.float32:
            return contextlib.nullcontext()
        return torch.autocast(device_type=device_type, dtype=self.dtype)

    def backward(self, loss: torch.Tensor) -> None:
        (self.scaler.scale(loss) if self.scaler else loss).backward()

    def step(self, optimizer) -> None:
        if self.scaler:
            self.scaler.step(optimizer)
            self.scaler.update()
        else:
            optimizer.step()


def generate_performance_report(profiler: PerformanceProfiler, path: str = "performance_report.html") -> str:
    s = profiler.summary()
    rows = "".join(f"<tr><td>{r.step}</td><td>{r.step_ms:.2f}</td><td>{r.tokens_per_sec:,.0f}</td>"
                   f"<td>{100 * r.mfu:.1f}</td><td>{r.memory.peak_allocated_gb:.2f}</td></tr>" for r in profiler.records)
    html = (f"<html><body><h1>performance report</h1><pre>{json.dumps(s, indent=2)}</pre>"
            f"<table border='1' cellpadding='3'><tr><th>step</th><th>ms</th><th>tok/s</th><th>MFU %</th>"
            f"<th>peak GB</th></tr>{rows}</table></body></html>")
    with open(path, "w") as f:
        f.write(html)
    return path


def print_performance_report(profiler: PerformanceProfiler) -> None:
    for k, v in profiler.summary().items():
        print(f"  {k}: {v}")


class CUDATimer:
    """CUDA-event stopwatch with synchronise on both sides (benchmark methodology of the reference,
    benchmarks/run_benchmark.py:155-207)."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        self.elapsed_ms = 0.0

    def start(self) -> None:
        if self.cuda:
            torch.cuda.synchronize()
            self._a, self._b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._a.record()
        else:
            self._t = time.perf_counter()

    def stop(self) -> float:
        if self.cuda:
            self._b.record()
            torch.cuda.synchronize()
            self.elapsed_ms = self._a.elapsed_time(self._b)
        else:
            self.elapsed_ms = (time.perf_counter() - self._t) * 1e3
        return self.elapsed_ms
