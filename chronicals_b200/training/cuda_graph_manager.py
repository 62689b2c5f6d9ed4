"""Capture and replay of training steps (or any callable) as CUDA graphs.

Reference: chronicals/training/cuda_graph_manager.py:44-88 config and
statistics, :91-130 memory pool, :133-204 ``CapturedGraph`` with static input
buffers, :207-605 manager (warm-up, capture, replay, eviction), :608-695
helpers.  The reference constructs its manager but never replays a graph from
the training loop; here ``ChronicalsTrainer`` replays the captured step when
``use_cuda_graphs=True`` and this manager offers the same facility for user
callables, keyed by input shapes.
"""
from __future__ import annotations

import functools
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class CUDAGraphConfig:
    enabled: bool = True
    warmup_steps: int = 3
    capture_mode: str = "thread_local"
    use_memory_pool: bool = True
    static_shapes: bool = True
    max_cached_graphs: int = 16
    shape_buckets: List[int] = field(default_factory=lambda: [128, 256, 512, 1024, 2048, 4096])
    fallback_on_error: bool = True


@dataclass
class GraphStatistics:
    captures: int = 0
    replays: int = 0
    eager_runs: int = 0
    evictions: int = 0
    capture_failures: int = 0

    @property
    def hit_rate(self) -> float:
        tot = self.replays + self.eager_runs
        return self.replays / tot if tot else 0.0


class CUDAGraphMemoryPool:
    """One private allocator pool shared by every graph of a manager."""

    def __init__(self):
        self.handle = torch.cuda.graph_pool_handle() if torch.cuda.is_available() else None


class CapturedGraph:
    """A graph plus the static tensors it reads and writes."""

    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], pool: Optional[CUDAGraphMemoryPool] = None,
                 warmup_steps: int = 3, capture_mode: str = "thread_local"):
        self.static_inputs = [x.clone() for x in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup_steps)):
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        kw = {"pool": pool.handle} if pool is not None and pool.handle is not None else {}
        with torch.cuda.graph(self.graph, capture_error_mode=capture_mode, **kw):
            self.static_outputs = fn(*self.static_inputs)

    def replay(self, *inputs: torch.Tensor):
        for dst, src in zip(self.static_inputs, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_outputs          # static tensors: overwritten by the next replay
        return self.static_outputs


def bucket_length(n: int, buckets: Sequence[int]) -> int:
    """Smallest bucket >= n (sequence lengths are padded up so few graphs cover all shapes)."""
    for b in sorted(buckets):
        if n <= b:
            return b
    return n


class CUDAGraphManager:
    def __init__(self, config: Optional[CUDAGraphConfig] = None):
        self.config = config or CUDAGraphConfig()
        self.stats = GraphStatistics()
        self.pool = CUDAGraphMemoryPool() if self.config.use_memory_pool else None
        self._graphs: "OrderedDict[Tuple, CapturedGraph]" = OrderedDict()
        self._warm: Dict[Tuple, int] = {}

    @staticmethod
    def _key(name: str, inputs: Sequence[torch.Tensor]) -> Tuple:
        return (name,) + tuple((tuple(x.shape), x.dtype) for x in inputs)

    def warmup_step(self, key: Tuple) -> bool:
        """Counts eager runs of a shape; True once enough have happened to capture."""
        self._warm[key] = self._warm.get(key, 0) + 1
        return self._warm[key] > self.config.warmup_steps

    def capture(self, name: str, fn: Callable, *inputs: torch.Tensor) -> Optional[CapturedGraph]:
        key = self._key(name, inputs)
        try:
            g = CapturedGraph(fn, inputs, self.pool, self.config.warmup_steps, self.config.capture_mode)
        except Exception:
            self.stats.capture_failures += 1
            if self.config.fallback_on_error:
                return None
            raise
        self._graphs[key] = g
        self.stats.captures += 1
        while len(self._graphs) > self.config.max_cached_graphs:
            self._graphs.popitem(last=False)
            self.stats.evictions += 1
        return g

    capture_training_step = capture

    def replay(self, name: str, *inputs: torch.Tensor):
        g = self._graphs[self._key(name, inputs)]
        self._graphs.move_to_end(self._key(name, inputs))
        self.stats.replays += 1
        return g.replay(*inputs)

    def replay_or_run(self, name: str, fn: Callable, *inputs: torch.Tensor):
        """Replay the graph for these shapes; capture it after the warm-up count; run eagerly otherwise."""
        if not (self.config.enabled and torch.cuda.is_available() and all(x.is_cuda for x in inputs)):
            self.stats.eager_runs += 1
            return fn(*inputs)
        key = self._key(name, inputs)
        if key in self._graphs:
            return self.replay(name, *inputs)
        if self.warmup_step(key) and self.capture(name, fn, *inputs) is not None:
            return self.replay(name, *inputs)
        self.stats.eager_runs += 1
        return fn(*inputs)

    def clear(self) -> None:
        self._graphs.clear()
        self._warm.clear()

    def get_statistics(self) -> Dict[str, Any]:
        s = self.stats
        return {"captures": s.captures, "replays": s.replays, "eager_runs": s.eager_runs, "evictions": s.evictions,
                "capture_failures": s.capture_failures, "hit_rate": s.hit_rate, "cached": len(self._graphs)}


def create_cuda_graph_training_step(model, optimizer, loss_fn: Optional[Callable] = None,
                                    manager: Optional[CUDAGraphManager] = None) -> Callable:
    """``step(input_ids, labels) -> loss`` whose forward+backward+update replays from a graph.
    The optimizer must expose ``prepare_step`` / ``launch_step`` (``FusedAdamW`` does)."""
    manager = manager or CUDAGraphManager()

    def body(ids: torch.Tensor, labels: torch.Tensor):
        out = model(ids, labels=labels)
        loss = out.loss if loss_fn is None else loss_fn(out, labels)
        loss.backward()
        optimizer.launch_step()
        return loss.detach()

    def step(ids: torch.Tensor, labels: torch.Tensor):
        optimizer.ensure_state()
        optimizer.zero_grad(set_to_none=True)
        optimizer.prepare_step()
        return manager.replay_or_run("train_step", body, ids, labels)

    return step


def cuda_graph_capture(fn: Optional[Callable] = None, *, manager: Optional[CUDAGraphManager] = None):
    """Decorator: the decorated tensor function replays from a per-shape graph after warm-up."""
    mgr = manager or CUDAGraphManager()

    def deco(f):
        @functools.wraps(f)
        def wrapped(*inputs):
            return mgr.replay_or_run(f.__name__, f, *inputs)
        wrapped.graph_manager = mgr
        return wrapped

    return deco(fn) if fn is not None else deco


def enable_cuda_graphs(trainer_or_config, enabled: bool = True):
    """README-documented switch: sets ``use_cuda_graphs`` on a trainer or a ``TrainingConfig``."""
    target = getattr(trainer_or_config, "args", trainer_or_config)
    target.use_cuda_graphs = enabled
    if hasattr(trainer_or_config, "use_cuda_graphs"):
        trainer_or_config.use_cuda_graphs = enabled and torch.cuda.is_available()
    return trainer_or_config
