"""Asynchronous offload of saved activations to pinned host memory.

Reference: chronicals/training/async_activation_offload.py:67-136 config and statistics,
:143-209 ``CUDAStreamManager``, :216-300 ``PinnedMemoryPool``, :307-662
``ActivationOffloadManager`` (pack/unpack hooks, device-to-host copies on a side stream,
prefetch), :669-708 ``OffloadActivations`` context, :715-810 ``CheckpointWithOffload``,
:817-906 utilities.  The reference builds this but never wires it; here
``TrainingConfig.use_activation_offloading`` routes gradient checkpointing through it, and it is
mostly useful for the 7B / 14B configurations (a 0.5B step keeps every activation in 180 GB).

Mechanism: ``torch.autograd.graph.saved_tensors_hooks``.  ``pack`` starts a device→host copy on the
offload stream into a pooled pinned buffer and drops the device tensor once the copy has finished;
``unpack`` brings it back on the prefetch stream and makes the compute stream wait for it.
"""
from __future__ import annotations

import contextlib
import threading
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
from torch.utils.checkpoint import checkpoint as _checkpoint


@dataclass
class OffloadConfig:
    enabled: bool = True
    use_pin_memory: bool = True
    use_streams: bool = True
    min_tensor_numel: int = 1024          # smaller tensors stay on the device
    prefetch_ahead: int = 2
    max_pinned_gb: float = 64.0
    keep_on_device: int = 2               # the most recent N packed tensors are not offloaded (used first in backward)


@dataclass
class OffloadStats:
    tensors_offloaded: int = 0
    tensors_kept: int = 0
    bytes_offloaded: int = 0
    bytes_restored: int = 0
    pool_hits: int = 0
    pool_misses: int = 0

    def summary(self) -> Dict[str, float]:
        return {"tensors_offloaded": self.tensors_offloaded, "tensors_kept": self.tensors_kept,
                "offloaded_gb": self.bytes_offloaded / 2**30, "restored_gb": self.bytes_restored / 2**30,
                "pool_hit_rate": self.pool_hits / max(1, self.pool_hits + self.pool_misses)}


class CUDAStreamManager:
    """The offload (D2H) and prefetch (H2D) streams."""

    def __init__(self, device=None):
        self.cuda = torch.cuda.is_available()
        self.device = device
        self.offload_stream = torch.cuda.Stream(device) if self.cuda else None
        self.prefetch_stream = torch.cuda.Stream(device) if self.cuda else None

    def compute_stream(self):
        return torch.cuda.current_stream(self.device) if self.cuda else None


class PinnedMemoryPool:
    """Reuses pinned host buffers by (dtype, numel) so steady-state steps do not call the pinned allocator."""

    def __init__(self, max_bytes: int = 64 << 30, pin: bool = True):
        self.max_bytes, self.pin = max_bytes, pin and torch.cuda.is_available()
        self.free: Dict[Tuple[torch.dtype, int], List[torch.Tensor]] = {}
        self.bytes = 0
        self.lock = threading.Lock()

    def get(self, like: torch.Tensor, stats: Optional[OffloadStats] = None) -> torch.Tensor:
        key = (like.dtype, like.numel())
        with self.lock:
            lst = self.free.get(key)
            if lst:
                if stats:
                    stats.pool_hits += 1
                return lst.pop()
        if stats:
            stats.pool_misses += 1
        nb = like.numel() * like.element_size()
        pin = self.pin and self.bytes + nb <= self.max_bytes
        self.bytes += nb
        return torch.empty(like.numel(), dtype=like.dtype, pin_memory=pin)

    def put(self, buf: torch.Tensor) -> None:
        with self.lock:
            self.free.setdefault((buf.dtype, buf.numel()), []).append(buf)


class _Packed:
    __slots__ = ("host", "shape", "device", "event", "dev_tensor", "dtype")

    def __init__(self):
        self.host = self.shape = self.device = self.event = self.dev_tensor = self.dtype = None


class ActivationOffloadManager:
    def __init__(self, config: Optional[OffloadConfig] = None):
        self.config = config or OffloadConfig()
        self.streams = CUDAStreamManager() if self.config.use_streams else None
        self.pool = PinnedMemoryPool(int(self.config.max_pinned_gb * 2**30), self.config.use_pin_memory)
        self.stats = OffloadStats()
        self._recent: "OrderedDict[int, _Packed]" = OrderedDict()

    # -- hooks ---------------------------------------------------------------------------------------------
    def pack_tensor(self, t: torch.Tensor):
        c = self.config
        if (not c.enabled or not t.is_cuda or t.numel() < c.min_tensor_numel or isinstance(t, torch.nn.Parameter)
                or not t.is_contiguous()):
            self.stats.tensors_kept += 1
            return t
        p = _Packed()
        p.shape, p.device, p.dtype = t.shape, t.device, t.dtype
        p.host = self.pool.get(t, self.stats)
        if self.streams is not None and self.streams.cuda:
            s = self.streams.offload_stream
            s.wait_stream(torch.cuda.current_stream(t.device))
            # a pooled host buffer may still be the source of an earlier host-to-device copy
            s.wait_stream(self.streams.prefetch_stream)
            with torch.cuda.stream(s):
                p.host.copy_(t.reshape(-1), non_blocking=True)
                p.event = torch.cuda.Event()
                p.event.record(s)
            t.record_stream(s)                    # the device memory is reused only after the copy
        else:
            p.host.copy_(t.reshape(-1))
        self.stats.tensors_offloaded += 1
        self.stats.bytes_offloaded += t.numel() * t.element_size()
        # keep the newest few on the device too: they are needed first when backward starts
        if c.keep_on_device > 0:
            p.dev_tensor = t
            self._recent[id(p)] = p
            while len(self._recent) > c.keep_on_device:
                _, old = self._recent.popitem(last=False)
                old.dev_tensor = None
        return p

    def unpack_tensor(self, obj):
        if not isinstance(obj, _Packed):
            return obj
        if obj.dev_tensor is not None:
            t = obj.dev_tensor
            self._release(obj)
            return t
        if self.streams is not None and self.streams.cuda:
            s = self.streams.prefetch_stream
            if obj.event is not None:
                s.wait_event(obj.event)
            with torch.cuda.stream(s):
                t = torch.empty(obj.shape, dtype=obj.dtype, device=obj.device)
                t.reshape(-1).copy_(obj.host, non_blocking=True)
            torch.cuda.current_stream(obj.device).wait_stream(s)
            t.record_stream(torch.cuda.current_stream(obj.device))
        else:
            t = obj.host.to(obj.device).view(obj.shape)
        self.stats.bytes_restored += t.numel() * t.element_size()
        self._release(obj)
        return t

    def _release(self, obj: _Packed) -> None:
        self._recent.pop(id(obj), None)
        if obj.host is not None:
            self.pool.put(obj.host)
            obj.host = None
        obj.dev_tensor = None

    def get_stats(self) -> Dict[str, float]:
        return self.stats.summary()


class OffloadActivations(contextlib.AbstractContextManager):
    """``with OffloadActivations(cfg): loss = model(x)`` — tensors saved for backward inside the block
    are moved to pinned host memory and fetched back when backward needs them."""

    def __init__(self, config: Optional[OffloadConfig] = None, manager: Optional[ActivationOffloadManager] = None):
        self.manager = manager or ActivationOffloadManager(config)
        self._ctx = None

    def __enter__(self):
        self._ctx = torch.autograd.graph.saved_tensors_hooks(self.manager.pack_tensor, self.manager.unpack_tensor)
        self._ctx.__enter__()
        return self.manager

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)


class CheckpointWithOffload:
    """Activation checkpointing whose saved layer inputs live on the host between forward and backward."""

    def __init__(self, config: Optional[OffloadConfig] = None, use_reentrant: bool = False):
        self.manager = ActivationOffloadManager(config)
        self.use_reentrant = use_reentrant

    def __call__(self, fn: Callable, *args, **kwargs):
        with OffloadActivations(manager=self.manager):
            return _checkpoint(fn, *args, use_reentrant=self.use_reentrant, **kwargs)


def estimate_offload_savings(activation_gb: float, offload_fraction: float = 0.8, pcie_gbs: float = 55.0,
                             step_seconds: float = 1.0) -> Dict[str, float]:
    """Device memory freed and whether the transfers hide behind a step of the given length."""
    moved = activation_gb * offload_fraction
    t = 2.0 * moved / pcie_gbs
    return {"device_gb_saved": moved, "transfer_seconds": t, "hidden": t < step_seconds}


def should_offload(tensor: torch.Tensor, config: Optional[OffloadConfig] = None) -> bool:
    c = config or OffloadConfig()
    return bool(c.enabled and tensor.is_cuda and tensor.numel() >= c.min_tensor_numel)


def estimate_offload_bandwidth(tensor_size_mb: float, pcie_bandwidth_gbps: float = 55.0) -> float:
    """Milliseconds to move a tensor of ``tensor_size_mb`` MiB one way at ``pcie_bandwidth_gbps`` GB/s
    (reference async_activation_offload.py:817-833; its default is PCIe 4 x16, a B200 sits on PCIe 5 x16)."""
    return tensor_size_mb / 1024.0 / pcie_bandwidth_gbps * 1e3


def estimate_activation_memory(batch_size: int, seq_len: int, hidden_size: int, intermediate_size: int, num_layers: int,
                               dtype_bytes: int = 2) -> Dict[str, float]:
    """Activation footprint (MiB) of a decoder stack without savings, with sqrt(L) checkpointing, and with
    checkpointing plus host offload of the checkpointed inputs (reference :836-880)."""
    import math
    tok = batch_size * seq_len
    per_layer = tok * dtype_bytes * (hidden_size + intermediate_size + 3 * hidden_size + hidden_size) / 2**20
    every = max(1, int(math.sqrt(num_layers)))
    baseline = num_layers * per_layer
    checkpointed = (num_layers // every + every) * per_layer
    offload = every * per_layer
    return {"per_layer_mb": per_layer, "baseline_mb": baseline, "checkpointed_mb": checkpointed, "offload_mb": offload,
            "checkpoint_every": every, "savings_vs_baseline": baseline / offload,
            "savings_vs_checkpoint": checkpointed / offload}


def create_offload_manager(num_layers: Optional[int] = None, use_checkpointing: bool = True, **offload_kwargs):
    """``CheckpointWithOffload`` when checkpointing is wanted (and the layer count is known), else a bare
    ``ActivationOffloadManager``; keyword arguments are ``OffloadConfig`` fields (reference :887-906)."""
    config = OffloadConfig(**offload_kwargs)
    if use_checkpointing and num_layers is not None:
        return CheckpointWithOffload(config)
    return ActivationOffloadManager(config)
