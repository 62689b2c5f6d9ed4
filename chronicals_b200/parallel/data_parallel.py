"""Data-parallel gradient reduction.

``GradientReducer`` owns flat, bucket-ordered gradient buffers.  After the
backward pass every gradient is copied into its bucket (one multi-tensor copy
per bucket), the bucket is averaged across ranks, and ``p.grad`` is re-pointed at
its slice of the bucket, so the optimizer reads reduced values without a copy
back.  Buckets are ordered last-layer-first so the first collective can start
while the host is still queueing the rest.

Back-ends:

* ``"nccl"`` / ``"gloo"`` — ``torch.distributed.all_reduce`` per bucket (the
  comparison baseline; also what runs on CPU ranks);
* ``"fused"`` — the in-kernel peer-memory reduce (``parallel.symm``), falling
  back to the process-group path when peer access is unavailable.

The reference has no multi-GPU support, so there is no counterpart to cite.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class _Bucket:
    def __init__(self, params: List[torch.nn.Parameter], dtype: torch.dtype, device: torch.device):
        self.params = params
        self.numels = [p.numel() for p in params]
        # 16-byte aligned slices so vectorised kernels can run on each view
        self.offsets: List[int] = []
        o = 0
        for n in self.numels:
            self.offsets.append(o)
            o += (n + 7) // 8 * 8
        self.flat = torch.zeros(o, dtype=dtype, device=device)
        self.views = [self.flat[a:a + n].view(p.shape) for a, n, p in zip(self.offsets, self.numels, params)]
        self.work = None


class GradientReducer:
    def __init__(self, model: torch.nn.Module, backend: str = "nccl", bucket_mb: float = 32.0,
                 process_group=None, average: bool = True):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("GradientReducer needs an initialised process group")
        self.group = process_group
        self.world = dist.get_world_size(process_group)
        self.backend = backend
        self.average = average
        params = [p for p in model.parameters() if p.requires_grad]
        # de-duplicate tied parameters, keep reverse registration order (≈ order gradients become ready)
        seen, ordered = set(), []
        for p in reversed(params):
            if id(p) not in seen:
                seen.add(id(p))
                ordered.append(p)
        limit = int(bucket_mb * 2**20)
        self.buckets: List[_Bucket] = []
        cur: List[torch.nn.Parameter] = []
        size = 0
        for p in ordered:
            nb = p.numel() * p.element_size()
            if cur and (size + nb > limit or p.dtype != cur[0].dtype):
                self.buckets.append(_Bucket(cur, cur[0].dtype, cur[0].device))
                cur, size = [], 0
            cur.append(p)
            size += nb
        if cur:
            self.buckets.append(_Bucket(cur, cur[0].dtype, cur[0].device))
        self._fused = None
        if backend == "fused":
            try:
                from .symm import FusedAllReduce
                self._fused = FusedAllReduce(self.buckets, self.group)
            except Exception as e:     # peer access / symmetric memory unavailable: baseline path
                print(f"[parallel] fused collectives unavailable ({e}); using the process-group path")
                self._fused = None

    @property
    def num_buckets(self) -> int:
        return len(self.buckets)

    @torch.no_grad()
    def reduce_gradients(self) -> None:
        """Average every gradient across ranks; afterwards ``p.grad`` aliases the reduced bucket."""
        gloo = dist.get_backend(self.group) == "gloo"
        for b in self.buckets:
            srcs, dsts = [], []
            for p, v in zip(b.params, b.views):
                if p.grad is None:
                    v.zero_()
                elif p.grad.data_ptr() != v.data_ptr():
                    srcs.append(p.grad)
                    dsts.append(v)
            if srcs:
                torch._foreach_copy_(dsts, srcs)
            if self._fused is not None:
                self._fused.all_reduce(b)
            elif gloo or not self.average:
                b.work = dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            else:
                b.work = dist.all_reduce(b.flat, op=dist.ReduceOp.AVG, group=self.group, async_op=True)
        for b in self.buckets:
            if b.work is not None:
                b.work.wait()
                b.work = None
                if gloo and self.average:
                    b.flat.div_(self.world)
            for p, v in zip(b.params, b.views):
                p.grad = v

    def broadcast_parameters(self, model: torch.nn.Module, src: int = 0) -> None:
        """Make every rank start from rank ``src``'s weights."""
        for p in model.parameters():
            dist.broadcast(p.data, src=src, group=self.group)
