"""Sharded data-parallel optimizer with the collectives fused into the update (ZeRO-1 layout).

All trainable parameters live in one flat bf16 buffer in symmetric memory (the model's parameters
become views of it), and gradients are gathered into an identically laid-out symmetric gradient
buffer.  Rank ``r`` owns the ``r``-th 1/W slice: it keeps AdamW moments only for that slice.  One
optimizer step is, on every rank, on the current stream:

1. barrier (all ranks' gradients are in their buffers);
2. ``rs_reduce_sqnorm``: pull my slice from all W gradient buffers, average in fp32, keep the fp32
   result locally, produce my share of the squared gradient norm  — the reduce-scatter, fused with
   the cast, the 1/W scale and the norm;
3. barrier carrying each rank's norm share (4 floats) — the only all-reduce, done by the flag pad;
4. ``adamw_shard_allgather``: clip coefficient from the W shares, AdamW on my slice, and the new
   bf16 parameters stored straight into every rank's parameter buffer — the all-gather, fused
   with the update;
5. barrier (all parameters are in place before the next forward reads them).

No NCCL call is made in a step.  The step is capturable in a CUDA graph (``prepare_step`` holds the
host part, ``launch_step`` the kernels).  The reference has no counterpart (single GPU).
"""
from __future__ import annotations

import ctypes
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext
from . import symm

CHUNK = 1024       # granularity of the per-element hyper-parameter group table


class ShardedFusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, group=None, master_weights: bool = False, wait_budget_us: int = 2_000_000):
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        if not symm.peer_access_available(group):
            raise RuntimeError("peer access between the local GPUs is not available")
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.ctx = symm.SymmetricContext(group, wait_budget_us)
        self.rank, self.world = self.ctx.rank, self.ctx.world
        self._layout()
        self._move_params_to_symmetric_memory(master_weights)
        self.last_grad_norm: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------------------------------ layout
    def _layout(self) -> None:
        self.entries: List[Dict[str, Any]] = []
        off = 0
        for gi, g in enumerate(self.param_groups):
            for p in g["params"]:
                if not p.requires_grad:
                    continue
                if p.dtype != torch.bfloat16 or not p.is_cuda:
                    raise ValueError("ShardedFusedAdamW handles bf16 CUDA parameters")
                n = p.numel()
                self.entries.append({"p": p, "off": off, "n": n, "group": gi})
                off += (n + CHUNK - 1) // CHUNK * CHUNK          # every tensor starts on a chunk boundary
        unit = CHUNK * self.world
        self.total = (off + unit - 1) // unit * unit
        self.shard = self.total // self.world
        self.lo, self.hi = self.rank * self.shard, (self.rank + 1) * self.shard

    def _move_params_to_symmetric_memory(self, master_weights: bool) -> None:
        dev = self.entries[0]["p"].device
        self.param_buf = symm.SymmetricBuffer(self.total, torch.bfloat16, self.ctx.group)
        self.grad_buf = symm.SymmetricBuffer(self.total, torch.bfloat16, self.ctx.group)
        groups = torch.zeros(self.total // CHUNK, dtype=torch.uint8)
        with torch.no_grad():
            for e in self.entries:
                view = self.param_buf.local[e["off"]: e["off"] + e["n"]].view(e["p"].shape)
                view.copy_(e["p"].data)
                e["p"].data = view                                  # the model now reads the symmetric buffer
                e["gview"] = self.grad_buf.local[e["off"]: e["off"] + e["n"]].view(e["p"].shape)
                groups[e["off"] // CHUNK: (e["off"] + e["n"] + CHUNK - 1) // CHUNK] = e["group"]
        self.chunk_group = groups[self.lo // CHUNK: self.hi // CHUNK].contiguous().to(dev)
        self.reduced = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.master = self.param_buf.local[self.lo:self.hi].float() if master_weights else None
        self.partials = torch.zeros(self.ctx.grid, dtype=torch.float32, device=dev)
        self.payload = torch.zeros(self.ctx.payload_floats, dtype=torch.float32, device=dev)
        self.hyper = torch.zeros(len(self.param_groups) * 8, dtype=torch.float32, device=dev)
        self.norm_out = torch.zeros(3, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        dist.barrier(group=self.ctx.group)

    # ------------------------------------------------------------------------------------------ step
    def ensure_state(self) -> None:
        pass                                                        # everything is allocated in __init__

    def prepare_step(self) -> None:
        self.step_count += 1
        t = self.step_count
        vals: List[float] = []
        for g in self.param_groups:
            b1, b2 = g["betas"]
            vals += [float(g["lr"]), float(g["weight_decay"]), b1, b2, float(g["eps"]), 1.0 - b1 ** t, 1.0 - b2 ** t, 0.0]
        self.hyper.copy_(torch.tensor(vals, dtype=torch.float32), non_blocking=True)

    @torch.no_grad()
    def launch_step(self) -> None:
        srcs, dsts = [], []
        for e in self.entries:
            g = e["p"].grad
            if g is None:
                e["gview"].zero_()
            elif g.data_ptr() != e["gview"].data_ptr():
                srcs.append(g)
                dsts.append(e["gview"])
        if srcs:
            torch._foreach_copy_(dsts, srcs)
        lib = symm._lib()
        s = _ext.stream_ptr()
        st = self.ctx.status.data_ptr()
        self.ctx.barrier()
        code = lib.cb_rs_reduce_sqnorm(self.grad_buf.ptrs, self.world, self.lo, self.hi, self.reduced.data_ptr(),
                                       self.partials.data_ptr(), self.payload.data_ptr(), st, s)
        _ext.check(code, "rs_reduce_sqnorm")
        gathered = self.ctx.barrier(self.payload)
        code = lib.cb_adamw_shard_allgather(self.param_buf.ptrs, self.world, self.rank, self.lo, self.hi,
                                            self.reduced.data_ptr(), self.exp_avg.data_ptr(),
                                            self.exp_avg_sq.data_ptr(), _ext.ptr(self.master),
                                            self.chunk_group.data_ptr(), self.hyper.data_ptr(), gathered.data_ptr(),
                                            float(self.max_grad_norm or 0.0), self.norm_out.data_ptr(), st, s)
        _ext.check(code, "adamw_shard_allgather")
        self.ctx.barrier()
        self.last_grad_norm = self.norm_out[1]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.prepare_step()
        self.launch_step()
        return loss

    # ------------------------------------------------------------------------------------------ state
    def state_dict(self) -> Dict[str, Any]:
        """This rank's shard of the optimizer state (write one file per rank)."""
        return {"step_count": self.step_count, "rank": self.rank, "world": self.world, "total": self.total,
                "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
                "master": self.master.cpu() if self.master is not None else None,
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd.get("world") != self.world or sd.get("total") != self.total:
            raise ValueError("sharded optimizer state was written with a different world size or model; "
                             "consolidate it with parallel.zero.consolidate_states first")
        self.step_count = int(sd["step_count"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        if self.master is not None and sd.get("master") is not None:
            self.master.copy_(sd["master"])
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update({k: v for k, v in saved.items() if k in ("lr", "weight_decay", "betas", "eps")})


def consolidate_states(shards: List[Dict[str, Any]]) -> Dict[str, Any]:
    """Concatenate per-rank shards (in rank order) into a world-size-independent flat state; a new
    run with a different number of ranks re-slices it with :func:`reshard_state`."""
    shards = sorted(shards, key=lambda s: s["rank"])
    return {"step_count": shards[0]["step_count"], "total": shards[0]["total"],
            "exp_avg": torch.cat([s["exp_avg"] for s in shards]), "exp_avg_sq": torch.cat([s["exp_avg_sq"] for s in shards]),
            "param_groups": shards[0]["param_groups"]}


def reshard_state(flat: Dict[str, Any], rank: int, world: int, total: Optional[int] = None) -> Dict[str, Any]:
    """Slice a consolidated state for ``rank`` of ``world`` (the flat layout pads to a multiple of
    ``1024 * world``; a different world size may need a few zero elements appended)."""
    n = flat["exp_avg"].numel()
    unit = CHUNK * world
    tot = total or (n + unit - 1) // unit * unit

    def fit(t):
        if t.numel() < tot:
            t = torch.cat((t, torch.zeros(tot - t.numel(), dtype=t.dtype)))
        return t[:tot]
    sh = tot // world
    return {"step_count": flat["step_count"], "rank": rank, "world": world, "total": tot,
            "exp_avg": fit(flat["exp_avg"])[rank * sh:(rank + 1) * sh].clone(),
            "exp_avg_sq": fit(flat["exp_avg_sq"])[rank * sh:(rank + 1) * sh].clone(), "master": None,
            "param_groups": flat["param_groups"]}
