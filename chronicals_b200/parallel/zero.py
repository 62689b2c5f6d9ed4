"""Sharded data-parallel optimizer whose collectives are fused into the update and overlap the backward pass
(ZeRO-1 layout).

All trainable parameters live in one flat bf16 buffer in symmetric (peer-mapped) memory — the model's
parameters become views of it — and gradients are gathered into an identically laid-out symmetric gradient
buffer.  The buffer is cut into *buckets* of consecutive parameters (about one decoder layer each).  Rank
``r`` owns the ``r``-th 1/W slice of every bucket and keeps AdamW moments only for those slices.

During the backward pass a post-accumulate hook on every parameter copies the finished gradient into the
gradient buffer; when the last gradient of a bucket has arrived the bucket's reduce-scatter is queued on a
side stream, so it runs while the main stream is still computing earlier layers:

    side stream, per bucket :  barrier (all ranks hold this bucket's gradients)
                               ``rs_bucket``: pull my slice from all W gradient buffers over NVLink, average in
                               fp32, keep the result locally, emit sum-of-squares partials — the reduce-scatter
                               fused with the cast, the 1/W scale and the norm (small grid of 128-thread
                               blocks that share SMs with the compute kernels)
    main stream, after bwd  :  join the side stream; sum the partials
                               barrier carrying each rank's norm share (4 floats) — the only all-reduce
                               ``adamw_shard_allgather``: clip coefficient from the W shares, AdamW on my slices,
                               new bf16 parameters stored straight into every rank's parameter buffer — the
                               all-gather fused with the update
                               barrier (all parameters are in place before the next forward reads them)

No NCCL call is made in a step, so the whole step (hooks included) can be captured in one CUDA graph:
``prepare_step`` is the host part, ``launch_step`` the tail after the backward pass.

On CPU (gloo) the same bucket bookkeeping runs on ``torch.distributed`` collectives; that path is the oracle
of the layout and of the state re-sharding, the kernels are tested on GPUs against the unsharded optimizer.
The reference has no counterpart (single GPU).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext

CHUNK = 1024       # granularity of the per-element hyper-parameter group table


class _Bucket:
    __slots__ = ("index", "entries", "lo", "hi", "shard", "loc", "pending", "ready")

    def __init__(self, index: int):
        self.index = index
        self.entries: List[Dict[str, Any]] = []
        self.lo = self.hi = self.shard = self.loc = 0
        self.pending = 0
        self.ready = False


class ShardedFusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, group=None, master_weights: bool = False, wait_budget_us: int = 2_000_000,
                 bucket_mb: float = 24.0, overlap: bool = False, rs_grid: int = 148):
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("ShardedFusedAdamW needs an initialised process group")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.bucket_bytes = int(bucket_mb * 2**20)
        self.overlap = overlap
        self.rs_grid = int(rs_grid)
        p0 = next(p for g in self.param_groups for p in g["params"] if p.requires_grad)
        self.device, self.dtype = p0.device, p0.dtype
        self.fused = self.device.type == "cuda"
        if self.fused:
            from . import symm
            if not symm.peer_access_available(group):
                raise RuntimeError("peer access between the local GPUs is not available")
            self.symm = symm
            self.ctx = symm.SymmetricContext(group, wait_budget_us)
        self._layout()
        self._move_params(master_weights)
        self._install_hooks()
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.accumulating = False          # True on micro-steps that only accumulate (no reduce, no update)
        self.direct_writes = 0             # gradients that arrived already inside the buffer (diagnostic counter)
        # with ``profile = True`` (eager steps only) CUDA events bracket every bucket's reduce-scatter and the tail
        # of the step; ``profile_report()`` turns the last step's events into hidden / exposed times
        self.profile = False
        self._events: Dict[str, Any] = {}

    # ------------------------------------------------------------------------------------------ layout
    def _layout(self) -> None:
        """Buckets of consecutive parameters; every bucket's length is a multiple of ``CHUNK * world`` and every
        tensor starts on a chunk boundary, so a chunk never straddles tensors, groups or ranks."""
        W = self.world
        self.buckets: List[_Bucket] = []
        self.entries: List[Dict[str, Any]] = []
        cur = _Bucket(0)
        off = 0
        esz = 2 if self.dtype == torch.bfloat16 else 4
        for gi, g in enumerate(self.param_groups):
            for p in g["params"]:
                if not p.requires_grad:
                    continue
                if p.dtype != self.dtype or p.device != self.device:
                    raise ValueError("ShardedFusedAdamW needs all parameters on one device in one dtype")
                if self.fused and p.dtype != torch.bfloat16:
                    raise ValueError("the fused path handles bf16 parameters")
                n = p.numel()
                e = {"p": p, "off": off, "n": n, "group": gi, "bucket": cur}
                cur.entries.append(e)
                self.entries.append(e)
                off += (n + CHUNK - 1) // CHUNK * CHUNK
                if (off - cur.lo) * esz >= self.bucket_bytes:
                    off = self._close(cur, off)
                    self.buckets.append(cur)
                    cur = _Bucket(len(self.buckets))
                    cur.lo = off
        if cur.entries:
            off = self._close(cur, off)
            self.buckets.append(cur)
        self.total = off
        self.shard = self.total // W
        loc = 0
        for b in self.buckets:
            b.shard = (b.hi - b.lo) // W
            b.loc = loc
            loc += b.shard

    def _close(self, b: _Bucket, off: int) -> int:
        unit = CHUNK * self.world
        b.hi = b.lo + (off - b.lo + unit - 1) // unit * unit
        return b.hi

    def _slice(self, b: _Bucket, rank: Optional[int] = None):
        r = self.rank if rank is None else rank
        return b.lo + r * b.shard, b.lo + (r + 1) * b.shard

    def _move_params(self, master_weights: bool) -> None:
        dev = self.device
        if self.fused:
            self.param_buf = self.symm.SymmetricBuffer(self.total, torch.bfloat16, self.group)
            self.grad_buf = self.symm.SymmetricBuffer(self.total, torch.bfloat16, self.group)
            self.param_flat, self.grad_flat = self.param_buf.local, self.grad_buf.local
        else:
            self.param_flat = torch.zeros(self.total, dtype=self.dtype, device=dev)
            self.grad_flat = torch.zeros(self.total, dtype=self.dtype, device=dev)
        groups = torch.zeros(self.total // CHUNK, dtype=torch.uint8)
        with torch.no_grad():
            for e in self.entries:
                view = self.param_flat[e["off"]: e["off"] + e["n"]].view(e["p"].shape)
                view.copy_(e["p"].data)
                e["p"].data = view                                  # the model now reads the flat buffer
                e["gview"] = self.grad_flat[e["off"]: e["off"] + e["n"]].view(e["p"].shape)
                groups[e["off"] // CHUNK: (e["off"] + e["n"] + CHUNK - 1) // CHUNK] = e["group"]
        mine_groups, offs = [], []
        for b in self.buckets:
            lo, hi = self._slice(b)
            mine_groups.append(groups[lo // CHUNK: hi // CHUNK])
            offs.append(torch.arange(lo, hi, CHUNK, dtype=torch.int64))
        self.chunk_group = torch.cat(mine_groups).contiguous().to(dev)
        self.chunk_off = torch.cat(offs).contiguous().to(dev)
        self.reduced = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.master = self._gather_local(self.param_flat).float() if master_weights else None
        if self.fused:
            # sum-of-squares partials: one row of `4 * full_grid` floats (one per warp) per bucket; a bucket reduced by the small
            # co-resident grid fills only the head of its row, the rest stays zero (the buffer is cleared after
            # every step's sum)
            self.full_grid = 4 * torch.cuda.get_device_properties(dev).multi_processor_count
            self.rs_grid = max(1, min(self.rs_grid, self.full_grid))
            self.partials = torch.zeros(len(self.buckets) * self.full_grid * 4, dtype=torch.float32, device=dev)   # 4 warps per block
            self.payload = torch.zeros(self.ctx.payload_floats, dtype=torch.float32, device=dev)
            self.hyper = torch.zeros(len(self.param_groups) * 8, dtype=torch.float32, device=dev)
            self.norm_out = torch.zeros(3, dtype=torch.float32, device=dev)
            self.side = torch.cuda.Stream(device=dev)
            self._bind()
            torch.cuda.synchronize()
        else:
            self.sq_total = torch.zeros(1, dtype=torch.float32, device=dev)
        dist.barrier(group=self.group)

    def _bind(self) -> None:
        import ctypes
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib = self.symm._lib()
        for name, args in (("cb_rs_bucket", [P, I, L, L, P, P, I, P, P]),
                           ("cb_sum_partials", [P, I, P, P]),
                           ("cb_adamw_shard_allgather_table", [P, I, I, L, P, P, P, P, P, P, P, P, F, P, P, P])):
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, ctypes.c_int
        self.lib = lib

    def _gather_local(self, flat: torch.Tensor) -> torch.Tensor:
        """This rank's slices of a flat [total] tensor, concatenated in bucket order ([shard])."""
        return torch.cat([flat[slice(*self._slice(b))] for b in self.buckets])

    # ------------------------------------------------------------------------------------------ hooks
    def _install_hooks(self) -> None:
        self._handles = []
        for e in self.entries:
            self._handles.append(e["p"].register_post_accumulate_grad_hook(lambda p, e=e: self._on_grad(e)))
            if e["p"].dim() == 2:
                # weight-gradient kernels write straight into the gradient buffer (ops.grad_destination)
                e["p"]._cb_grad_out = (lambda e=e: None if e.get("filled", False) else e["gview"].view(e["p"].shape))
        self._reset_pending()

    def _reset_pending(self) -> None:
        for b in self.buckets:
            b.pending = len(b.entries)
            b.ready = False
        self._forked = False
        self._n_ready = 0

    @torch.no_grad()
    def _on_grad(self, e: Dict[str, Any]) -> None:
        """A parameter's gradient is final for this backward pass: move it into the gradient buffer and, when
        its bucket is complete, queue the bucket's reduce-scatter."""
        p = e["p"]
        g = p.grad
        if g is None:
            return
        if g.data_ptr() == e["gview"].data_ptr():
            self.direct_writes += 1             # the producing kernel wrote into the buffer; nothing to copy
        else:
            if e.get("filled", False):
                e["gview"].add_(g)              # a later micro-batch of a gradient-accumulation window
            else:
                e["gview"].copy_(g)
        # the buffer holds the gradient now: drop the autograd-side tensor (or the adopted view of the buffer,
        # into which the next backward pass would otherwise accumulate in place)
        p.grad = None
        e["filled"] = True
        e["seen"] = True
        b = e["bucket"]
        if b.pending == 0:
            # first gradient of a new backward pass after one that was not followed by a step (warm-up,
            # accumulation): every bucket starts counting again
            for o in self.buckets:
                o.pending, o.ready = len(o.entries), False
            self._n_ready = 0
        b.pending -= 1
        if b.pending == 0 and not self.accumulating:
            b.ready = True
            self._n_ready += 1
            if self.overlap:
                # the bucket that completes last has nothing left to hide behind: it runs on the main stream with
                # the whole GPU instead of the small co-resident grid
                self._reduce_bucket(b, overlapped=self._n_ready < len(self.buckets))

    def begin_micro_step(self, last: bool = True) -> None:
        """Call before every backward pass of a gradient-accumulation window; ``last`` marks the micro-step whose
        backward pass is followed by ``step()``.  With one micro-batch per optimizer step nothing has to be called."""
        self.accumulating = not last
        for b in self.buckets:
            b.pending = len(b.entries)
            b.ready = False
        self._n_ready = 0
        if self.fused and self.profile and not torch.cuda.is_current_stream_capturing():
            self._events["micro_start"] = torch.cuda.Event(enable_timing=True)
            self._events["micro_start"].record(torch.cuda.current_stream(self.device))

    # ------------------------------------------------------------------------------------------ reduce-scatter
    def _reduce_bucket(self, b: _Bucket, overlapped: bool, barrier: bool = True) -> None:
        lo, hi = self._slice(b)
        out = self.reduced[b.loc: b.loc + b.shard]
        for e in b.entries:
            e["filled"] = False                          # the next backward pass starts this gradient afresh
        if not self.fused:
            g = self.grad_flat[b.lo:b.hi].float()
            dist.all_reduce(g, group=self.group)
            out.copy_(g[lo - b.lo: hi - b.lo] / self.world)
            self.sq_total += out.pow(2).sum()
            return
        main = torch.cuda.current_stream(self.device)
        stream = self.side if overlapped else main
        if overlapped:
            ev = torch.cuda.Event()
            ev.record(main)
            self.side.wait_event(ev)                     # the bucket's gradients are complete on the main stream
            self._forked = True
        elif getattr(self, "_forked", False) and barrier:
            # Barriers share one epoch counter and one flag pad per rank, so two of them must never run at the same
            # time: a barrier on the main stream waits for the side stream's reduce-scatters (and barriers) first.
            # (Without this join the hook path timed out on 8 GPUs: "peer flag never arrived".)
            ev = torch.cuda.Event()
            ev.record(self.side)
            main.wait_event(ev)
        grid = self.rs_grid if overlapped else self.full_grid
        prof = self.profile and not torch.cuda.is_current_stream_capturing()
        if prof:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), overlapped)
            self._events.setdefault("buckets", {})[b.index] = ev
            ready = torch.cuda.Event(enable_timing=True)
            ready.record(main)
            self._events.setdefault("ready", {})[b.index] = ready
        with torch.cuda.stream(stream):
            if prof:
                ev[0].record(stream)
            if barrier:
                self.ctx.barrier()                       # every rank holds this bucket's gradients
            code = self.lib.cb_rs_bucket(self.grad_buf.ptrs, self.world, lo, hi, out.data_ptr(),
                                         self.partials[b.index * self.full_grid * 4:].data_ptr(), grid,
                                         self.ctx.status.data_ptr(), stream.cuda_stream)
            _ext.check(code, "rs_bucket")
            _ext.count_launch(2 if barrier else 1)
            if prof:
                ev[1].record(stream)

    # ------------------------------------------------------------------------------------------ step
    def ensure_state(self) -> None:
        pass                                                        # everything is allocated in __init__

    def prepare_step(self) -> None:
        self.step_count += 1
        if self.fused:
            self.hyper.copy_(torch.tensor(self._hyper_values(), dtype=torch.float32), non_blocking=True)

    def _hyper_values(self) -> List[float]:
        t = self.step_count
        vals: List[float] = []
        for g in self.param_groups:
            b1, b2 = g["betas"]
            vals += [float(g["lr"]), float(g["weight_decay"]), b1, b2, float(g["eps"]), 1.0 - b1 ** t, 1.0 - b2 ** t, 0.0]
        return vals

    @torch.no_grad()
    def launch_step(self) -> None:
        """Everything after the backward pass: buckets that were not reduced from the hooks, the norm exchange,
        the update and the all-gather."""
        for e in self.entries:                           # parameters whose hook did not fire in the last backward
            if not e.pop("seen", False):
                g = e["p"].grad
                if g is not None and g.data_ptr() != e["gview"].data_ptr():
                    e["gview"].copy_(g)
                    e["p"].grad = None
                elif g is None and not e.get("filled", False):
                    e["gview"].zero_()
        first = True
        for b in self.buckets:
            if not (b.ready and self.overlap):
                # after the backward pass one barrier covers every bucket that is still to be reduced
                self._reduce_bucket(b, overlapped=False, barrier=first)
                first = False
        if self.fused:
            main = torch.cuda.current_stream(self.device)
            prof = self.profile and not torch.cuda.is_current_stream_capturing()
            if prof:
                for name in ("bwd_end", "joined", "step_end"):
                    self._events[name] = torch.cuda.Event(enable_timing=True)
                self._events["bwd_end"].record(main)
            if self._forked:
                ev = torch.cuda.Event()
                ev.record(self.side)
                main.wait_event(ev)                      # join: every bucket's reduce-scatter has finished
            if prof:
                self._events["joined"].record(main)
            s = main.cuda_stream
            st = self.ctx.status.data_ptr()
            _ext.check(self.lib.cb_sum_partials(self.partials.data_ptr(), self.partials.numel(), self.payload.data_ptr(), s),
                       "sum_partials")
            self.partials.zero_()
            gathered = self.ctx.barrier(self.payload)
            code = self.lib.cb_adamw_shard_allgather_table(
                self.param_buf.ptrs, self.world, self.rank, self.shard, self.chunk_off.data_ptr(),
                self.reduced.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), _ext.ptr(self.master),
                self.chunk_group.data_ptr(), self.hyper.data_ptr(), gathered.data_ptr(),
                float(self.max_grad_norm or 0.0), self.norm_out.data_ptr(), st, s)
            _ext.check(code, "adamw_shard_allgather")
            _ext.count_launch(2)
            self.ctx.barrier()
            self.last_grad_norm = self.norm_out[1]
            if prof:
                self._events["step_end"].record(main)
        else:
            self._step_reference()
        self._reset_pending()
        self.accumulating = False

    def _step_reference(self) -> None:
        tot = self.sq_total.clone()
        dist.all_reduce(tot, group=self.group)
        self.sq_total.zero_()
        norm = tot.sqrt()
        clip = (self.max_grad_norm / (norm + 1e-6)).clamp(max=1.0) if self.max_grad_norm else torch.ones_like(norm)
        t = self.step_count
        mine = self._gather_local(self.param_flat)
        w = self.master if self.master is not None else mine.float()
        new = torch.empty_like(w)
        groups = self.chunk_group.long().repeat_interleave(CHUNK)
        for gi, g in enumerate(self.param_groups):
            sel = groups == gi
            if not bool(sel.any()):
                continue
            b1, b2 = g["betas"]
            gr = self.reduced[sel] * clip
            x = w[sel] * (1.0 - g["lr"] * g["weight_decay"])
            m = self.exp_avg[sel].mul_(b1).add_(gr, alpha=1 - b1)
            v = self.exp_avg_sq[sel].mul_(b2).addcmul_(gr, gr, value=1 - b2)
            self.exp_avg[sel], self.exp_avg_sq[sel] = m, v
            x = x - (g["lr"] / (1 - b1 ** t)) * m / ((v / (1 - b2 ** t)).sqrt() + g["eps"])
            new[sel] = x
        if self.master is not None:
            self.master.copy_(new)
        new = new.to(self.dtype)
        parts = [torch.empty_like(new) for _ in range(self.world)]
        dist.all_gather(parts, new, group=self.group)
        for r, part in enumerate(parts):                 # the all-gather: every rank's slices go back into place
            for b in self.buckets:
                lo, hi = self._slice(b, r)
                self.param_flat[lo:hi].copy_(part[b.loc: b.loc + b.shard])
        self.last_grad_norm = norm.squeeze(0)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.prepare_step()
        self.launch_step()
        return loss

    def profile_report(self) -> Dict[str, Any]:
        """Timings of the last profiled step (synchronises): per bucket the reduce-scatter's duration and how
        long after the bucket's last gradient it finished; for the step the time the main stream spent waiting
        for the side stream after the backward pass (exposed reduce-scatter) and the norm exchange + update +
        all-gather tail."""
        if not self._events or "bwd_end" not in self._events:
            return {}
        torch.cuda.synchronize(self.device)
        e = self._events
        rows = []
        for i, (a, b, overlapped) in sorted(e.get("buckets", {}).items()):
            rows.append({"bucket": i, "mb": round((self.buckets[i].hi - self.buckets[i].lo) * 2 / 2**20, 1),
                         "overlapped": bool(overlapped), "rs_ms": round(a.elapsed_time(b), 4),
                         "ready_to_done_ms": round(e["ready"][i].elapsed_time(b), 4),
                         "done_before_bwd_end_ms": round(b.elapsed_time(e["bwd_end"]), 4)})
        extra = {}
        if "micro_start" in e:                       # backward pass of the last micro-step on the main stream
            extra["bwd_ms"] = round(e["micro_start"].elapsed_time(e["bwd_end"]), 4)
        return {**extra, "buckets": rows, "exposed_wait_ms": round(e["bwd_end"].elapsed_time(e["joined"]), 4),
                "tail_ms": round(e["joined"].elapsed_time(e["step_end"]), 4),
                "hidden_rs_ms": round(sum(r["rs_ms"] for r in rows if r["done_before_bwd_end_ms"] >= 0), 4)}

    def zero_grad(self, set_to_none: bool = True) -> None:
        """Gradients live in the flat buffer: discarding them means that the next backward pass overwrites its
        slots instead of adding to them (as ``step()`` arranges by itself for the gradients it consumed)."""
        for e in self.entries:
            e["p"].grad = None
            e["filled"] = False
        self._reset_pending()

    # ------------------------------------------------------------------------------------------ state
    def state_dict(self) -> Dict[str, Any]:
        """This rank's shard of the optimizer state (one file per rank)."""
        return {"kind": "zero1", "step_count": self.step_count, "rank": self.rank, "world": self.world,
                "total": self.total, "layout": [(e["off"], e["n"]) for e in self.entries],
                "buckets": [(b.lo, b.hi) for b in self.buckets],
                "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
                "master": self.master.cpu() if self.master is not None else None,
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd.get("world") != self.world or sd.get("total") != self.total:
            return self.load_resharded([sd]) if sd.get("world") == 1 else self._mismatch()
        self.step_count = int(sd["step_count"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        if self.master is not None and sd.get("master") is not None:
            self.master.copy_(sd["master"])
        self._load_groups(sd)

    @staticmethod
    def _mismatch():
        raise ValueError("sharded optimizer state was written with a different world size; pass the states of all "
                         "saved ranks to load_resharded()")

    def _load_groups(self, sd) -> None:
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update({k: v for k, v in saved.items() if k in ("lr", "weight_decay", "betas", "eps")})

    def load_resharded(self, states: List[Dict[str, Any]]) -> None:
        """Restart at a different number of ranks: ``states`` are the ``state_dict()`` of every rank of the run that
        wrote the checkpoint (any order)."""
        self.load_consolidated(consolidate_states(states))
        self._load_groups(states[0])

    def load_consolidated(self, per_tensor: Dict[str, Any]) -> None:
        """Load a world-size-independent state: one fp32 tensor per parameter (parameter order) for every state
        vector, as produced by :func:`consolidate_states` or by the other optimizers' consolidation helpers."""
        self.step_count = int(per_tensor["step_count"])
        for name, dst in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq), ("master", self.master)):
            vals = per_tensor.get(name)
            if dst is None or vals is None:
                continue
            flat = torch.zeros(self.total, dtype=torch.float32)
            for e, t in zip(self.entries, vals):
                flat[e["off"]: e["off"] + e["n"]] = t.reshape(-1).float()
            dst.copy_(self._gather_local(flat))
        if per_tensor.get("param_groups"):
            self._load_groups(per_tensor)


def consolidate_states(shards: List[Dict[str, Any]]) -> Dict[str, Any]:
    """Per-rank shards → one world-size-independent state: for every state vector a list with one fp32 tensor per
    parameter, in parameter order.  :func:`reshard_state` (or ``ShardedFusedAdamW.load_resharded``) lays those
    out for a new world size."""
    shards = sorted(shards, key=lambda s: s["rank"])
    W = shards[0]["world"]
    if len(shards) != W:
        raise ValueError(f"need the state of all {W} saved ranks, got {len(shards)}")
    total, buckets, layout = shards[0]["total"], shards[0]["buckets"], shards[0]["layout"]
    out: Dict[str, Any] = {"step_count": shards[0]["step_count"], "param_groups": shards[0]["param_groups"],
                           "numels": [n for _, n in layout]}
    for name in ("exp_avg", "exp_avg_sq", "master"):
        if shards[0].get(name) is None:
            out[name] = None
            continue
        flat = torch.zeros(total, dtype=torch.float32)
        for r, s in enumerate(shards):
            loc = 0
            for lo, hi in buckets:
                sh = (hi - lo) // W
                flat[lo + r * sh: lo + (r + 1) * sh] = s[name][loc: loc + sh].float()
                loc += sh
        out[name] = [flat[off: off + n].clone() for off, n in layout]
    return out


def reshard_state(consolidated: Dict[str, Any], optimizer: "ShardedFusedAdamW") -> Dict[str, Any]:
    """The ``state_dict()`` that ``optimizer`` (any world size, same parameters) would have written for the
    consolidated state."""
    sd = optimizer.state_dict()
    sd["step_count"] = consolidated["step_count"]
    for name in ("exp_avg", "exp_avg_sq", "master"):
        vals = consolidated.get(name)
        if vals is None:
            sd[name] = None
            continue
        flat = torch.zeros(optimizer.total, dtype=torch.float32)
        for e, t in zip(optimizer.entries, vals):
            flat[e["off"]: e["off"] + e["n"]] = t
        sd[name] = optimizer._gather_local(flat)
    sd["param_groups"] = consolidated["param_groups"]
    return sd
