"""ZeRO-3: parameters, gradients and optimizer state sharded over the data-parallel ranks.

The reference has no sharding of any kind (single GPU; its config only carries a placeholder flag,
chronicals/config/config.py:525-526), so this module is new.

Units.  The model is cut into units — one per decoder layer plus one "outer" unit (embedding, final norm,
LM head).  Each unit's parameters are laid out in one flat bf16 vector of which rank r permanently keeps
only slice r (its *shard*, in peer-mapped symmetric memory) together with fp32 AdamW moments for that
slice.  The full vector exists on a rank only while the unit computes:

* before a unit's forward (and again before its backward) the full vector is re-materialised by
  ``allgather_pull`` — one kernel that reads the W shards straight out of the peers' memory over NVLink.
  Shards change only in the optimizer step, which ends with a barrier, so the pulls need no flags.  The
  pull of the next unit runs on a side stream while the current unit computes.
* the unit's parameters are views of that full vector; after use its storage is released
  (``untyped_storage().resize_(0)``) and re-created before the backward — views saved by autograd stay valid.
* gradients accumulate into a per-unit slot of a symmetric gradient buffer (two slots, alternating).  When
  the next unit's backward starts, the finished unit is reduce-scattered: a barrier, then
  ``rs_reduce_sqnorm`` pulls this rank's slice from all W gradient buffers, averages in fp32, keeps the
  result for the optimizer and adds to the squared-norm share.
* ``step()``: one barrier exchanges the norm shares, then ``adamw_shard_local`` updates each shard in place.

On CPU (gloo) the same control flow runs on ``torch.distributed`` collectives — that path is the test
oracle of the bookkeeping; the kernels are tested on GPUs against the unsharded optimizer.
"""
from __future__ import annotations

import ctypes
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _ext

ALIGN = 1024


class _Unit:
    def __init__(self, name: str, params: List[nn.Parameter], world: int):
        self.name = name
        self.params = params
        self.offsets: List[int] = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + 7) // 8 * 8
        unit = ALIGN * world
        self.n = (off + unit - 1) // unit * unit
        self.shard_n = self.n // world
        self.full: Optional[torch.Tensor] = None        # flat bf16 [n]; storage released between uses
        self.resident = False
        self.gather_event: Optional[torch.cuda.Event] = None
        self.grad_slot: Optional[int] = None             # which gradient buffer holds this unit's gradients
        self.pending_reduce = False


class Zero3Engine:
    """Wraps a ``CausalLM``; owns the shards and the optimizer.  Usage per step::

        loss = engine.forward_backward(input_ids, labels=labels)
        engine.step()
    """

    def __init__(self, model: nn.Module, lr: float = 1e-5, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, group=None, wait_budget_us: int = 2_000_000, prefetch: bool = True,
                 backend: str = "fused"):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("ZeRO-3 needs an initialised process group")
        self.model = model
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, tuple(betas), eps, weight_decay, max_grad_norm
        self.step_count = 0
        p0 = next(model.parameters())
        self.device, self.dtype = p0.device, p0.dtype
        # "fused": gathers and reduce-scatters are peer-memory kernels; "nccl": the same schedule on
        # all_gather_into_tensor / reduce_scatter_tensor (the comparison arm; the compute kernels are the same)
        self.fused = self.device.type == "cuda" and backend == "fused"
        self.nccl = self.device.type == "cuda" and backend != "fused"
        if self.device.type == "cuda" and self.dtype != torch.bfloat16:
            raise ValueError("the GPU ZeRO-3 paths handle bf16 parameters")
        self.prefetch = prefetch and self.device.type == "cuda"
        layers = list(model.model.layers)
        outer = [p for n, p in model.named_parameters() if not n.startswith("model.layers.")]
        self.units: List[_Unit] = [_Unit("outer", outer, self.world)]
        self.units += [_Unit(f"layer{i}", list(l.parameters()), self.world) for i, l in enumerate(layers)]
        self.layer_units = self.units[1:]
        self._build_shards(wait_budget_us)
        self._install_hooks(layers)
        self.last_grad_norm: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------------------------------ set-up
    def _build_shards(self, wait_budget_us: int) -> None:
        W, r, dev = self.world, self.rank, self.device
        if self.fused:
            from . import symm
            self.symm = symm
            self.ctx = symm.SymmetricContext(self.group, wait_budget_us)
            self.status = self.ctx.status
            self.lib = symm._lib()
            for name, args in (("cb_allgather_pull", [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p,
                                                       ctypes.c_void_p, ctypes.c_void_p]),
                               ("cb_adamw_shard_local", [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong] + [ctypes.c_void_p] * 7
                                + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p])):
                fn = getattr(self.lib, name)
                fn.argtypes, fn.restype = args, ctypes.c_int
            self.side = torch.cuda.Stream(device=dev)
        elif self.nccl:
            from . import symm
            self.lib = symm._lib()
            fn = self.lib.cb_adamw_shard_local
            fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong] + [ctypes.c_void_p] * 7 + [
                ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
            fn.restype = ctypes.c_int
            self.status = _ext.status_buffer(dev)
            self.side = torch.cuda.Stream(device=dev)
        max_layer_n = max((u.n for u in self.layer_units), default=ALIGN * W)
        for u in self.units:
            flat = torch.zeros(u.n, dtype=self.dtype, device=dev)
            for p, off in zip(u.params, u.offsets):
                flat[off:off + p.numel()].copy_(p.data.reshape(-1))
            lo = r * u.shard_n
            if self.fused:
                u.shard = self.symm.SymmetricBuffer(u.shard_n, torch.bfloat16, self.group)
                u.shard.local.copy_(flat[lo:lo + u.shard_n])
                u.shard_t = u.shard.local
            else:
                u.shard_t = flat[lo:lo + u.shard_n].clone()
            u.exp_avg = torch.zeros(u.shard_n, dtype=torch.float32, device=dev)
            u.exp_avg_sq = torch.zeros(u.shard_n, dtype=torch.float32, device=dev)
            u.reduced = torch.zeros(u.shard_n, dtype=torch.float32, device=dev)
            u.chunk_group = torch.zeros(u.shard_n // ALIGN, dtype=torch.uint8, device=dev)
            u.full = torch.empty(u.n, dtype=self.dtype, device=dev)
            for p, off in zip(u.params, u.offsets):
                p.data = u.full[off:off + p.numel()].view(p.shape)
            self._release(u)
            del flat
        # gradient buffers: two alternating slots for the layers, one for the outer unit
        if self.fused:
            self.gslots = [self.symm.SymmetricBuffer(max_layer_n, torch.bfloat16, self.group) for _ in range(2)]
            self.gouter = self.symm.SymmetricBuffer(self.units[0].n, torch.bfloat16, self.group)
            self.gslot_t = [b.local for b in self.gslots]
            self.gouter_t = self.gouter.local
            self.partials = torch.zeros(self.ctx.grid, dtype=torch.float32, device=dev)
            self.payload = torch.zeros(self.ctx.payload_floats, dtype=torch.float32, device=dev)
            self.hyper = torch.zeros(8, dtype=torch.float32, device=dev)
            self.norm_out = torch.zeros(3, dtype=torch.float32, device=dev)
        else:
            self.gslot_t = [torch.zeros(max_layer_n, dtype=self.dtype, device=dev) for _ in range(2)]
            self.gouter_t = torch.zeros(self.units[0].n, dtype=self.dtype, device=dev)
            if self.nccl:
                self.hyper = torch.zeros(8, dtype=torch.float32, device=dev)
                self.norm_out = torch.zeros(3, dtype=torch.float32, device=dev)
                self.gathered = torch.zeros(self.world * 4, dtype=torch.float32, device=dev)
                self.rs_out = torch.zeros(max(u.shard_n for u in self.units), dtype=self.dtype, device=dev)
        self.sq_total = torch.zeros(1, dtype=torch.float32, device=dev)
        if self.fused:
            torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _install_hooks(self, layers) -> None:
        for i, layer in enumerate(layers):
            layer.register_forward_pre_hook(lambda m, a, i=i: self._before_forward(i))
            layer.register_forward_hook(lambda m, a, o, i=i: self._after_forward(i))
            layer.register_full_backward_pre_hook(lambda m, g, i=i: self._before_backward(i))

    # ------------------------------------------------------------------------------------------ parameters
    def _release(self, u: _Unit) -> None:
        u.full.untyped_storage().resize_(0)
        u.resident = False
        u.gather_event = None

    def _gather(self, u: _Unit, side: bool) -> None:
        """Re-materialise the unit's full parameter vector from all ranks' shards."""
        if u.resident:
            return
        nbytes = u.n * u.full.element_size()
        u.full.untyped_storage().resize_(nbytes)
        if self.fused:
            main = torch.cuda.current_stream()
            stream = self.side if (side and self.prefetch) else main
            if stream is not main:
                stream.wait_stream(main)            # the block may be recycled memory still in use by queued work
            with torch.cuda.stream(stream):
                code = self.lib.cb_allgather_pull(u.shard.ptrs, self.world, u.shard_n, u.full.data_ptr(),
                                                  self.status.data_ptr(), stream.cuda_stream)
                _ext.check(code, "allgather_pull")
                if stream is not main:
                    u.gather_event = torch.cuda.Event()
                    u.gather_event.record(stream)
        elif self.nccl:
            main = torch.cuda.current_stream()
            stream = self.side if (side and self.prefetch) else main
            if stream is not main:
                stream.wait_stream(main)
            with torch.cuda.stream(stream):
                dist.all_gather_into_tensor(u.full, u.shard_t, group=self.group)
                if stream is not main:
                    u.gather_event = torch.cuda.Event()
                    u.gather_event.record(stream)
        else:
            parts = [torch.empty_like(u.shard_t) for _ in range(self.world)]
            dist.all_gather(parts, u.shard_t, group=self.group)
            u.full.copy_(torch.cat(parts))
        u.resident = True

    def _wait(self, u: _Unit) -> None:
        if u.gather_event is not None:
            torch.cuda.current_stream().wait_event(u.gather_event)
            u.gather_event = None

    def _before_forward(self, i: int) -> None:
        u = self.layer_units[i]
        self._gather(u, side=False)
        self._wait(u)
        if i + 1 < len(self.layer_units):
            self._gather(self.layer_units[i + 1], side=True)

    def _after_forward(self, i: int) -> None:
        if torch.is_grad_enabled() and i == len(self.layer_units) - 1:
            return                                  # the last layer is the first one the backward needs
        self._release(self.layer_units[i])

    # ------------------------------------------------------------------------------------------ gradients
    def _assign_grads(self, u: _Unit, buf: torch.Tensor) -> None:
        buf[: u.n].zero_()
        for p, off in zip(u.params, u.offsets):
            p.grad = buf[off:off + p.numel()].view(p.shape)

    def _before_backward(self, i: int) -> None:
        u = self.layer_units[i]
        nxt = i + 1                                   # the unit whose backward has just finished
        if nxt < len(self.layer_units) and self.layer_units[nxt].pending_reduce:
            self._reduce_unit(self.layer_units[nxt])
        self._gather(u, side=False)
        self._wait(u)
        if i - 1 >= 0:
            self._gather(self.layer_units[i - 1], side=True)
        u.grad_slot = i % 2
        self._assign_grads(u, self.gslot_t[u.grad_slot])
        u.pending_reduce = True

    def _reduce_unit(self, u: _Unit) -> None:
        """Reduce-scatter (average) the unit's gradients into ``u.reduced`` (fp32, my slice)."""
        lo, hi = self.rank * u.shard_n, (self.rank + 1) * u.shard_n
        if self.fused:
            buf = self.gouter if u is self.units[0] else self.gslots[u.grad_slot]
            self.ctx.barrier()                        # every rank has finished this unit's backward
            code = self.lib.cb_rs_reduce_sqnorm(buf.ptrs, self.world, lo, hi, u.reduced.data_ptr(), self.partials.data_ptr(),
                                                self.payload.data_ptr(), self.status.data_ptr(), _ext.stream_ptr())
            _ext.check(code, "rs_reduce_sqnorm")
            self.sq_total += self.payload[0]
        elif self.nccl:
            buf_t = self.gouter_t if u is self.units[0] else self.gslot_t[u.grad_slot]
            out = self.rs_out[: u.shard_n]
            dist.reduce_scatter_tensor(out, buf_t[: u.n], op=dist.ReduceOp.AVG, group=self.group)
            u.reduced.copy_(out)
            self.sq_total += u.reduced.pow(2).sum()
        else:
            buf_t = self.gouter_t if u is self.units[0] else self.gslot_t[u.grad_slot]
            g = buf_t[: u.n].float()
            dist.all_reduce(g, group=self.group)
            u.reduced.copy_(g[lo:hi] / self.world)
            self.sq_total += u.reduced.pow(2).sum()
        for p in u.params:
            p.grad = None
        u.pending_reduce = False
        if u is not self.units[0]:
            self._release(u)

    # ------------------------------------------------------------------------------------------ step API
    def forward_backward(self, input_ids: torch.Tensor, labels: torch.Tensor, **kw) -> torch.Tensor:
        outer = self.units[0]
        self.sq_total.zero_()
        self._gather(outer, side=False)
        self._assign_grads(outer, self.gouter_t)
        outer.pending_reduce = True
        loss = self.model(input_ids, labels=labels, **kw).loss
        loss.backward()
        if self.layer_units and self.layer_units[0].pending_reduce:
            self._reduce_unit(self.layer_units[0])
        self._reduce_unit(outer)
        self._release(outer)
        return loss.detach()

    @torch.no_grad()
    def forward_only(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None, **kw):
        """Evaluation forward: units are gathered and released by the same hooks, nothing is kept for a backward."""
        outer = self.units[0]
        self._gather(outer, side=False)
        out = self.model(input_ids, labels=labels, **kw)
        for u in self.units:
            if u.resident:
                self._release(u)
        return out

    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        t = self.step_count
        b1, b2 = self.betas
        if self.fused:
            self.hyper.copy_(torch.tensor([self.lr, self.weight_decay, b1, b2, self.eps, 1.0 - b1 ** t, 1.0 - b2 ** t, 0.0],
                                          dtype=torch.float32), non_blocking=True)
            self.payload.zero_()
            self.payload[0:1].copy_(self.sq_total)
            gathered = self.ctx.barrier(self.payload)
            for u in self.units:
                code = self.lib.cb_adamw_shard_local(u.shard_t.data_ptr(), self.world, u.shard_n, u.reduced.data_ptr(),
                                                     u.exp_avg.data_ptr(), u.exp_avg_sq.data_ptr(), None,
                                                     u.chunk_group.data_ptr(), self.hyper.data_ptr(), gathered.data_ptr(),
                                                     float(self.max_grad_norm or 0.0), self.norm_out.data_ptr(),
                                                     self.status.data_ptr(), _ext.stream_ptr())
                _ext.check(code, "adamw_shard_local")
            self.ctx.barrier()                        # new shards are visible before anyone pulls them
            self.last_grad_norm = self.norm_out[1]
            return
        tot = self.sq_total.clone()
        dist.all_reduce(tot, group=self.group)
        if self.nccl:
            # the update kernel of the fused path, fed with the all-reduced squared norm in slot 0
            self.hyper.copy_(torch.tensor([self.lr, self.weight_decay, b1, b2, self.eps, 1.0 - b1 ** t, 1.0 - b2 ** t, 0.0],
                                          dtype=torch.float32), non_blocking=True)
            self.gathered.zero_()
            self.gathered[0:1].copy_(tot)
            for u in self.units:
                code = self.lib.cb_adamw_shard_local(u.shard_t.data_ptr(), self.world, u.shard_n, u.reduced.data_ptr(),
                                                     u.exp_avg.data_ptr(), u.exp_avg_sq.data_ptr(), None,
                                                     u.chunk_group.data_ptr(), self.hyper.data_ptr(),
                                                     self.gathered.data_ptr(), float(self.max_grad_norm or 0.0),
                                                     self.norm_out.data_ptr(), self.status.data_ptr(), _ext.stream_ptr())
                _ext.check(code, "adamw_shard_local")
            self.last_grad_norm = self.norm_out[1]
            return
        norm = tot.sqrt()
        clip = (self.max_grad_norm / (norm + 1e-6)).clamp(max=1.0) if self.max_grad_norm else torch.ones_like(norm)
        for u in self.units:
            g = u.reduced * clip
            w = u.shard_t.float() * (1.0 - self.lr * self.weight_decay)
            u.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
            u.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
            w -= (self.lr / (1 - b1 ** t)) * u.exp_avg / ((u.exp_avg_sq / (1 - b2 ** t)).sqrt() + self.eps)
            u.shard_t.copy_(w.to(u.shard_t.dtype))
        self.last_grad_norm = norm.squeeze(0)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------------------------------ state
    @torch.no_grad()
    def gather_full_state_dict(self) -> Dict[str, torch.Tensor]:
        """HuggingFace-named full tensors on every rank (checkpoint consolidation; collective, not hot)."""
        for u in self.units:
            self._gather(u, side=False)
        if self.fused:
            torch.cuda.synchronize()
        sd = {k: v.detach().clone() for k, v in self.model.hf_state_dict().items()}
        for u in self.units:
            self._release(u)
        return sd

    def _param_order(self) -> Dict[int, int]:
        return {id(p): i for i, p in enumerate(p for p in self.model.parameters() if p.requires_grad)}

    def state_dict(self) -> Dict[str, Any]:
        """This rank's optimizer shard.  ``layout`` lists, per unit, (offset in the unit's flat vector, numel,
        index of the parameter in ``model.parameters()`` order) so that other layouts can re-assemble it."""
        order = self._param_order()
        return {"kind": "zero3", "step_count": self.step_count, "rank": self.rank, "world": self.world,
                "units": [{"name": u.name, "exp_avg": u.exp_avg.cpu(), "exp_avg_sq": u.exp_avg_sq.cpu(),
                           "shard": u.shard_t.detach().cpu(),
                           "layout": [(off, p.numel(), order[id(p)]) for p, off in zip(u.params, u.offsets)]}
                          for u in self.units]}

    def load_consolidated(self, cons: Dict[str, Any]) -> None:
        """Load per-parameter state tensors (``model.parameters()`` order) written by any optimizer layout; the
        weights themselves come from :meth:`load_full_state_dict`."""
        order = self._param_order()
        self.step_count = int(cons["step_count"])
        for u in self.units:
            for name, dst in (("exp_avg", u.exp_avg), ("exp_avg_sq", u.exp_avg_sq)):
                flat = torch.zeros(u.n, dtype=torch.float32)
                for p, off in zip(u.params, u.offsets):
                    flat[off:off + p.numel()] = cons[name][order[id(p)]].reshape(-1).float()
                dst.copy_(flat[self.rank * u.shard_n:(self.rank + 1) * u.shard_n])

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd["world"] != self.world:
            raise ValueError("ZeRO-3 state was written with a different world size; pass the states of all saved "
                             "ranks to load_resharded()")
        self.step_count = int(sd["step_count"])
        for u, s in zip(self.units, sd["units"]):
            u.exp_avg.copy_(s["exp_avg"])
            u.exp_avg_sq.copy_(s["exp_avg_sq"])
            u.shard_t.copy_(s["shard"])

    def load_resharded(self, states: List[Dict[str, Any]]) -> None:
        """Restart at a different number of ranks: ``states`` are the ``state_dict()`` of every rank of the run
        that wrote the checkpoint.  Each unit's flat vectors are re-assembled in rank order and re-sliced for this
        world size (the tail padding of a unit depends on the world size and holds zeros)."""
        states = sorted(states, key=lambda s: s["rank"])
        if len(states) != states[0]["world"]:
            raise ValueError(f"need the state of all {states[0]['world']} saved ranks, got {len(states)}")
        self.step_count = int(states[0]["step_count"])
        lo = self.rank
        for ui, u in enumerate(self.units):
            for name, dst in (("exp_avg", u.exp_avg), ("exp_avg_sq", u.exp_avg_sq), ("shard", u.shard_t)):
                flat = torch.cat([s["units"][ui][name].reshape(-1) for s in states])
                if flat.numel() < u.n:
                    flat = torch.cat((flat, torch.zeros(u.n - flat.numel(), dtype=flat.dtype)))
                dst.copy_(flat[lo * u.shard_n:(lo + 1) * u.shard_n].to(dst.dtype))

    @torch.no_grad()
    def load_full_state_dict(self, hf_state: Dict[str, torch.Tensor]) -> None:
        """Scatter full (HuggingFace-named) tensors into the shards: units are made resident, the model copies
        the tensors into its parameter views, and every rank keeps its slice."""
        for u in self.units:
            self._gather(u, side=False)
        if self.fused:
            torch.cuda.synchronize()
        self.model.load_hf_state_dict(hf_state, strict=False)
        for u in self.units:
            u.shard_t.copy_(u.full[self.rank * u.shard_n:(self.rank + 1) * u.shard_n])
            self._release(u)
        if self.fused:
            torch.cuda.synchronize()
        dist.barrier(group=self.group)


class Zero3Optimizer(torch.optim.Optimizer):
    """Optimizer-shaped handle on a :class:`Zero3Engine` so that learning-rate schedulers, checkpoint code and the
    trainer loop can treat ZeRO-3 like any other optimizer.  ``param_groups[0]["lr"]`` is copied into the engine
    before every step; gradients live inside the engine, so ``zero_grad`` has nothing to do."""

    def __init__(self, engine: Zero3Engine):
        self.engine = engine
        self._handle = torch.nn.Parameter(torch.zeros(1, device=engine.device), requires_grad=False)
        super().__init__([self._handle], dict(lr=engine.lr, betas=engine.betas, eps=engine.eps,
                                              weight_decay=engine.weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        g = self.param_groups[0]
        self.engine.lr, self.engine.weight_decay = float(g["lr"]), float(g["weight_decay"])
        self.engine.step()
        return None

    def zero_grad(self, set_to_none: bool = True) -> None:
        return None

    @property
    def last_grad_norm(self):
        return self.engine.last_grad_norm

    def state_dict(self):
        return {"zero3": self.engine.state_dict(), "lr": self.param_groups[0]["lr"]}

    def load_state_dict(self, sd) -> None:
        self.engine.load_state_dict(sd["zero3"])
        self.param_groups[0]["lr"] = sd.get("lr", self.param_groups[0]["lr"])

    def load_resharded(self, states) -> None:
        self.engine.load_resharded([s["zero3"] for s in states])
        self.param_groups[0]["lr"] = states[0].get("lr", self.param_groups[0]["lr"])

    def load_consolidated(self, cons) -> None:
        self.engine.load_consolidated(cons)
        groups = cons.get("param_groups") or []
        if groups and "lr" in groups[0]:
            self.param_groups[0]["lr"] = groups[0]["lr"]


def consolidate_zero3_states(states: List[Dict[str, Any]]) -> Dict[str, Any]:
    """``Zero3Engine.state_dict()`` of every saved rank → one fp32 tensor per parameter (``model.parameters()``
    order) for both moments: the exchange format shared with ``FusedAdamW`` and ``ShardedFusedAdamW``."""
    states = sorted((s.get("zero3", s) for s in states), key=lambda s: s["rank"])
    if len(states) != states[0]["world"]:
        raise ValueError(f"need the state of all {states[0]['world']} saved ranks, got {len(states)}")
    n_params = 1 + max(i for u in states[0]["units"] for _, _, i in u["layout"])
    out: Dict[str, Any] = {"step_count": states[0]["step_count"], "master": None, "param_groups": None}
    for name in ("exp_avg", "exp_avg_sq"):
        vals: List[Optional[torch.Tensor]] = [None] * n_params
        for ui, u in enumerate(states[0]["units"]):
            flat = torch.cat([s["units"][ui][name].reshape(-1).float() for s in states])
            for off, n, idx in u["layout"]:
                vals[idx] = flat[off:off + n].clone()
        out[name] = vals
    return out
