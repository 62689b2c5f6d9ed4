"""AdamW with global-norm clipping inside the optimizer, one kernel for all tensors.

API follows the reference's ``FusedAdamW`` (chronicals/optimizers/
fused_adamw.py:104-167 constructor, :221-324 ``step``, :462-471 state dict with a
shared ``step_count``) and its ``FusedAdamWFP8`` (:474-588, fp32 master
weights).  Where the reference launches one Triton kernel per parameter tensor
and reads the clip coefficient back to the host, this implementation:

* on CUDA launches one multi-tensor kernel over a device-resident tensor
  table (``cb_adamw_multi``) and one sum-of-squares kernel pair
  (``cb_grad_clip_coef``) whose clip coefficient stays on the device — a step
  performs no host synchronisation and can be captured in a CUDA graph;
* on CPU runs the same arithmetic in PyTorch (``ops.ref.adamw_step_``).

Moments are always fp32, whatever the parameter dtype.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional

import torch

from ..ops import _ext
from ..ops import ref


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, use_triton: bool = True, use_foreach: bool = True,
                 master_weights: bool = False, extra_sq_norm: Optional[torch.Tensor] = None):
        if lr < 0 or eps < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid AdamW hyper-parameters")
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.max_grad_norm = max_grad_norm
        self.use_kernels = use_triton          # name kept for signature compatibility: selects the fused kernel
        self.use_foreach = use_foreach
        self.master_weights = master_weights
        self.step_count = 0
        self._tables: Dict[Any, Dict[str, Any]] = {}
        self._hyper: Dict[Any, torch.Tensor] = {}
        self._clip_out: Dict[Any, torch.Tensor] = {}
        self.last_grad_norm: Optional[torch.Tensor] = None
        # sum of squared gradients contributed by other ranks/shards (device scalar), added before the sqrt
        self.extra_sq_norm = extra_sq_norm

    # ------------------------------------------------------------------------------------------ state
    def _init_state(self, p: torch.Tensor) -> Dict[str, Any]:
        st = self.state[p]
        if "exp_avg" not in st:
            st["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
            st["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
            if self.master_weights and p.dtype != torch.float32:
                st["master"] = p.detach().float().clone()
        return st

    def ensure_state(self) -> None:
        """Allocate moments (and the device hyper-parameter table) for every trainable parameter
        now, instead of lazily in the first step."""
        for g in self.param_groups:
            for p in g["params"]:
                if p.requires_grad:
                    self._init_state(p)
                    if p.is_cuda:
                        self._hyper_device(p.device)

    def state_dict(self) -> Dict[str, Any]:
        sd = super().state_dict()
        sd["step_count"] = self.step_count
        return sd

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        state_dict = dict(state_dict)
        self.step_count = int(state_dict.pop("step_count", 0))
        super().load_state_dict(state_dict)
        # torch casts every floating-point state tensor to the parameter dtype on load, which would round the fp32
        # moments and master copy of bf16 parameters to bf16 (and halve the buffers the kernels index as fp32):
        # put the saved tensors back unchanged
        saved = state_dict["state"]
        ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for pid, p in zip(ids, params):
            src = saved.get(pid)
            if src is None:
                continue
            for name in ("exp_avg", "exp_avg_sq", "master"):
                t = src.get(name)
                if torch.is_tensor(t):
                    self.state[p][name] = t.detach().to(device=p.device, dtype=torch.float32).clone()
        self._tables.clear()

    def _trainable(self) -> List[torch.Tensor]:
        return [p for g in self.param_groups for p in g["params"] if p.requires_grad]

    def consolidated_state(self) -> Dict[str, Any]:
        """World-size-independent form of the state: one flat fp32 tensor per parameter, in parameter order
        (the exchange format between this optimizer and the sharded ones)."""
        out: Dict[str, Any] = {"step_count": self.step_count, "exp_avg": [], "exp_avg_sq": [], "master": None,
                               "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}
        for p in self._trainable():
            st = self._init_state(p)
            out["exp_avg"].append(st["exp_avg"].detach().reshape(-1).float().cpu())
            out["exp_avg_sq"].append(st["exp_avg_sq"].detach().reshape(-1).float().cpu())
        return out

    def load_consolidated(self, cons: Dict[str, Any]) -> None:
        self.step_count = int(cons["step_count"])
        masters = cons.get("master")
        for i, p in enumerate(self._trainable()):
            st = self._init_state(p)
            st["exp_avg"].copy_(cons["exp_avg"][i].view(p.shape))
            st["exp_avg_sq"].copy_(cons["exp_avg_sq"][i].view(p.shape))
            if masters is not None and "master" in st:
                st["master"].copy_(masters[i].view(p.shape))
        for g, saved in zip(self.param_groups, cons.get("param_groups") or []):
            g.update({k: v for k, v in saved.items() if k in ("lr", "weight_decay", "betas", "eps")})
        self._tables.clear()

    # ------------------------------------------------------------------------------------------ CUDA path
    def _build_table(self, key, plist: List[torch.Tensor], groups: List[int]) -> Dict[str, Any]:
        dev = plist[0].device
        chunk = _ext.lib().cb_opt_chunk()
        sts = [self._init_state(p) for p in plist]
        keep: List[torch.Tensor] = []

        def dev_tensor(values, dtype):
            # pinned staging + async copy: legal while a CUDA graph is being captured (the
            # copy becomes a node that re-reads the pinned buffer, which `keep` holds alive)
            host = torch.tensor(values, dtype=dtype).pin_memory()
            keep.append(host)
            return host.to(dev, non_blocking=True)

        def ptrs(ts):
            return dev_tensor([t.data_ptr() if t is not None else 0 for t in ts], torch.int64)
        numel = [p.numel() for p in plist]
        starts = [0]
        for n in numel:
            starts.append(starts[-1] + (n + chunk - 1) // chunk)
        has_master = any("master" in s for s in sts)
        for p, st in zip(plist, sts):
            for name in ("exp_avg", "exp_avg_sq", "master"):
                t = st.get(name)
                if t is not None and (t.dtype != torch.float32 or t.numel() != p.numel() or not t.is_contiguous()):
                    raise RuntimeError(f"FusedAdamW state '{name}' must be contiguous float32 with {p.numel()} elements, "
                                       f"got {t.dtype} x {t.numel()}")
        tab = {
            "params": plist,
            "p": ptrs(plist), "g": ptrs([p.grad for p in plist]),
            "m": ptrs([s["exp_avg"] for s in sts]), "v": ptrs([s["exp_avg_sq"] for s in sts]),
            "master": ptrs([s.get("master") for s in sts]) if has_master else None,
            "numel": dev_tensor(numel, torch.int64),
            "group": dev_tensor(groups, torch.int32),
            "chunk_start": dev_tensor(starts, torch.int32),
            "_keep": keep,
            "total_chunks": starts[-1], "n": len(plist),
            "partials": torch.empty(starts[-1], dtype=torch.float32, device=dev),
            "grad_ptrs": [p.grad.data_ptr() for p in plist],
            "is_bf16": plist[0].dtype == torch.bfloat16,
        }
        self._tables[key] = tab
        return tab

    def _hyper_device(self, dev) -> torch.Tensor:
        h = self._hyper.get(dev)
        if h is None:
            h = torch.zeros(len(self.param_groups) * 8, dtype=torch.float32, device=dev)
            self._hyper[dev] = h
        return h

    def prepare_step(self) -> None:
        """Host half of a step: advance the step counter and refresh the device copy of the
        per-group hyper-parameters (learning rate from the scheduler, bias corrections).
        Not capturable; when the device half is replayed from a CUDA graph, call this before
        every replay."""
        self.step_count += 1
        t = self.step_count
        vals: List[float] = []
        for g in self.param_groups:
            b1, b2 = g["betas"]
            vals += [float(g["lr"]), float(g["weight_decay"]), b1, b2, float(g["eps"]),
                     1.0 - b1 ** t, 1.0 - b2 ** t, 0.0]
        host = torch.tensor(vals, dtype=torch.float32)
        for dev, h in self._hyper.items():
            if h.numel() != host.numel():
                self._hyper[dev] = h = torch.zeros(host.numel(), dtype=torch.float32, device=dev)
            h.copy_(host, non_blocking=True)      # pageable source: staged before the call returns

    def _step_cuda(self, key, plist, groups) -> None:
        L = _ext.lib()
        tab = self._tables.get(key)
        if tab is None or tab["n"] != len(plist) or any(a is not b for a, b in zip(tab["params"], plist)):
            tab = self._build_table(key, plist, groups)
        else:
            gp = [p.grad.data_ptr() for p in plist]
            if gp != tab["grad_ptrs"]:
                # gradients were re-allocated (zero_grad(set_to_none=True)): only the pointer array changes.
                # The table holds no reference to the gradient tensors, so last step's buffers are free by now.
                host = torch.tensor(gp, dtype=torch.int64).pin_memory()
                tab["_keep_g"] = host
                tab["g"].copy_(host, non_blocking=True)
                tab["grad_ptrs"] = gp
        tab["hyper"] = self._hyper_device(plist[0].device)
        out = self._clip_out.get(key)
        if out is None:
            out = torch.zeros(3, dtype=torch.float32, device=plist[0].device)
            self._clip_out[key] = out
        s = _ext.stream_ptr()
        clip_ptr = None
        if self.max_grad_norm and self.max_grad_norm > 0:
            code = L.cb_grad_clip_coef(tab["g"].data_ptr(), tab["numel"].data_ptr(), tab["chunk_start"].data_ptr(),
                                       tab["n"], tab["total_chunks"], tab["partials"].data_ptr(),
                                       _ext.ptr(self.extra_sq_norm), float(self.max_grad_norm), out.data_ptr(),
                                       int(tab["is_bf16"]), s)
            _ext.check(code, "grad_clip_coef")
            clip_ptr = out[2:].data_ptr()
            self.last_grad_norm = out[1]
        code = L.cb_adamw_multi(tab["p"].data_ptr(), tab["g"].data_ptr(), tab["m"].data_ptr(), tab["v"].data_ptr(),
                                tab["master"].data_ptr() if tab["master"] is not None else None,
                                tab["numel"].data_ptr(), tab["group"].data_ptr(), tab["chunk_start"].data_ptr(),
                                tab["n"], tab["total_chunks"], tab["hyper"].data_ptr(), clip_ptr,
                                int(tab["is_bf16"]), s)
        _ext.check(code, "adamw_multi")

    # ------------------------------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:          # make sure the hyper table exists on every device in use
            for p in group["params"]:
                if p.is_cuda and p.grad is not None:
                    self._hyper_device(p.device)
        self.prepare_step()
        self.launch_step()
        return loss

    @torch.no_grad()
    def launch_step(self) -> None:
        """Device half of a step (kernel launches only; capturable in a CUDA graph)."""
        buckets: Dict[Any, Any] = {}
        cpu_items = []
        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("FusedAdamW does not support sparse gradients")
                fast = (p.is_cuda and self.use_kernels and p.dtype in (torch.bfloat16, torch.float32)
                        and p.grad.dtype == p.dtype and p.is_contiguous() and p.grad.is_contiguous())
                if fast:
                    key = (p.device.index, p.dtype)
                    b = buckets.setdefault(key, ([], []))
                    b[0].append(p)
                    b[1].append(gi)
                else:
                    cpu_items.append((gi, p))
        if buckets and len(buckets) > 1 and self.max_grad_norm and self.max_grad_norm > 0:
            # mixed dtypes: the norm must span every tensor, so fall back to the reference arithmetic
            for key, (plist, groups) in buckets.items():
                cpu_items.extend(zip(groups, plist))
            buckets = {}
        for key, (plist, groups) in buckets.items():
            self._step_cuda(key, plist, groups)
        if cpu_items:
            self._step_reference(cpu_items)

    def _step_reference(self, items) -> None:
        clip = 1.0
        if self.max_grad_norm and self.max_grad_norm > 0:
            sq = torch.zeros((), dtype=torch.float32, device=items[0][1].device)
            for _, p in items:
                sq = sq + p.grad.float().pow(2).sum()
            if self.extra_sq_norm is not None:
                sq = sq + self.extra_sq_norm.to(sq.device).reshape(())
            self.last_grad_norm = sq.sqrt()
            clip = ref.clip_coef_from_sqnorm(sq, self.max_grad_norm)
        for gi, p in items:
            g = self.param_groups[gi]
            st = self._init_state(p)
            b1, b2 = g["betas"]
            ref.adamw_step_(p, p.grad, st["exp_avg"], st["exp_avg_sq"], self.step_count, g["lr"], b1, b2, g["eps"],
                            g["weight_decay"], clip, st.get("master"))


class FusedAdamWFP8(FusedAdamW):
    """AdamW keeping fp32 master weights for low-precision parameters
    (reference fused_adamw.py:474-588)."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 1.0, **kw):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         max_grad_norm=max_grad_norm, master_weights=True, **kw)


def benchmark_optimizer(num_params: int = 50_000_000, steps: int = 10, device: str = "cuda") -> Dict[str, float]:
    """Times ``FusedAdamW`` against ``torch.optim.AdamW(fused=True)`` with CUDA events."""
    if not torch.cuda.is_available():
        return {}
    res = {}
    for name in ("fused_adamw", "torch_fused"):
        p = torch.nn.Parameter(torch.randn(num_params, device=device, dtype=torch.bfloat16))
        p.grad = torch.randn_like(p)
        opt = FusedAdamW([p], lr=1e-4) if name == "fused_adamw" else torch.optim.AdamW([p], lr=1e-4, fused=True)
        for _ in range(3):
            opt.step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            opt.step()
        b.record()
        torch.cuda.synchronize()
        res[name + "_ms"] = a.elapsed_time(b) / steps
    return res
