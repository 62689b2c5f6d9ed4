"""``ChronicalsTrainer``: the training loop.

Constructor, method names and ``TrainerState`` follow the reference
(chronicals/training/chronicals_trainer.py:367-380 ``TrainerState``, :396-422
constructor, :1447-1504 ``train``, :1665-1844 hot loop, :1982-2105 evaluate /
checkpoints, :2107-2258 diagnostics).  What differs underneath:

* the model is this framework's own packed-layout decoder (HuggingFace-style
  ``nn.Module`` models that return ``.loss`` are still accepted);
* labels are shifted for the fused cross-entropy (the reference passes them
  unshifted to its cut-cross-entropy);
* no per-micro-step ``loss.item()``: losses accumulate on the device and are
  read once per logging interval;
* the whole micro-step (forward, backward, clip, AdamW) can be captured in one
  CUDA graph and replayed (``use_cuda_graphs=True``), with the host only copying
  the next batch into static buffers;
* data parallelism: gradients are reduced across ranks by
  ``chronicals_b200.parallel`` when ``torch.distributed`` is initialised;
* checkpoints are safetensors under HuggingFace names with RNG state, data
  cursor and ``save_total_limit`` pruning.
"""
from __future__ import annotations

import gc
import json
import math
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Union

import torch
import torch.nn as nn

from ..checkpoint import io as ckpt_io
from ..config.config import ChronicalsConfig, TrainingConfig
from ..data.sequence_packer import PackedBatch
from ..optimizers.fused_adamw import FusedAdamW
from ..optimizers.optimizers import ScheduleFreeAdamW, create_optimizer, create_scheduler


@dataclass
class TrainerState:
    global_step: int = 0
    epoch: int = 0
    best_loss: float = float("inf")
    total_tokens: int = 0
    total_time: float = 0.0
    log_history: List[Dict[str, Any]] = field(default_factory=list)
    micro_step: int = 0            # micro-batches consumed over all epochs
    micro_in_epoch: int = 0        # micro-batches consumed in the current epoch (the data cursor for resume)
    real_tokens: int = 0           # tokens that carry a label (padding and masked positions excluded)


def print_chronicals_banner(num_gpus: int = 1, model_name: str = "", extra: Optional[Dict[str, Any]] = None) -> None:
    line = "=" * 64
    print(line)
    print("  CHRONICALS-B200  |  hand-written sm_100a kernels, tcgen05 + TMA + TMEM")
    if model_name:
        print(f"  model: {model_name}")
    print(f"  GPUs: {num_gpus}")
    for k, v in (extra or {}).items():
        print(f"  {k}: {v}")
    print(line)


def _batch_fields(batch: Any) -> Dict[str, Any]:
    """Normalise a batch (PackedBatch | dict | tuple) to a dict of model inputs."""
    if isinstance(batch, PackedBatch):
        return batch.to_dict()
    if isinstance(batch, dict):
        return batch
    if isinstance(batch, (list, tuple)) and len(batch) >= 2:
        return {"input_ids": batch[0], "labels": batch[1]}
    raise TypeError(f"unsupported batch type {type(batch)!r}")


def setup_torch_compile_for_training(model=None, mode: str = "default", **kwargs):
    """API parity with the reference (chronicals_trainer.py:273-364), which tunes ``torch._dynamo`` /
    Inductor flags before compiling the model.  This framework has no tracing compiler on its hot path:
    fusion is done by the hand-written kernels and launch overhead is removed by capturing the step in a
    CUDA graph (``TrainingConfig.use_cuda_graphs``).  Returns the model unchanged plus what was (not) done."""
    return model, {"compiled": False, "mode": mode, "reason": "hand-written kernels + CUDA-graph step replace torch.compile"}


class ChronicalsTrainer:
    def __init__(self, model: nn.Module, args: Union[TrainingConfig, ChronicalsConfig, Any] = None,
                 train_dataloader: Optional[Iterable] = None, eval_dataloader: Optional[Iterable] = None,
                 tokenizer=None, callbacks: Optional[List[Callable]] = None,
                 model_config: Optional[ChronicalsConfig] = None, config=None):
        # README form: ChronicalsTrainer(model, tokenizer, config)
        if config is not None and args is not None and not isinstance(args, (TrainingConfig, ChronicalsConfig)):
            tokenizer, args = args, config
        elif isinstance(train_dataloader, (TrainingConfig, ChronicalsConfig)) and not isinstance(
                args, (TrainingConfig, ChronicalsConfig)):
            tokenizer, args, train_dataloader = args, train_dataloader, None
        if isinstance(args, ChronicalsConfig):
            model_config = model_config or args
            args = args.to_training_config()
        self.model = model
        self.args: TrainingConfig = args if args is not None else TrainingConfig()
        self.train_dataloader = train_dataloader
        self.eval_dataloader = eval_dataloader
        self.tokenizer = tokenizer
        self.callbacks = callbacks or []
        self.model_config = model_config or getattr(model, "config", None)
        self.state = TrainerState()
        self.optimizer = None
        self.scheduler = None
        self._graph = None
        self.graph_kernel_launches = 0
        self._static: Dict[str, torch.Tensor] = {}
        self._loss_acc: Optional[torch.Tensor] = None
        self._setup_training()

    # ==================================================================================== setup
    def _get(self, name: str, default=None):
        return getattr(self.args, name, default)

    def _setup_training(self) -> None:
        a = self.args
        self._active_optimizations: Dict[str, bool] = {}
        # distributed context (initialised by the launcher / parallel.bootstrap)
        import torch.distributed as dist
        # ``args.use_distributed = False`` keeps a trainer single-process inside a multi-rank job
        self.dist = dist if (dist.is_available() and dist.is_initialized()
                             and self._get("use_distributed", True)) else None
        self.rank = self.dist.get_rank() if self.dist else 0
        self.world_size = self.dist.get_world_size() if self.dist else 1
        if torch.cuda.is_available():
            local = int(os.environ.get("LOCAL_RANK", "0")) if self.dist else torch.cuda.current_device()
            self.device = torch.device("cuda", local)
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        if torch.manual_seed is not None and a.seed is not None:
            torch.manual_seed(int(a.seed))
        self.model = self.model.to(self.device)
        self.is_native_model = hasattr(self.model, "hf_state_dict")
        on_gpu = self.device.type == "cuda"
        self._autocast_dtype = torch.bfloat16 if (a.bf16 and on_gpu) else (
            torch.float16 if (self._get("fp16", False) and on_gpu) else None)
        # native model: parameters are already in the compute dtype, no autocast needed
        self._use_autocast = self._autocast_dtype is not None and not self.is_native_model
        if self.is_native_model:
            self.model.z_loss_weight = float(a.z_loss_weight or 0.0)
            self.model.label_smoothing = float(a.label_smoothing or 0.0)
        self._active_optimizations["fused_kernels"] = on_gpu and self.is_native_model
        self._active_optimizations["cut_cross_entropy"] = self.is_native_model
        self._active_optimizations["varlen_attention"] = bool(a.use_flash_varlen)
        self._active_optimizations["sequence_packing"] = bool(a.use_sequence_packing)

        # FP8 (MXFP8 block-scaled GEMMs) for native models on GPU
        self.fp8_context = None
        if a.fp8 and on_gpu and self.is_native_model and self._get("enable_mxfp8", False):
            from ..utils.fp8_deepseek import FP8Context, convert_model_to_fp8
            convert_model_to_fp8(self.model, exclude_patterns=list(a.fp8_exclude_patterns),
                                 mode=str(self._get("fp8_mode", "mxfp8")))
            self.fp8_context = FP8Context(self.model)
        self._active_optimizations["fp8"] = self.fp8_context is not None

        # gradient checkpointing
        if a.use_gradient_checkpointing:
            if hasattr(self.model, "gradient_checkpointing_enable"):
                try:
                    self.model.gradient_checkpointing_enable(ratio=1.0, offload=bool(a.use_activation_offloading))
                except TypeError:
                    self.model.gradient_checkpointing_enable()
            else:
                from .gradient_checkpointing import apply_gradient_checkpointing
                apply_gradient_checkpointing(self.model, a.checkpoint_ratio)
        self._active_optimizations["gradient_checkpointing"] = bool(a.use_gradient_checkpointing)
        self._active_optimizations["activation_offloading"] = bool(a.use_gradient_checkpointing
                                                                   and a.use_activation_offloading
                                                                   and getattr(self.model, "activation_offload", None))

        # packer for raw (un-packed) sample lists handed to train(dataset)
        self.packer = None
        if a.use_sequence_packing:
            from ..data.sequence_packer import SequencePacker
            self.packer = SequencePacker(max_seq_length=a.max_seq_length, strategy=a.packing_strategy,
                                         mask_first_token_of_packed=a.mask_first_token_of_packed)

        if self.world_size > 1 and self._get("broadcast_parameters", True):
            with torch.no_grad():                                  # every rank starts from rank 0's weights
                for p in self.model.parameters():
                    self.dist.broadcast(p.data, src=0)
        # tensor + sequence parallel: every rank keeps 1/tp of the projections and of the vocabulary and sees
        # the same batch; only the replicated norm/embedding gradients are summed across ranks
        self.tp_model = False
        if a.parallel.tp > 1:
            if a.parallel.tp != self.world_size or not self.is_native_model:
                raise ValueError("tensor parallelism needs a native model and parallel.tp == world size "
                                 f"(tp={a.parallel.tp}, world={self.world_size})")
            from ..parallel.tensor_parallel import TensorParallelCausalLM, TPState
            backend = "fused" if (a.parallel.comm_backend == "fused" and self.device.type == "cuda") else "nccl"
            self.model = TensorParallelCausalLM.from_full(self.model, TPState(backend=backend,
                                                                            wait_budget_us=a.parallel.wait_budget_us))
            self.tp_model = True
        self._sharded_optimizer = False
        self._setup_optimizer()
        self.total_steps = self._estimate_total_steps()
        self._setup_scheduler()

        # data-parallel gradient reduction
        self.dp = None
        if self.world_size > 1 and not getattr(self, "_sharded_optimizer", False) and not self.tp_model:
            from ..parallel.data_parallel import GradientReducer
            self.dp = GradientReducer(self.model, backend=a.parallel.comm_backend, bucket_mb=a.parallel.bucket_mb)

        # reporting / profiling
        self.reporter = None
        if a.visual_reporting and self.rank == 0:
            from ..utils.visual_reporter import VisualReporter
            self.reporter = VisualReporter(os.path.join(a.output_dir, "reports"))
        self.profiler = None
        if a.enable_profiling:
            from ..utils.profiling_utils import PerformanceProfiler
            self.profiler = PerformanceProfiler(enabled=True)
        self.num_params = sum(p.numel() for p in self.model.parameters())
        self.flops_per_token = 6 * self.num_params
        # with several ranks the step is captured only when it contains no NCCL call (sharded fused optimizer)
        # (sharded fused optimizer, or adapter buckets reduced by the peer-memory all-reduce)
        no_nccl_in_step = self.world_size == 1 or self._sharded_optimizer or (
            self.dp is not None and getattr(self.dp, "_fused", None) is not None)
        self.use_cuda_graphs = bool(a.use_cuda_graphs) and on_gpu and self.is_native_model \
            and a.gradient_accumulation_steps == 1 and no_nccl_in_step \
            and not self.tp_model and self.zero3 is None
        self._active_optimizations["cuda_graphs"] = self.use_cuda_graphs
        # host-side failure detection: heartbeat over the process-group store, checked before each step
        self.watchdog = None
        if self.world_size > 1 and self._get("use_watchdog", True):
            try:
                from ..parallel.watchdog import watchdog_from_process_group
                self.watchdog = watchdog_from_process_group(timeout=float(self._get("watchdog_timeout_s", 120.0)),
                                                            interval=float(self._get("watchdog_interval_s", 2.0)))
                if self.watchdog is not None:
                    self.watchdog.start()
            except Exception as e:                     # never fatal: the job then relies on collective timeouts
                print(f"[watchdog] disabled: {e}")
                self.watchdog = None
        # tracing: NVTX ranges around the phases and an optional torch.profiler chrome trace
        self._nvtx = bool(a.enable_profiling) and on_gpu
        self._trace = None
        self._log_file = None
        if self.rank == 0 and self._get("log_jsonl", True):
            os.makedirs(a.output_dir, exist_ok=True)
            self._log_file = os.path.join(a.output_dir, "train_log.jsonl")

    def _estimate_total_steps(self) -> int:
        a = self.args
        if a.max_steps and a.max_steps > 0:
            return int(a.max_steps)
        try:
            n = len(self.train_dataloader)  # type: ignore[arg-type]
        except Exception:
            n = 1000
        return max(1, n * max(1, a.num_train_epochs) // max(1, a.gradient_accumulation_steps))

    def _setup_optimizer(self) -> None:
        a = self.args
        t = a.optimizer_type
        self.use_external_grad_clip = True
        self.zero3 = None
        if a.parallel.zero_stage == 3 and self.world_size > 1 and not getattr(self, "tp_model", False):
            # parameters, gradients and AdamW state sharded over the data-parallel ranks (parallel/zero3.py)
            if not self.is_native_model:
                raise ValueError("ZeRO-3 needs a native model")
            if a.gradient_accumulation_steps != 1:
                raise ValueError("ZeRO-3 reduces gradients every micro-step: set gradient_accumulation_steps = 1")
            from ..parallel.zero3 import Zero3Engine, Zero3Optimizer
            self.zero3 = Zero3Engine(self.model, lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                     weight_decay=a.weight_decay, max_grad_norm=a.max_grad_norm,
                                     wait_budget_us=a.parallel.wait_budget_us)
            self.optimizer = Zero3Optimizer(self.zero3)
            self.use_external_grad_clip = False
            self._sharded_optimizer = True           # no separate gradient reducer
            self._active_optimizations["fused_optimizer"] = True
            return
        if self._get("use_lora_plus", False) or t in ("lora_plus", "loraplus"):
            from ..optimizers.lora_plus_optimizer import create_lora_plus_optimizer
            self.optimizer = create_lora_plus_optimizer(
                self.model, base_lr=a.learning_rate, lr_ratio=float(self._get("lora_plus_ratio", 16.0)),
                betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon, weight_decay=a.weight_decay,
                max_grad_norm=a.max_grad_norm)
            self.use_external_grad_clip = False
        elif (t == "fused_adamw" and a.use_fused_adamw and self.world_size > 1 and not getattr(self, "tp_model", False)
              and ((a.parallel.comm_backend == "fused" and self.device.type == "cuda" and self._fused_comm_possible())
                   or (a.parallel.zero_stage == 1 and self.device.type != "cuda"))):
            # optimizer state sharded over the ranks; on GPUs the gradient reduce-scatter (per bucket, from backward
            # hooks), clip, AdamW and parameter all-gather are peer-memory kernels, on CPU ranks the same
            # bookkeeping runs on process-group collectives
            from ..parallel.zero import ShardedFusedAdamW
            self.optimizer = ShardedFusedAdamW([p for p in self.model.parameters() if p.requires_grad],
                                               lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2),
                                               eps=a.adam_epsilon, weight_decay=a.weight_decay,
                                               max_grad_norm=a.max_grad_norm,
                                               wait_budget_us=a.parallel.wait_budget_us,
                                               bucket_mb=a.parallel.shard_bucket_mb,
                                               overlap=a.parallel.overlap_grad_reduce, rs_grid=a.parallel.reduce_grid)
            self.use_external_grad_clip = False
            self._sharded_optimizer = True
        elif t == "fused_adamw" and a.use_fused_adamw:
            # under tensor parallelism the clip coefficient needs the norm over all ranks' shards, computed outside
            self.optimizer = FusedAdamW([p for p in self.model.parameters() if p.requires_grad], lr=a.learning_rate,
                                        betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                        weight_decay=a.weight_decay,
                                        max_grad_norm=0.0 if getattr(self, "tp_model", False) else a.max_grad_norm)
            self.use_external_grad_clip = False      # clipping happens inside the optimizer kernel
        else:
            self.optimizer = create_optimizer(self.model, "adamw" if t == "fused_adamw" else t, lr=a.learning_rate,
                                              weight_decay=a.weight_decay, betas=(a.adam_beta1, a.adam_beta2),
                                              eps=a.adam_epsilon, max_grad_norm=a.max_grad_norm)
        self._active_optimizations["fused_optimizer"] = isinstance(self.optimizer, FusedAdamW)

    def _fused_comm_possible(self) -> bool:
        try:
            from ..parallel import symm
            ok = symm.peer_access_available() and all(p.dtype == torch.bfloat16 for p in self.model.parameters()
                                                      if p.requires_grad)
        except Exception:
            ok = False
        if not ok and self.rank == 0:
            print("[parallel] fused collectives need peer access and bf16 parameters; using the NCCL path")
        return ok

    def _setup_scheduler(self) -> None:
        a = self.args
        if isinstance(self.optimizer, ScheduleFreeAdamW):
            self.scheduler = None
            return
        ws = a.warmup_steps if self._get("warmup_steps", -1) is not None and self._get("warmup_steps", -1) >= 0 else None
        self.scheduler = create_scheduler(self.optimizer, a.lr_scheduler_type, self.total_steps, a.warmup_ratio,
                                          a.lr_min_ratio, a.wsd_stable_ratio, warmup_steps=ws)

    # ==================================================================================== step machinery
    def _prepare_inputs(self, batch: Any) -> Dict[str, Any]:
        f = _batch_fields(batch)
        nb = bool(self.args.non_blocking_transfers)
        out: Dict[str, Any] = {}
        for k in ("input_ids", "labels", "position_ids", "cu_seqlens", "attention_mask"):
            v = f.get(k)
            if isinstance(v, torch.Tensor):
                out[k] = v.to(self.device, non_blocking=nb)
        for k in ("max_seqlen", "seqlens_host"):
            if f.get(k) is not None:
                out[k] = f[k]
        if "labels" not in out and "input_ids" in out:
            out["labels"] = out["input_ids"]
        return out

    def _forward_loss(self, inp: Dict[str, Any]) -> torch.Tensor:
        if self.is_native_model:
            o = self.model(inp["input_ids"], position_ids=inp.get("position_ids"), labels=inp["labels"],
                           cu_seqlens=inp.get("cu_seqlens"), max_seqlen=inp.get("max_seqlen"),
                           seqlens_host=inp.get("seqlens_host"), shift_labels=bool(self._get("shift_labels", True)))
            return o.loss
        kw = {"input_ids": inp["input_ids"], "labels": inp["labels"]}
        if inp.get("attention_mask") is not None and not self.args.use_sequence_packing:
            kw["attention_mask"] = inp["attention_mask"]
        if self._use_autocast:
            with torch.autocast(device_type=self.device.type, dtype=self._autocast_dtype):
                return self.model(**kw).loss
        return self.model(**kw).loss

    def _backward_and_maybe_step(self, loss: torch.Tensor, do_step: bool) -> None:
        a = self.args
        scaled = loss / a.gradient_accumulation_steps if a.gradient_accumulation_steps > 1 else loss
        if hasattr(self.optimizer, "begin_micro_step"):
            self.optimizer.begin_micro_step(last=do_step)     # bucket reduce-scatters start from the last backward only
        timed = getattr(self, "time_backward", False) and self.device.type == "cuda" \
            and not torch.cuda.is_current_stream_capturing()
        if timed:                                             # eager profiling aid: device time of the backward pass
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        scaled.backward()
        if timed:
            e1.record()
            self._backward_events = (e0, e1)
        if not do_step:
            return
        if self.dp is not None:
            self.dp.reduce_gradients()
        if self.tp_model:
            self.model.sync_replicated_grads()
            if a.max_grad_norm and a.max_grad_norm > 0:
                self.model.clip_grad_norm_(a.max_grad_norm)       # norm over all ranks' shards
        if self.use_external_grad_clip and a.max_grad_norm and a.max_grad_norm > 0:
            torch.nn.utils.clip_grad_norm_([p for p in self.model.parameters() if p.grad is not None], a.max_grad_norm)
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        if self.fp8_context is not None:
            self.fp8_context.invalidate_caches()

    def training_step(self, batch: Any, do_step: bool = True) -> torch.Tensor:
        """One micro-step (forward, backward and — when ``do_step`` — the optimizer update).
        Returns the detached loss tensor on the device (no host synchronisation)."""
        if self.use_cuda_graphs and do_step:
            return self._graphed_step(batch)
        if self.zero3 is not None:
            inp = self._prepare_inputs(batch)
            loss = self.zero3.forward_backward(inp["input_ids"], labels=inp["labels"], position_ids=inp.get("position_ids"),
                                               cu_seqlens=inp.get("cu_seqlens"), max_seqlen=inp.get("max_seqlen"),
                                               seqlens_host=inp.get("seqlens_host"),
                                               shift_labels=bool(self._get("shift_labels", True)))
            self.optimizer.step()
            return loss
        if self._nvtx:
            nvtx = torch.cuda.nvtx
            nvtx.range_push("data")
            inp = self._prepare_inputs(batch)
            nvtx.range_pop()
            nvtx.range_push("forward")
            loss = self._forward_loss(inp)
            nvtx.range_pop()
            nvtx.range_push("backward+optimizer" if do_step else "backward")
            self._backward_and_maybe_step(loss, do_step)
            nvtx.range_pop()
            return loss.detach()
        inp = self._prepare_inputs(batch)
        loss = self._forward_loss(inp)
        self._backward_and_maybe_step(loss, do_step)
        return loss.detach()

    _training_step = training_step

    # -- CUDA graph of the whole step ----------------------------------------------------------------------
    def _graphed_step(self, batch: Any) -> torch.Tensor:
        f = _batch_fields(batch)
        ids = f["input_ids"]
        max_docs = int(self._get("cuda_graph_max_documents", 0) or 0)
        if max_docs > 0 and isinstance(f.get("cu_seqlens"), torch.Tensor):
            # packed batches hold a varying number of documents: pad the boundary list to a fixed length with
            # empty documents (the attention kernels skip them) so that one captured graph serves every batch
            cu = f["cu_seqlens"]
            if cu.numel() - 1 > max_docs:
                raise ValueError(f"batch holds {cu.numel() - 1} documents, cuda_graph_max_documents is {max_docs}")
            f = dict(f)
            f["cu_seqlens"] = torch.cat((cu, cu[-1:].expand(max_docs + 1 - cu.numel())))
            f["max_seqlen"] = int(self.args.max_seq_length)
            f["seqlens_host"] = None
        key = (tuple(ids.shape), tuple(f["cu_seqlens"].shape) if isinstance(f.get("cu_seqlens"), torch.Tensor) else None,
               f.get("max_seqlen"), tuple(f["seqlens_host"]) if f.get("seqlens_host") is not None and
               not isinstance(f.get("cu_seqlens"), torch.Tensor) else None)
        if self._graph is None or self._graph["key"] != key:
            self._capture_graph(f, key)
        g = self._graph
        nb = bool(self.args.non_blocking_transfers)
        for k, dst in g["static"].items():
            src = f.get(k) if k != "labels" or "labels" in f else f["input_ids"]
            dst.copy_(src.reshape(dst.shape), non_blocking=nb)
        if hasattr(self.optimizer, "prepare_step"):
            self.optimizer.prepare_step()
        g["graph"].replay()
        # the update ran inside the graph: tell torch's scheduler bookkeeping that an optimizer step happened
        # (it otherwise warns that lr_scheduler.step() came first)
        self.optimizer._opt_called = True
        return g["loss"]

    def _capture_graph(self, f: Dict[str, Any], key) -> None:
        """Warm up eagerly (allocates optimizer state, rope tables, autotunes nothing), then capture
        forward + backward + optimizer kernels of one micro-step into a CUDA graph."""
        a = self.args
        static: Dict[str, torch.Tensor] = {}
        for k in ("input_ids", "labels", "position_ids", "cu_seqlens"):
            v = f.get(k) if k != "labels" else f.get("labels", f["input_ids"])
            if isinstance(v, torch.Tensor):
                static[k] = v.to(self.device).clone()
        meta = {k: f[k] for k in ("max_seqlen", "seqlens_host") if f.get(k) is not None}
        if hasattr(self.model, "prepare_rope"):
            self.model.prepare_rope(int(meta.get("max_seqlen") or static["input_ids"].shape[-1]), self.device)
        inp = dict(static)
        inp.update(meta)
        if not hasattr(self.optimizer, "launch_step"):
            raise RuntimeError("CUDA-graph capture of the step needs an optimizer with a capturable device half "
                               "(FusedAdamW / LoRAPlusAdamW)")
        # warm-up and capture run on streams of their own, so the gradient-accumulation nodes see another stream
        # than the one the parameters were created on: intended here, torch's notice about it is switched off
        quiet = getattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch", None)
        if quiet is not None:
            quiet(False)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, int(a.cuda_graph_warmup_steps)) if self.state.micro_step == 0 else 1):
                loss = self._forward_loss(inp)
                loss.backward()
                if self.dp is not None:
                    self.dp.reduce_gradients()
                self.optimizer.zero_grad(set_to_none=True)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.optimizer.ensure_state()      # moments must exist before capture, or their zero-fill would be replayed
        from ..ops import _ext
        launched_before = _ext.launches()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode=str(self._get("cuda_graph_capture_mode", "thread_local"))):
            loss = self._forward_loss(inp)
            loss.backward()
            if self.dp is not None:
                self.dp.reduce_gradients()
            self.optimizer.launch_step()
            loss_out = loss.detach()
        self.graph_kernel_launches = _ext.launches() - launched_before     # own kernels per replay
        self._graph = {"graph": graph, "static": static, "loss": loss_out, "key": key}

    # ==================================================================================== train
    def train(self, train_dataset: Optional[Iterable] = None, resume_from_checkpoint: Optional[str] = None
              ) -> TrainerState:
        a = self.args
        if train_dataset is not None:
            self.train_dataloader = self._dataloader_from_dataset(train_dataset)
            self.total_steps = self._estimate_total_steps()
            self._setup_scheduler()
        if self.train_dataloader is None:
            raise ValueError("no training data: pass train_dataloader to the constructor or a dataset to train()")
        start_epoch = 0
        skip_micro = 0
        if resume_from_checkpoint:
            start_epoch = self.resume_from_checkpoint(resume_from_checkpoint)
            skip_micro = int(self.state.micro_in_epoch)       # cursor inside the epoch the checkpoint was taken in
        if self.rank == 0:
            print_chronicals_banner(self.world_size, type(self.model).__name__,
                                    {"params": f"{self.num_params / 1e6:.1f} M", "total steps": self.total_steps,
                                     "optimizations": ", ".join(k for k, v in self._active_optimizations.items() if v)})
        gc_was = gc.isenabled()
        if a.disable_gc_during_training:
            gc.disable()
        if self.watchdog is not None and not self.watchdog.heartbeat.running:
            self.watchdog.start()
        self.model.train()
        if isinstance(self.optimizer, ScheduleFreeAdamW):
            self.optimizer.train_mode()
        t_start = time.perf_counter()
        try:
            for epoch in range(start_epoch, max(1, a.num_train_epochs)):
                self.state.epoch = epoch
                try:
                    avg = self._train_epoch_fast(epoch, skip_micro if epoch == start_epoch else 0)
                except Exception as e:
                    if self.watchdog is not None:                      # let the peers stop launching work
                        self.watchdog.report_failure(e)
                        self.watchdog.stop()
                    raise
                if a.max_steps > 0 and self.state.global_step >= a.max_steps:
                    break
                if self.eval_dataloader is not None:
                    ev = self.evaluate()
                    if self.rank == 0:
                        print(f"[epoch {epoch}] eval loss {ev:.4f}")
                    self.state.best_loss = min(self.state.best_loss, ev)
                if a.save_steps and a.save_steps > 0:
                    self.state.epoch, self.state.micro_in_epoch = epoch + 1, 0     # resume starts the next epoch
                    self.save_checkpoint(f"checkpoint-epoch-{epoch}")
        finally:
            if a.disable_gc_during_training and gc_was:
                gc.enable()
            if self._trace not in (None, False):
                try:
                    self._trace.stop()
                except Exception:
                    pass
                self._trace = None
            if self.watchdog is not None:
                self.watchdog.stop()              # no heartbeat thread outlives the loop it guards
        self.state.total_time += time.perf_counter() - t_start
        if a.save_steps is not None and a.save_steps >= 0 and self._get("save_final", True):
            self.save_checkpoint("final")
        if self.reporter is not None:
            try:
                self.reporter.save_metrics_json()
                self.reporter.generate_html_report()
            except Exception as e:  # reporting must never fail a run
                print(f"[reporter] skipped: {e}")
        if self.rank == 0:
            self._print_final_stats()
        return self.state

    def _dataloader_from_dataset(self, dataset) -> Iterable:
        """Samples (dicts with ``input_ids``) → packed rows → micro-batches."""
        from ..data.data_loader import create_packed_dataloader
        a = self.args
        # tensor-parallel ranks work on the same tokens (sequence parallelism and the vocabulary-parallel loss
        # split one batch); only data-parallel ranks read different slices
        dp_rank, dp_world = (0, 1) if self.tp_model else (self.rank, self.world_size)
        return create_packed_dataloader(dataset, batch_size=a.per_device_train_batch_size,
                                        max_length=a.max_seq_length, strategy=a.packing_strategy,
                                        use_packing=a.use_sequence_packing, seed=a.seed,
                                        rank=dp_rank, world_size=dp_world)

    def _train_epoch_fast(self, epoch: int, skip_micro: int = 0) -> float:
        a = self.args
        accum = max(1, a.gradient_accumulation_steps)
        on_gpu = self.device.type == "cuda"
        tokens_since_log = 0
        real_since_log = 0
        losses_since_log: List[torch.Tensor] = []
        epoch_loss_sum, epoch_loss_n = 0.0, 0
        if on_gpu:
            torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        micro_in_epoch = 0
        self.state.micro_in_epoch = skip_micro
        for batch in self.train_dataloader:
            if a.max_steps > 0 and self.state.global_step >= a.max_steps:
                break
            micro_in_epoch += 1
            if micro_in_epoch <= skip_micro:
                continue
            self.state.micro_in_epoch = micro_in_epoch
            do_step = (micro_in_epoch % accum) == 0
            if self.watchdog is not None:
                try:
                    self.watchdog.check(self.state.global_step)     # before the first launch of the step
                except Exception as e:
                    self._on_peer_failure(e)
                    raise
            if self._trace is None and a.enable_profiling and self.rank == 0:
                self._trace = self._start_trace()
            try:
                if self.profiler is not None:
                    with self.profiler.profile_step():
                        loss = self.training_step(batch, do_step)
                else:
                    loss = self.training_step(batch, do_step)
            except Exception as e:
                if self.watchdog is not None:
                    self.watchdog.report_failure(e)                # peers leave at their next check
                raise
            if self._trace not in (None, False):
                self._trace.step()
            losses_since_log.append(loss)
            f = _batch_fields(batch)
            ntok = int(f["input_ids"].numel())
            tokens_since_log += ntok
            self.state.total_tokens += ntok
            self.state.micro_step += 1
            if not do_step:
                continue
            if self.scheduler is not None:
                self.scheduler.step()
            self.state.global_step += 1
            for cb in self.callbacks:
                cb(self, self.state)
            if a.empty_cache_steps and self.state.global_step % a.empty_cache_steps == 0 and on_gpu:
                torch.cuda.empty_cache()
            if a.logging_steps and self.state.global_step % a.logging_steps == 0:
                if on_gpu:
                    torch.cuda.synchronize(self.device)
                dt = time.perf_counter() - t0
                avg_loss = float(torch.stack([l.float() for l in losses_since_log]).mean().item())
                if self.world_size > 1:
                    t = torch.tensor([avg_loss], device=self.device)
                    self.dist.all_reduce(t)
                    avg_loss = float(t.item()) / self.world_size
                tps = tokens_since_log * self.world_size / dt if dt > 0 else 0.0
                self._log_step_fast(avg_loss, tps)
                epoch_loss_sum += avg_loss
                epoch_loss_n += 1
                losses_since_log, tokens_since_log = [], 0
                if on_gpu:
                    torch.cuda.synchronize(self.device)
                t0 = time.perf_counter()
            if a.eval_steps and self.eval_dataloader is not None and self.state.global_step % a.eval_steps == 0:
                self.evaluate()
                self.model.train()
            if a.save_steps and a.save_steps > 0 and self.state.global_step % a.save_steps == 0:
                self.save_checkpoint(f"checkpoint-{self.state.global_step}")
        if losses_since_log:
            avg_loss = float(torch.stack([l.float() for l in losses_since_log]).mean().item())
            epoch_loss_sum += avg_loss
            epoch_loss_n += 1
            self.state.log_history.append({"step": self.state.global_step, "loss": avg_loss})
        return epoch_loss_sum / max(1, epoch_loss_n)

    _train_epoch = _train_epoch_fast

    def _start_trace(self):
        """torch.profiler schedule from the ``profiling_*`` flags; writes a chrome trace per active window."""
        a = self.args
        try:
            from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler
            os.makedirs(a.profiling_output_dir, exist_ok=True)
            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if self.device.type == "cuda" else [])
            prof = profile(activities=acts,
                           schedule=schedule(wait=a.profiling_wait_steps, warmup=a.profiling_warmup_steps,
                                             active=a.profiling_active_steps, repeat=1),
                           on_trace_ready=tensorboard_trace_handler(a.profiling_output_dir),
                           record_shapes=a.profiling_record_shapes, profile_memory=a.profiling_profile_memory,
                           with_stack=a.profiling_with_stack, with_flops=a.profiling_with_flops)
            prof.start()
            return prof
        except Exception as e:
            print(f"[profiling] torch.profiler trace disabled: {e}")
            return False

    def _on_peer_failure(self, exc: Exception) -> None:
        """A peer stopped answering or reported an error: launch nothing more, keep this rank's state."""
        print(f"[rank {self.rank}] peer failure detected before step {self.state.global_step}: {exc}")
        try:
            out = os.path.join(self.args.output_dir, f"emergency-{self.state.global_step}")
            os.makedirs(out, exist_ok=True)
            st = {k: v for k, v in asdict(self.state).items() if k != "log_history"}
            ckpt_io.save_training_state(out, self.optimizer, self.scheduler if self.rank == 0 else None, st,
                                        self.state.log_history, self.rank, self.world_size)
            if self.rank == 0 and not self.tp_model:
                ckpt_io.save_model(self.model, out, safe=bool(self._get("save_safetensors", True)))
            print(f"[rank {self.rank}] emergency state written to {out}")
        except Exception as e:                                         # best effort
            print(f"[rank {self.rank}] emergency checkpoint failed: {e}")

    def _log_step_fast(self, loss: float, tokens_per_sec: float) -> None:
        a = self.args
        lr = self.optimizer.param_groups[0]["lr"]
        mfu = self.flops_per_token * tokens_per_sec / (a.gpu_peak_tflops * 1e12 * self.world_size) if a.track_mfu else 0.0
        mem = torch.cuda.max_memory_allocated(self.device) / 2**30 if self.device.type == "cuda" else 0.0
        rec = {"step": self.state.global_step, "loss": loss, "lr": lr, "tokens_per_sec": tokens_per_sec,
               "mfu": mfu, "peak_memory_gb": mem, "epoch": self.state.epoch}
        self.state.log_history.append(rec)
        self.state.best_loss = min(self.state.best_loss, loss)
        if self.rank == 0:
            print(f"step {self.state.global_step:>6d} | loss {loss:.4f} | lr {lr:.2e} | "
                  f"{tokens_per_sec:,.0f} tok/s | MFU {100 * mfu:.1f}% | mem {mem:.1f} GB")
            if self._log_file:
                with open(self._log_file, "a") as f:
                    f.write(json.dumps(rec) + "\n")
            if self.reporter is not None:
                self.reporter.log_step(self.state.global_step, loss, lr, tokens_per_sec, mem)

    def _print_final_stats(self) -> None:
        s = self.state
        tps = s.total_tokens * self.world_size / s.total_time if s.total_time > 0 else 0.0
        print(f"training done: {s.global_step} steps, {s.total_tokens * self.world_size:,} tokens, "
              f"{s.total_time:.1f} s, {tps:,.0f} tok/s overall, best loss {s.best_loss:.4f}")

    # ==================================================================================== evaluate
    @torch.no_grad()
    def evaluate(self, eval_dataloader: Optional[Iterable] = None) -> float:
        dl = eval_dataloader or self.eval_dataloader
        if dl is None:
            raise ValueError("no eval dataloader")
        sf = isinstance(self.optimizer, ScheduleFreeAdamW)
        if sf:
            self.optimizer.eval_mode()
        self.model.eval()
        tot, n = torch.zeros((), device=self.device), 0
        for batch in dl:
            inp = self._prepare_inputs(batch)
            if self.zero3 is not None:
                with torch.no_grad():
                    tot += self.zero3.forward_only(inp["input_ids"], labels=inp["labels"],
                                                   position_ids=inp.get("position_ids"), cu_seqlens=inp.get("cu_seqlens"),
                                                   max_seqlen=inp.get("max_seqlen"),
                                                   shift_labels=bool(self._get("shift_labels", True))).loss.float()
            else:
                tot += self._forward_loss(inp).float()
            n += 1
        if self.world_size > 1:
            t = torch.stack((tot, torch.tensor(float(n), device=self.device)))
            self.dist.all_reduce(t)
            tot, n = t[0], int(t[1].item())
        self.model.train()
        if sf:
            self.optimizer.train_mode()
        return float(tot.item()) / max(1, n)

    # ==================================================================================== checkpoints
    def save_checkpoint(self, name: str) -> str:
        a = self.args
        out = os.path.join(a.output_dir, name)
        # a tensor-parallel model re-assembles the full HuggingFace-named tensors with a collective gather
        full_state = self.model.gather_full_state_dict() if self.tp_model else (
            self.zero3.gather_full_state_dict() if self.zero3 is not None else None)
        if self.rank == 0:
            ckpt_io.save_model(self.model, out, safe=bool(self._get("save_safetensors", True)), state=full_state)
            lora_cfg = getattr(self.model, "lora_config", None)
            if lora_cfg is not None:
                ckpt_io.save_lora_adapter(self.model, out, lora_cfg["rank"], lora_cfg["alpha"],
                                          lora_cfg["target_modules"], lora_cfg.get("dropout", 0.0))
            with open(os.path.join(out, "training_config.json"), "w") as f:
                f.write(a.to_json())
        st = {k: v for k, v in asdict(self.state).items() if k != "log_history"}
        ckpt_io.save_training_state(out, self.optimizer, self.scheduler if self.rank == 0 else None, st,
                                    self.state.log_history, self.rank, self.world_size)
        if self.rank == 0:
            if self.reporter is not None:
                self.reporter.log_checkpoint(self.state.global_step, out)
            if name.startswith("checkpoint-") and name[len("checkpoint-"):].isdigit():
                ckpt_io.prune_checkpoints(a.output_dir, a.save_total_limit)
        if self.dist is not None:
            self.dist.barrier()
        return out

    def load_checkpoint(self, checkpoint_dir: str, load_optimizer: bool = True) -> Dict[str, Any]:
        if self.zero3 is not None:
            # parameter storage is released between uses; the engine scatters the full tensors into its shards
            self.zero3.load_full_state_dict(ckpt_io.read_weights(checkpoint_dir))
        else:
            ckpt_io.load_model_weights(self.model, checkpoint_dir, strict=False)
        if os.path.exists(os.path.join(checkpoint_dir, "adapter_model.safetensors")):
            ckpt_io.load_lora_adapter(self.model, checkpoint_dir)
        st = ckpt_io.load_training_state(checkpoint_dir, self.optimizer if load_optimizer else None,
                                         self.scheduler if load_optimizer else None, self.rank, self.world_size)
        for k, v in st.items():
            if hasattr(self.state, k) and k != "log_history":
                setattr(self.state, k, v)
        hist = os.path.join(checkpoint_dir, "training_history.json")
        if os.path.exists(hist):
            with open(hist) as f:
                self.state.log_history = json.load(f)
        self._graph = None
        return st

    def resume_from_checkpoint(self, checkpoint_dir: str) -> int:
        self.load_checkpoint(checkpoint_dir)
        return int(self.state.epoch)

    def push_to_hub(self, repo_id: str, token: Optional[str] = None) -> None:
        """Upload ``<output_dir>/final``; needs ``huggingface_hub`` and network access."""
        try:
            from huggingface_hub import HfApi
        except Exception as e:
            raise RuntimeError("push_to_hub requires the huggingface_hub package") from e
        from ..config.config import HF_WRITE_TOKEN
        HfApi(token=token or HF_WRITE_TOKEN or None).upload_folder(
            folder_path=os.path.join(self.args.output_dir, "final"), repo_id=repo_id)

    # ==================================================================================== diagnostics
    def get_active_optimizations(self) -> Dict[str, bool]:
        return dict(self._active_optimizations)

    def print_optimization_summary(self) -> None:
        print("active optimizations:")
        for k, v in self._active_optimizations.items():
            print(f"  [{'x' if v else ' '}] {k}")

    def get_performance_diagnostic(self) -> Dict[str, Any]:
        hist = [h for h in self.state.log_history if "tokens_per_sec" in h]
        tps = sum(h["tokens_per_sec"] for h in hist) / len(hist) if hist else 0.0
        a = self.args
        d = {"avg_tokens_per_sec": tps,
             "mfu": self.flops_per_token * tps / (a.gpu_peak_tflops * 1e12 * self.world_size),
             "num_params": self.num_params, "world_size": self.world_size,
             "active_optimizations": self.get_active_optimizations(),
             "recommendations": self._get_recommendations()}
        return d

    def _get_recommendations(self) -> List[str]:
        a, rec = self.args, []
        if self.device.type == "cuda" and not self.use_cuda_graphs and a.gradient_accumulation_steps == 1:
            rec.append("enable use_cuda_graphs: the step is launch-bound for small models")
        if a.use_gradient_checkpointing and self.num_params < 3e9:
            rec.append("disable use_gradient_checkpointing: activations of models under 3B fit in 180 GB")
        if not a.use_sequence_packing:
            rec.append("enable use_sequence_packing to avoid compute on padding")
        return rec
