"""Headline benchmark: tokens/s of a Qwen2.5-0.5B-architecture full fine-tune step.

    python bench.py --gpus N --steps K --warmup W            (this framework)
    python bench.py --impl reference --gpus N ...            (the unmodified reference)

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ...``
(RANK / LOCAL_RANK / WORLD_SIZE are read from the environment).  Random-init
weights of the named architecture, seeded synthetic token ids, micro-batch
8 x 1024 per GPU (weak scaling), bf16, AdamW.  Rank 0 prints one JSON line.

Two timed regions, both CUDA events with a barrier + synchronize on either side
and the maximum over ranks:

* ``value``  - K optimizer steps replaying device-resident batches;
* ``e2e``    - K steps through ``ChronicalsTrainer.train()`` where every step copies
               its batch from pinned host memory and reads the loss back.

The working set of a step (weights, activations, optimizer state: several GB) is
far larger than the 126 MB L2, so no explicit flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PUBLISHED_TOK_S = 41184.0          # reference README: full fine-tune, 1x A100-40GB
MODEL = "qwen2.5-0.5b"
MICRO_BATCH, SEQ_LEN = 8, 1024
N_PARAMS_05B = 494_032_768


# ------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def _dist_setup():
    import torch
    sys.path.insert(0, ROOT)
    from chronicals_b200.parallel.bootstrap import init_distributed
    rank, local_rank, world = init_distributed(timeout_s=180.0)     # a wedged collective ends the run quickly
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    return rank, local_rank, world


def _barrier_sync(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def _max_ms(ms, world):
    from chronicals_b200.parallel.bootstrap import max_over_ranks
    return max_over_ranks(ms) if world > 1 else ms


class TimedLoader:
    """Yields ``warmup + steps`` host batches; records CUDA events when batch ``warmup`` is
    requested and when the iterator is exhausted, each after a barrier + synchronize."""

    def __init__(self, batches, warmup, steps, world):
        import torch
        self.batches, self.warmup, self.steps, self.world = batches, warmup, steps, world
        self.start = torch.cuda.Event(enable_timing=True) if torch.cuda.is_available() else None
        self.end = torch.cuda.Event(enable_timing=True) if torch.cuda.is_available() else None
        self.t0 = self.t1 = 0.0
        self.on_start = None
        self.on_end = None

    def __len__(self):
        return self.warmup + self.steps

    def __iter__(self):
        n = len(self.batches)
        for i in range(self.warmup + self.steps):
            if i == self.warmup:
                _barrier_sync(self.world)
                if self.on_start:
                    self.on_start()
                self.t0 = time.perf_counter()
                if self.start is not None:
                    self.start.record()
            yield self.batches[i % n]
        if self.end is not None:
            self.end.record()
        _barrier_sync(self.world)
        self.t1 = time.perf_counter()
        if self.on_end:
            self.on_end()

    def elapsed_ms(self):
        if self.start is not None:
            return self.start.elapsed_time(self.end)
        return (self.t1 - self.t0) * 1e3


def _host_batches(n, vocab, seed, pin):
    import torch
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, vocab, (MICRO_BATCH, SEQ_LEN), generator=g, dtype=torch.long)
        b = {"input_ids": ids, "labels": ids.clone()}
        if pin:
            b = {k: v.pin_memory() for k, v in b.items()}
        out.append(b)
    return out


# ------------------------------------------------------------------------------------------- this framework
def run_ours(args):
    import torch
    rank, local_rank, world = _dist_setup()
    from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
    from chronicals_b200 import ops as _ops
    from chronicals_b200.ops import _ext

    dev = torch.device("cuda", local_rank)
    cfg = ChronicalsConfig.from_model_name(args.model)
    model = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=1234)
    n_params = sum(p.numel() for p in model.parameters())
    targs = TrainingConfig(
        output_dir=os.path.join("/tmp", f"cb_bench_{os.getpid()}"), num_train_epochs=1,
        per_device_train_batch_size=MICRO_BATCH, max_seq_length=SEQ_LEN, gradient_accumulation_steps=1,
        learning_rate=2e-5, weight_decay=0.01, max_grad_norm=1.0, lr_scheduler_type="constant", warmup_ratio=0.0,
        bf16=True, fp8=False, use_gradient_checkpointing=False, use_sequence_packing=False, z_loss_weight=0.0,
        logging_steps=1, save_steps=0, visual_reporting=False, use_cuda_graphs=not args.no_graph, seed=1234,
        gpu_peak_tflops=2250.0)
    targs.save_final = False
    targs.log_jsonl = False
    targs.parallel.dp = world
    comm = args.comm
    if comm == "auto":
        # the fused peer-memory path (reduce-scatter + AdamW + all-gather kernels) when every local GPU
        # can address every other one; NCCL all-reduce otherwise
        comm = "nccl"
        if world > 1:
            from chronicals_b200.parallel.symm import peer_access_available
            comm = "fused" if peer_access_available() else "nccl"
    targs.parallel.comm_backend = comm
    targs.parallel.overlap_grad_reduce = bool(args.overlap) and not args.no_overlap
    if args.reduce_grid > 0:
        targs.parallel.reduce_grid = args.reduce_grid
    pin = True
    batches = _host_batches(4, cfg.vocab_size, 1000 + rank, pin)

    # ---- device-resident region (kernel-only number)
    trainer = ChronicalsTrainer(model, targs, train_dataloader=None)
    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in batches]
    for i in range(args.warmup):
        trainer.training_step(dev_batches[i % len(dev_batches)])
    _barrier_sync(world)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = _ext.launches()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(args.steps):
        loss = trainer.training_step(dev_batches[i % len(dev_batches)])
    b.record()
    _barrier_sync(world)
    clocks = sampler.stop() if rank == 0 else None
    ms = _max_ms(a.elapsed_time(b), world)
    launches_eager = _ext.launches() - l0
    per_step_launches = trainer.graph_kernel_launches if trainer.use_cuda_graphs else launches_eager // max(1, args.steps)
    final_loss = float(loss.item())
    _ext.check_status(dev)

    # ---- end-to-end region through the public trainer API
    loader = TimedLoader(batches, args.warmup, args.steps, world)
    trainer.train_dataloader = loader
    trainer.args.max_steps = -1
    import contextlib
    import io
    sink = io.StringIO()
    with contextlib.redirect_stdout(sink if rank == 0 else sys.stdout):
        trainer.train()
    e2e_ms = _max_ms(loader.elapsed_ms(), world)
    _ext.check_status(dev)

    dp_profile = None
    graph_used = bool(trainer.use_cuda_graphs)            # as the timed steps ran
    if args.dp_profile:
        trainer.use_cuda_graphs = False                   # events cannot be read back from inside a replayed graph
        sharded = hasattr(trainer.optimizer, "profile_report")
        trainer.time_backward = True
        if sharded:
            trainer.optimizer.profile = True
        for i in range(3):
            trainer.training_step(dev_batches[i % len(dev_batches)])
        torch.cuda.synchronize()
        dp_profile = trainer.optimizer.profile_report() if sharded else {}
        e0, e1 = trainer._backward_events
        dp_profile["backward_ms_eager"] = round(e0.elapsed_time(e1), 4)     # comparable between N = 1 and N > 1
        trainer.time_backward = False
        if sharded:
            trainer.optimizer.profile = False
        _barrier_sync(world)
    tokens_per_step = MICRO_BATCH * SEQ_LEN * world
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e = tokens_per_step * args.steps / (e2e_ms / 1e3)
    if rank == 0:
        out = {
            "metric": "tokens/s (box total, device-timed, max over ranks), Qwen2.5-0.5B-arch full fine-tune",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "bf16",
            "data": "synthetic seeded uniform token ids, random-init weights",
            "impl": "chronicals_b200",
            "config": {"model": "Qwen2.5-0.5B architecture (24L, H896, 14q/2kv, d64, I4864, V151936, tied)",
                       "global_batch": MICRO_BATCH * world, "micro_batch_per_gpu": MICRO_BATCH, "seq_len": SEQ_LEN,
                       "parallelism": f"dp{world}", "optimizer": "AdamW (fp32 moments) + global-norm clip",
                       "loss": ("fused linear cross-entropy (bf16 logits resident between forward and backward, "
                                f"{MICRO_BATCH * SEQ_LEN * cfg.vocab_size * 2 / 2**30:.1f} GB)"
                                if MICRO_BATCH * SEQ_LEN * cfg.vocab_size * 2 <= _ops.CCE_RESIDENT_BYTES
                                else "fused linear cross-entropy (no logits)"), "cuda_graph": graph_used,
                       "comm": comm if world > 1 else "none",
                       "grad_reduce": ("per-bucket reduce-scatter from backward hooks on a side stream"
                                       if (world > 1 and comm == "fused" and args.overlap and not args.no_overlap) else
                                       "bucket reduce-scatter kernels after the backward pass, one barrier" if world > 1 else "none"),
                       "l2": "per-step working set is several GB (>> 126 MB L2); no explicit flush"},
            "mfu_6N_vs_2250TF": 6.0 * n_params * value / (2250e12 * world),
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": int(sum(v.numel() * v.element_size() for v in batches[0].values())),
                    "d2h_bytes_per_step": 4, "api": "ChronicalsTrainer.train()"},
            "gpu_launches": int(per_step_launches * args.steps),
            "final_loss": final_loss, "n_params": n_params,
        }
        if hasattr(trainer.optimizer, "buckets"):
            out["config"]["grad_buckets"] = len(trainer.optimizer.buckets)
            out["config"]["reduce_grid"] = int(trainer.optimizer.rs_grid)
            if dp_profile is not None:
                out["dp_profile"] = dp_profile
        print(json.dumps(out), flush=True)
    import shutil
    shutil.rmtree(targs.output_dir, ignore_errors=True)
    from chronicals_b200.parallel.bootstrap import shutdown
    shutdown()


# ------------------------------------------------------------------------------------------- the reference
def _clean_tmp_dirs():
    """Removes benchmark output directories of processes that no longer exist (each arm of a back-to-back
    series writes several GB of checkpoints; nothing else deletes them)."""
    import glob
    import shutil
    for d in glob.glob("/tmp/ref_bench_*") + glob.glob("/tmp/cb_bench_*"):
        try:
            pid = int(d.rsplit("_", 1)[1])
        except ValueError:
            continue
        if not os.path.exists(f"/proc/{pid}"):
            shutil.rmtree(d, ignore_errors=True)


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    sys.exit(0)


def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "chronicals")):
        _unavailable("baseline/_ref is missing (reference not installed)")
    try:
        import torch
        if not torch.cuda.is_available() and not args.tiny:
            _unavailable("no CUDA device")
        rank, local_rank, world = _dist_setup()
        sys.path.insert(0, ref_dir)
        import chronicals as ref_pkg                                      # the unmodified reference
        from chronicals.config.config import TrainingConfig as RefTrainingConfig
        from chronicals.training.chronicals_trainer import ChronicalsTrainer as RefTrainer
        from transformers import AutoModelForCausalLM, Qwen2Config
    except SystemExit:
        raise
    except Exception as e:
        _unavailable(f"reference import failed: {type(e).__name__}: {e}"[:300])

    try:
        dev = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
        if args.tiny:
            hf_cfg = Qwen2Config(vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=4096,
                                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
        else:
            hf_cfg = Qwen2Config(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                                 num_attention_heads=14, num_key_value_heads=2, max_position_embeddings=32768,
                                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
        hf_cfg._attn_implementation = "sdpa"
        torch.manual_seed(1234)
        model = AutoModelForCausalLM.from_config(hf_cfg, torch_dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                                                 attn_implementation="sdpa")
        n_params = sum(p.numel() for p in model.parameters())
        model = model.to(dev)
        if world > 1:
            # the reference ships no multi-GPU support: its trainer is given a DistributedDataParallel model
            # The wrapper forwards attribute look-ups to the wrapped model, so the reference's trainer finds
            # `lm_head`, `config`, `model.layers` … exactly as on one GPU and takes the same code path at every N
            # (with a plain DDP wrapper its `hasattr(model, "lm_head")` test fails and it silently falls back to
            # a different loss path).
            from torch.nn.parallel import DistributedDataParallel as DDP

            class TransparentDDP(DDP):
                def __getattr__(self, name):
                    try:
                        return super().__getattr__(name)
                    except AttributeError:
                        return getattr(super().__getattr__("module"), name)

            model = TransparentDDP(model, device_ids=[local_rank])
        # flag values of the reference's own benchmark recipe (benchmarks/run_benchmark.py:1027-1077),
        # with one optimizer step per 8 x 1024 micro-batch as the benchmark configuration names
        cfg = RefTrainingConfig()
        cfg.use_torch_compile = dev.type == "cuda" and not args.ref_no_compile
        cfg.torch_compile_mode = "default"
        cfg.torch_compile_fullgraph = False
        cfg.torch_compile_regional = True
        cfg.torch_compile_optimizer = True
        cfg.torch_compile_warmup_steps = 0
        cfg.use_fused_adamw = True
        cfg.use_fused_cross_entropy = False
        cfg.use_fused_rope = cfg.use_fused_swiglu = cfg.use_fused_rmsnorm = True
        cfg.use_liger_kernel = dev.type == "cuda"
        cfg.use_fused_linear_cross_entropy = True
        cfg.fp8 = False
        cfg.use_gradient_checkpointing = False
        cfg.optimizer_type = "fused_adamw"
        cfg.non_blocking_transfers = True
        cfg.disable_gc_during_training = True
        cfg.gradient_accumulation_steps = 1
        cfg.use_sequence_packing = False
        cfg.use_flash_varlen = False
        cfg.max_steps = -1
        cfg.num_train_epochs = 1
        cfg.per_device_train_batch_size = MICRO_BATCH
        cfg.max_seq_length = SEQ_LEN
        cfg.logging_steps = 1
        cfg.save_steps = 0
        cfg.output_dir = os.path.join(args.ref_output_root, f"ref_bench_{os.getpid()}")
        cfg.visual_reporting = False
        cfg.bf16 = True
        cfg.learning_rate = 2e-5
        batches = _host_batches(4, hf_cfg.vocab_size, 1000 + rank, dev.type == "cuda")
        if args.tiny:
            batches = [{k: v[:2, :128] % 32000 for k, v in b.items()} for b in batches]
        loader = TimedLoader(batches, args.warmup, args.steps, world)
        sampler = ClockSampler(local_rank)
        if rank == 0 and dev.type == "cuda":
            loader.on_start = sampler.start
        if args.ref_fail_after_timing:
            def _injected():
                raise RuntimeError("injected failure after the timed region")
            loader.on_end = _injected
        import contextlib
        import io
        sink = io.StringIO()
        post_timing_error = None
        _clean_tmp_dirs()                                   # checkpoints left by earlier arms on this box
        trainer = None
        try:
            with contextlib.redirect_stdout(sink):
                trainer = RefTrainer(model, cfg, loader)
                trainer.train()
        except Exception as e:
            # The reference's train() writes two full checkpoints per rank (model + fp32 moments) after the
            # last batch.  When that write fails (a full disk), the timed region has already been closed by the
            # loader, so the measurement stands and the failure is reported beside it.
            if loader.t1 <= 0.0:
                raise
            post_timing_error = f"{type(e).__name__}: {e}"[:300]
        finally:
            import shutil
            shutil.rmtree(cfg.output_dir, ignore_errors=True)
        ms = _max_ms(loader.elapsed_ms(), world)
        clocks = sampler.stop() if (rank == 0 and dev.type == "cuda") else None
        hist = getattr(trainer.state, "log_history", []) if trainer is not None else []
    except SystemExit:
        raise
    except Exception as e:
        import traceback
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"reference run failed: {type(e).__name__}: {e}"[:300])

    toks = batches[0]["input_ids"].numel() * world
    value = toks * args.steps / (ms / 1e3)
    if rank == 0:
        out = {
            "metric": "tokens/s (box total, device-timed, max over ranks), Qwen2.5-0.5B-arch full fine-tune",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "bf16",
            "data": "synthetic seeded uniform token ids, random-init weights", "impl": "reference",
            "config": {"model": "Qwen2.5-0.5B architecture via transformers Qwen2Config (random init)",
                       "global_batch": MICRO_BATCH * world, "seq_len": SEQ_LEN,
                       "parallelism": f"dp{world}" + (" (PyTorch DDP wrapped around the model)" if world > 1 else ""),
                       "stack": "reference ChronicalsTrainer.train(): Liger patches + torch.compile + its FusedAdamW",
                       "reference_version": getattr(ref_pkg, "__version__", "?")},
            "clocks": clocks,
            "e2e": {"value": value, "unit": "tokens/s", "note": "the reference's loop copies each batch from pinned "
                    "host memory and reads loss.item() every step, so its only number is end to end",
                    "h2d_bytes_per_step": int(sum(v.numel() * v.element_size() for v in batches[0].values())),
                    "d2h_bytes_per_step": 4},
            "n_params": n_params, "final_loss": (hist[-1].get("loss") if hist and isinstance(hist[-1], dict) else None),
        }
        if post_timing_error:
            out["post_timing_error"] = post_timing_error
        print(json.dumps(out), flush=True)
    from chronicals_b200.parallel.bootstrap import shutdown
    shutdown()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--overlap", action="store_true",
                    help="reduce-scatter every gradient bucket from a backward hook on a side stream (measured slower "
                         "than the default, which reduces all buckets after the backward pass)")
    ap.add_argument("--no-overlap", action="store_true", help="the default; kept for old command lines")
    ap.add_argument("--reduce-grid", type=int, default=0, help="blocks per bucket reduce-scatter kernel (0: default)")
    ap.add_argument("--dp-profile", action="store_true",
                    help="after the timed regions, run three eager steps with CUDA events around every gradient bucket's "
                         "reduce-scatter and add their hidden / exposed times to the JSON line (diagnostic)")
    ap.add_argument("--tiny", action="store_true", help="plumbing check of the reference arm on a tiny model")
    ap.add_argument("--ref-no-compile", action="store_true")
    ap.add_argument("--ref-fail-after-timing", action="store_true",
                    help="harness self-test: raise inside the reference's loop right after the timed region closed")
    ap.add_argument("--ref-output-root", default="/tmp",
                    help="where the reference trainer writes its (mandatory) checkpoints; removed afterwards")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torch.distributed.run
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29511"),
               os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args)
    else:
        import torch
        if not torch.cuda.is_available():
            # the flagship step only exists as sm_100a kernels: no CPU stand-in is timed
            print(json.dumps({"impl": "chronicals_b200", "unavailable": "no CUDA device"}), flush=True)
            sys.exit(1)
        run_ours(args)


if __name__ == "__main__":
    main()
