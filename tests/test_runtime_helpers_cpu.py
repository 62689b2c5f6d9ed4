"""Behaviour of the memory / runtime / observability helpers (what they do, not just that they exist)."""
import json
import os

import pytest
import torch
import torch.nn as nn

from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
from chronicals_b200.training.async_activation_offload import (ActivationOffloadManager, CheckpointWithOffload, OffloadActivations,
                                                               OffloadConfig, PinnedMemoryPool, create_offload_manager)
from chronicals_b200.training.cuda_graph_manager import CUDAGraphConfig, CUDAGraphManager, bucket_length
from chronicals_b200.training.gradient_checkpointing import GradientCheckpointer
from chronicals_b200.utils.compile_utils import CompiledLoRAModel, LoRAHotswapManager
from chronicals_b200.utils.profiling_utils import MFUTracker, PerformanceProfiler, ThroughputMonitor
from chronicals_b200.utils.visual_reporter import VisualReporter


def _tiny(layers=2):
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers, cfg.vocab_size, cfg.dtype = layers, 512, "float32"
    return cfg


def _grads(model, ids):
    model.zero_grad(set_to_none=True)
    model(ids, labels=ids).loss.backward()
    return [p.grad.clone() for p in model.parameters()]


def test_checkpointing_with_offload_gives_the_same_gradients():
    """Recomputing layers, with their saved inputs routed through the offload manager's pack / unpack hooks,
    changes no gradient (on CPU the hooks pass tensors through; the GPU suite checks the host round trip)."""
    cfg = _tiny(3)
    model = build_model(cfg, dtype=torch.float32, seed=0).train()
    ids = torch.randint(0, cfg.vocab_size, (2, 40), generator=torch.Generator().manual_seed(1))
    want = _grads(model, ids)
    model.gradient_checkpointing_enable(ratio=1.0, offload=True)
    assert isinstance(model.activation_offload, ActivationOffloadManager)
    assert all(l._use_checkpoint and l._offload is model.activation_offload for l in model.model.layers)
    got = _grads(model, ids)
    assert max((a - b).abs().max().item() for a, b in zip(got, want)) < 1e-6
    stats = model.activation_offload.get_stats()
    assert stats["tensors_kept"] > 0 and stats["tensors_offloaded"] == 0          # CPU tensors are never moved
    model.gradient_checkpointing_disable()
    assert all(l._offload is None and not l._use_checkpoint for l in model.model.layers)


def test_trainer_passes_activation_offloading_to_the_model(tmp_path):
    cfg = _tiny(2)
    a = TrainingConfig(output_dir=str(tmp_path), gradient_accumulation_steps=1, logging_steps=1, save_steps=0, bf16=False,
                       fp8=False, use_gradient_checkpointing=True, use_activation_offloading=True, visual_reporting=False)
    a.save_final = a.log_jsonl = False
    tr = ChronicalsTrainer(build_model(cfg, dtype=torch.float32, seed=0), a, None)
    assert tr.get_active_optimizations()["activation_offloading"]
    assert tr.model.activation_offload is not None
    ids = torch.randint(0, cfg.vocab_size, (2, 32))
    assert torch.isfinite(tr.training_step({"input_ids": ids, "labels": ids}))


def test_offload_context_and_checkpoint_wrapper_match_plain_autograd():
    lin = nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 16))
    x = torch.randn(4, 16, requires_grad=True)
    lin(x).pow(2).sum().backward()
    want = [p.grad.clone() for p in lin.parameters()] + [x.grad.clone()]
    for wrapper in ("context", "checkpoint", "factory"):
        for p in lin.parameters():
            p.grad = None
        x.grad = None
        if wrapper == "context":
            with OffloadActivations(OffloadConfig(min_tensor_numel=1)) as mgr:
                y = lin(x)
            assert isinstance(mgr, ActivationOffloadManager)
        elif wrapper == "checkpoint":
            y = CheckpointWithOffload(OffloadConfig())(lin, x)
        else:
            y = create_offload_manager(num_layers=2, min_tensor_numel=1)(lin, x)
        y.pow(2).sum().backward()
        got = [p.grad for p in lin.parameters()] + [x.grad]
        assert all(torch.allclose(a, b, atol=1e-6) for a, b in zip(got, want)), wrapper


def test_pinned_pool_reuses_buffers():
    pool = PinnedMemoryPool(max_bytes=1 << 20, pin=False)
    like = torch.empty(100)
    a = pool.get(like)
    pool.put(a)
    b = pool.get(like)
    assert a.data_ptr() == b.data_ptr()
    c = pool.get(like)
    assert c.data_ptr() != b.data_ptr()


def test_gradient_checkpointer_selects_and_reports():
    gc_ = GradientCheckpointer(num_layers=24, checkpoint_ratio=0.25)
    chosen = [i for i in range(24) if gc_.should_checkpoint(i)]
    assert len(chosen) == 6 and chosen == sorted(chosen)
    lin = nn.Linear(8, 8)
    x = torch.randn(2, 8, requires_grad=True)
    y = gc_.checkpoint(lambda t: lin(t).relu(), x, layer_idx=chosen[0])
    z = gc_.checkpoint(lambda t: lin(t).relu(), x, layer_idx=next(i for i in range(24) if i not in chosen))
    assert torch.allclose(y, z)
    s = gc_.memory_savings(2**30)
    assert abs(s["saved_fraction"] - 0.25) < 1e-9


def test_throughput_monitor_flags_a_regression_and_mfu_tracker_uses_6n():
    mon = ThroughputMonitor(window=4, threshold_pct=10.0)
    flags = [mon.update(100_000.0, i) for i in range(8)]
    assert not any(flags)
    drops = [mon.update(80_000.0, 8 + i) for i in range(4)]
    assert drops[-1] and mon.regressions and mon.regressions[-1]["best"] == pytest.approx(100_000.0)
    assert mon.regressions[-1]["mean"] < 0.9 * mon.regressions[-1]["best"]
    mfu = MFUTracker(num_params=494_000_000, peak_tflops=2250.0, num_gpus=8)
    assert mfu.compute(1_500_000.0) == pytest.approx(6 * 494e6 * 1.5e6 / (2250e12 * 8))
    assert mfu.average() == pytest.approx(mfu.history[0])


def test_profiler_records_steps_phases_and_writes_a_report(tmp_path):
    prof = PerformanceProfiler(enabled=True, num_params=1000, peak_tflops=1.0, use_nvtx=False)
    for _ in range(3):
        with prof.profile_step(tokens=512):
            with prof.profile_phase("forward"):
                torch.randn(64, 64) @ torch.randn(64, 64)
            with prof.profile_phase("backward"):
                torch.randn(64, 64) @ torch.randn(64, 64)
    s = prof.summary()
    assert s["steps"] == 3 and s["mean_tokens_per_sec"] > 0
    r = prof.records[0]
    assert r.timing.forward_ms > 0 and r.timing.backward_ms > 0 and r.tokens == 512
    path = prof.save_report(str(tmp_path / "perf" / "report.json"))
    data = json.load(open(path))
    assert data["summary"]["steps"] == 3 and len(data["records"]) == 3


def test_visual_reporter_writes_metrics_checkpoints_and_html(tmp_path):
    rep = VisualReporter(str(tmp_path), "unit")
    for i in range(5):
        rep.log_step(i + 1, 3.0 - 0.1 * i, 1e-4, 1000.0 + i, 1.5)
    ck = rep.log_checkpoint(5, "/somewhere/checkpoint-5", {"note": "x"})
    assert json.load(open(ck))["loss"] == pytest.approx(2.6)
    m = json.load(open(rep.save_metrics_json()))
    assert m["steps"] == [1, 2, 3, 4, 5] and len(m["losses"]) == 5 and m["checkpoints"][0]["note"] == "x"
    html = open(rep.generate_html_report()).read()
    assert "<svg" in html and "checkpoint-5" in html and "2.6000" in html


def test_graph_manager_runs_eagerly_without_cuda_and_buckets_lengths():
    mgr = CUDAGraphManager(CUDAGraphConfig(warmup_steps=1))
    calls = []

    def fn(x):
        calls.append(1)
        return x * 2
    x = torch.ones(4)
    for _ in range(3):
        assert torch.equal(mgr.replay_or_run("double", fn, x), x * 2)
    st = mgr.get_statistics()
    assert st["eager_runs"] == 3 and st["replays"] == 0 and len(calls) == 3
    assert bucket_length(300, [128, 256, 512, 1024]) == 512 and bucket_length(5000, [128, 256]) >= 5000


def test_lora_hotswap_replaces_adapter_weights_in_place_and_checks_shapes():
    from chronicals_b200.lora import LoRAConfig, apply_lora
    cfg = _tiny(1)
    model = build_model(cfg, dtype=torch.float32, seed=0)
    apply_lora(model, LoRAConfig(rank=4, alpha=8.0, target_modules=["q_proj", "v_proj"]))
    mgr = LoRAHotswapManager(model)
    targets = mgr._targets()
    assert targets, "model carries no adapter tensors"
    ptrs = {k: v.data_ptr() for k, v in targets.items()}
    adapter = {("base_model.model." + k): torch.full_like(v, 0.25) for k, v in targets.items()}
    assert mgr.register("quarter", adapter) == len(targets)
    assert mgr.swap("quarter") == len(targets) and mgr.active == "quarter"
    after = mgr._targets()
    assert all(v.data_ptr() == ptrs[k] for k, v in after.items())            # same storage: a captured graph stays valid
    assert all(torch.all(v == 0.25) for v in after.values())
    bad = {k: torch.zeros(3, 3) for k in targets}
    mgr.register("bad", bad)
    with pytest.raises(ValueError):
        mgr.swap("bad")
    wrapped = CompiledLoRAModel(model)
    wrapped.load_adapter("half", {k: torch.full_like(v, 0.5) for k, v in targets.items()})
    assert all(torch.all(v == 0.5) for v in wrapped.hotswap._targets().values())
