"""End-to-end plumbing on CPU: tiny Qwen2-architecture model, 10 AdamW steps, checkpoints, DP over gloo."""
import json
import os
import subprocess
import sys

import pytest
import torch

from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model
from chronicals_b200.checkpoint import io as ckpt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tiny_cfg(layers=2):
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers = layers
    cfg.vocab_size = 2048
    cfg.dtype = "float32"
    return cfg


def _batches(n, vocab, bs=2, seq=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, vocab, (bs, seq + 1), generator=g)
        out.append({"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()})
    return out


def _args(tmp, **kw):
    a = TrainingConfig(output_dir=str(tmp), num_train_epochs=1, gradient_accumulation_steps=1, learning_rate=1e-3,
                       lr_scheduler_type="constant", warmup_ratio=0.0, logging_steps=1, save_steps=0, bf16=False,
                       fp8=False, use_gradient_checkpointing=False, visual_reporting=False, z_loss_weight=0.0)
    a.shift_labels = False
    a.save_final = False
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_config_a_ten_steps_loss_decreases_on_fixed_batch(tmp_path):
    cfg = _tiny_cfg()
    model = build_model(cfg, dtype=torch.float32, seed=0)
    batch = _batches(1, cfg.vocab_size)[0]
    tr = ChronicalsTrainer(model, _args(tmp_path), [batch] * 10)
    st = tr.train()
    losses = [h["loss"] for h in st.log_history if "lr" in h]
    assert len(losses) == 10 and st.global_step == 10
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0] - 0.3
    assert abs(losses[0] - torch.log(torch.tensor(float(cfg.vocab_size))).item()) < 0.5


def test_determinism_same_seed_same_losses(tmp_path):
    cfg = _tiny_cfg()
    runs = []
    for _ in range(2):
        model = build_model(cfg, dtype=torch.float32, seed=0)
        tr = ChronicalsTrainer(model, _args(tmp_path), _batches(4, cfg.vocab_size))
        runs.append([h["loss"] for h in tr.train().log_history if "lr" in h])
    assert runs[0] == runs[1]


def test_grad_accumulation_equals_big_batch(tmp_path):
    cfg = _tiny_cfg()
    b = _batches(2, cfg.vocab_size, bs=2)
    big = {k: torch.cat((b[0][k], b[1][k])) for k in b[0]}
    m1 = build_model(cfg, dtype=torch.float32, seed=0)
    ChronicalsTrainer(m1, _args(tmp_path, gradient_accumulation_steps=2), b).train()
    m2 = build_model(cfg, dtype=torch.float32, seed=0)
    ChronicalsTrainer(m2, _args(tmp_path), [big]).train()
    # Adam's first update is lr * g / (|g| + eps): entries with |g| ~ eps may differ, all others agree
    for p, q in zip(m1.parameters(), m2.parameters()):
        d = (p - q).abs()
        assert d.mean().item() < 1e-5 and d.max().item() <= 2.1e-3


def test_gradient_checkpointing_same_gradients():
    cfg = _tiny_cfg()
    batch = _batches(1, cfg.vocab_size)[0]
    grads = []
    for ck in (False, True):
        m = build_model(cfg, dtype=torch.float32, seed=0)
        if ck:
            m.gradient_checkpointing_enable()
        m.train()
        m(batch["input_ids"], labels=batch["labels"], shift_labels=False).loss.backward()
        grads.append([p.grad.clone() for p in m.parameters()])
    for a, b in zip(*grads):
        assert torch.allclose(a, b, atol=1e-6)


def test_packed_batch_equals_separate_documents():
    """Two documents packed into one row give the same loss as the documents run on their own."""
    cfg = _tiny_cfg()
    m = build_model(cfg, dtype=torch.float32, seed=0).eval()
    g = torch.Generator().manual_seed(1)
    d1, d2 = torch.randint(0, cfg.vocab_size, (20,), generator=g), torch.randint(0, cfg.vocab_size, (13,), generator=g)
    from chronicals_b200.data.sequence_packer import FixedShapeSequencePacker
    pb = FixedShapeSequencePacker(48).pack_all_sequences([d1.tolist(), d2.tolist()])[0]
    f = pb.to_dict()
    packed = m(f["input_ids"], position_ids=f["position_ids"], labels=f["labels"], cu_seqlens=f["cu_seqlens"],
               max_seqlen=f["max_seqlen"]).loss
    order = [d1, d2] if pb.input_ids[0, 0] == d1[0] else [d2, d1]
    tot, n = 0.0, 0
    for d in order:
        l = m(d[None], labels=d[None]).loss
        tot += l.item() * (len(d) - 1)
        n += len(d) - 1
    assert abs(packed.item() - tot / n) < 1e-4


def test_checkpoint_roundtrip_and_hf_names(tmp_path):
    cfg = _tiny_cfg()
    model = build_model(cfg, dtype=torch.float32, seed=0)
    data = _batches(6, cfg.vocab_size)
    tr = ChronicalsTrainer(model, _args(tmp_path, save_steps=3, save_total_limit=1), data[:3])
    tr.train()
    ck = os.path.join(str(tmp_path), "checkpoint-3")
    assert os.path.exists(os.path.join(ck, "model.safetensors")) and os.path.exists(os.path.join(ck, "config.json"))
    keys = set(ckpt.read_weights(ck).keys())
    assert "model.embed_tokens.weight" in keys and "model.layers.0.self_attn.q_proj.weight" in keys
    assert "model.layers.1.mlp.gate_proj.weight" in keys and "model.layers.0.self_attn.k_proj.bias" in keys
    assert "lm_head.weight" not in keys                       # tied
    st = json.load(open(os.path.join(ck, "trainer_state.json")))
    assert st["global_step"] == 3 and st["micro_step"] == 3
    next_loss = tr.training_step(data[3]).item()
    model2 = build_model(cfg, dtype=torch.float32, seed=123)
    tr2 = ChronicalsTrainer(model2, _args(tmp_path), data[:3])
    tr2.load_checkpoint(ck)
    assert tr2.state.global_step == 3 and tr2.optimizer.step_count == 3
    assert abs(tr2.training_step(data[3]).item() - next_loss) < 1e-6
    for p, q in zip(model.parameters(), model2.parameters()):
        assert torch.allclose(p, q, atol=1e-7)


def test_save_total_limit_prunes(tmp_path):
    cfg = _tiny_cfg(1)
    tr = ChronicalsTrainer(build_model(cfg, dtype=torch.float32, seed=0),
                           _args(tmp_path, save_steps=1, save_total_limit=2), _batches(4, cfg.vocab_size))
    tr.train()
    kept = sorted(d for d in os.listdir(tmp_path) if d.startswith("checkpoint-") and d[11:].isdigit())
    assert kept == ["checkpoint-3", "checkpoint-4"]


def test_transformers_loads_our_checkpoint(tmp_path):
    transformers = pytest.importorskip("transformers")
    cfg = _tiny_cfg()
    model = build_model(cfg, dtype=torch.float32, seed=0).eval()
    ckpt.save_model(model, str(tmp_path))
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), torch_dtype=torch.float32).eval()
    ids = torch.randint(0, cfg.vocab_size, (1, 24))
    with torch.no_grad():
        ours = model(ids, return_logits=True).logits
        theirs = hf(ids).logits
    assert torch.allclose(ours, theirs, atol=2e-4), (ours - theirs).abs().max()


def test_readme_style_constructor(tmp_path):
    cfg = ChronicalsConfig(learning_rate=3e-4, batch_size=2, max_steps=2, use_lora=True, lora_rank=4,
                           mixed_precision="fp32")
    t = cfg.to_training_config(output_dir=str(tmp_path))
    assert t.learning_rate == 3e-4 and t.per_device_train_batch_size == 2 and t.max_steps == 2 and t.use_lora


@pytest.mark.parametrize("world", [2])
def test_dp_gloo_matches_single_process(tmp_path, world):
    """DP=2 over gloo with per-rank batch b equals one process with the concatenated batch."""
    script = os.path.join(ROOT, "tests", "_dp_worker.py")
    out = os.path.join(str(tmp_path), "dp.json")
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", script, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.load(open(out))
    assert max(abs(a - b) for a, b in zip(res["dp_losses"], res["single_losses"])) < 1e-4
    assert res["max_param_diff"] < 1e-4


def test_resume_in_the_middle_of_the_second_epoch_skips_only_that_epochs_batches(tmp_path):
    """The data cursor of a checkpoint counts micro-batches inside its epoch: resuming from step 5 of a run with
    3 batches per epoch continues with the third batch of epoch 1, not after a skip of five."""
    cfg = _tiny_cfg(1)
    data = _batches(3, cfg.vocab_size)
    full = ChronicalsTrainer(build_model(cfg, dtype=torch.float32, seed=0),
                             _args(tmp_path / "a", num_train_epochs=3, save_steps=5, save_total_limit=5), data)
    full.train()
    want = [h["loss"] for h in full.state.log_history if "lr" in h]
    assert len(want) == 9
    ck = os.path.join(str(tmp_path / "a"), "checkpoint-5")
    st = json.load(open(os.path.join(ck, "trainer_state.json")))
    assert st["epoch"] == 1 and st["micro_in_epoch"] == 2 and st["micro_step"] == 5
    resumed = ChronicalsTrainer(build_model(cfg, dtype=torch.float32, seed=7),
                                _args(tmp_path / "b", num_train_epochs=3), data)
    resumed.train(resume_from_checkpoint=ck)
    got = [h["loss"] for h in resumed.state.log_history if "lr" in h]
    assert resumed.state.global_step == 9
    assert len(got) == 9 and max(abs(a - b) for a, b in zip(got[5:], want[5:])) < 1e-6, (got, want)


def test_fused_adamw_state_stays_fp32_after_loading_into_bf16_parameters():
    """``torch.optim.Optimizer.load_state_dict`` casts floating-point state to the parameter dtype; the fused
    optimizer's moments and master copy must come back as fp32 (the kernel reads them as such)."""
    from chronicals_b200.optimizers import FusedAdamW
    from chronicals_b200.optimizers.optimizers_8bit import AdamW8bit
    p = torch.nn.Parameter(torch.randn(64, 96).to(torch.bfloat16))
    opt = FusedAdamW([p], lr=1e-2, master_weights=True)
    p.grad = torch.randn_like(p)
    opt.step()
    sd = opt.state_dict()
    q = torch.nn.Parameter(p.detach().clone())
    opt2 = FusedAdamW([q], lr=1e-2, master_weights=True)
    opt2.load_state_dict(sd)
    st = opt2.state[q]
    assert st["exp_avg"].dtype == st["exp_avg_sq"].dtype == st["master"].dtype == torch.float32
    assert torch.equal(st["exp_avg"], opt.state[p]["exp_avg"]) and opt2.step_count == 1
    # continuing from the loaded state equals continuing the original
    g = torch.randn_like(p)
    p.grad, q.grad = g.clone(), g.clone()
    opt.step()
    opt2.step()
    assert torch.equal(p, q)
    # 8-bit moments keep their integer codes and fp32 block maxima
    r = torch.nn.Parameter(torch.randn(8192).to(torch.bfloat16))
    o8 = AdamW8bit([r], lr=1e-2)
    r.grad = torch.randn_like(r)
    o8.step()
    r2 = torch.nn.Parameter(r.detach().clone())
    o8b = AdamW8bit([r2], lr=1e-2)
    o8b.load_state_dict(o8.state_dict())
    s8 = o8b.state[r2]
    assert s8["exp_avg"].dtype == torch.int8 and s8["exp_avg_sq"].dtype == torch.uint8
    assert s8["exp_avg_absmax"].dtype == torch.float32 and torch.equal(s8["exp_avg_absmax"], o8.state[r]["exp_avg_absmax"])
