"""Optimizers, schedulers, LoRA / LoRA+ on CPU."""
import math

import pytest
import torch
import torch.nn as nn

from chronicals_b200 import ChronicalsConfig, build_model
from chronicals_b200.lora.lora_optimized import (LoRAModel, OptimizedLoRALinear, apply_lora_to_model, count_lora_params)
from chronicals_b200.optimizers import (AdamAtan2, AdamW8bit, FusedAdamW, HybridMuonAdamW, LoRAPlusAdamW,
                                        LoRAPlusOptimizer, LoRAPlusParameterGroups, Muon, OneCycleLR, ScheduleFreeAdamW,
                                        WSDScheduler, create_lora_plus_optimizer, create_optimizer, create_scheduler,
                                        newton_schulz_orthogonalize)


def _quad_problem(opt_fn, steps=200):
    torch.manual_seed(0)
    w = nn.Parameter(torch.randn(16, 16))
    target = torch.randn(16, 16)
    opt = opt_fn([w])
    first = None
    for _ in range(steps):
        loss = (w - target).pow(2).mean()
        first = first or loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    return first, loss.item()


@pytest.mark.parametrize("name,fn", [
    ("fused_adamw", lambda p: FusedAdamW(p, lr=5e-2, weight_decay=0.0)),
    ("schedule_free", lambda p: ScheduleFreeAdamW(p, lr=5e-2)),
    ("muon", lambda p: Muon(p, lr=5e-2)),
    ("adam_atan2", lambda p: AdamAtan2(p, lr=2e-2)),
    ("adamw8bit", lambda p: AdamW8bit(p, lr=5e-2, weight_decay=0.0, min_8bit_size=16)),
])
def test_optimizers_reduce_a_quadratic(name, fn):
    first, last = _quad_problem(fn)
    assert last < 0.2 * first, (name, first, last)


def test_schedule_free_eval_train_swap():
    w = nn.Parameter(torch.ones(4))
    opt = ScheduleFreeAdamW([w], lr=0.1)
    for _ in range(3):
        w.grad = torch.ones(4)
        opt.step()
    x = w.detach().clone()
    opt.eval_mode()
    assert not torch.equal(w.detach(), x)
    opt.train_mode()
    assert torch.equal(w.detach(), x)


def test_newton_schulz_orthogonalises():
    g = torch.randn(32, 48)
    o = newton_schulz_orthogonalize(g, steps=12)
    s = torch.linalg.svdvals(o.float())
    assert s.max() < 1.3 and s.min() > 0.3


def test_wsd_schedule_shape_and_group_ratio():
    a, b = nn.Parameter(torch.zeros(1)), nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([{"params": [a], "lr": 1.0}, {"params": [b], "lr": 16.0}])
    sch = WSDScheduler(opt, total_steps=100, warmup_ratio=0.1, stable_ratio=0.6, min_lr_ratio=0.1)
    lrs = []
    for _ in range(100):
        lrs.append([g["lr"] for g in opt.param_groups])
        opt.step()
        sch.step()
    assert abs(lrs[0][0] - 0.1) < 1e-9 and abs(lrs[9][0] - 1.0) < 1e-9
    assert all(abs(l[0] - 1.0) < 1e-9 for l in lrs[10:70])
    assert lrs[99][0] < 0.12 and all(x[0] >= y[0] - 1e-12 for x, y in zip(lrs[70:], lrs[71:]))
    assert all(abs(l[1] / l[0] - 16.0) < 1e-9 for l in lrs)
    assert sch.state_dict()["last_epoch"] == 100


def test_one_cycle_keeps_group_ratio_and_factories():
    a, b = nn.Parameter(torch.zeros(1)), nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([{"params": [a], "lr": 1.0}, {"params": [b], "lr": 16.0}])
    sch = OneCycleLR(opt, total_steps=50)
    peak = 0
    for _ in range(50):
        peak = max(peak, opt.param_groups[0]["lr"])
        assert abs(opt.param_groups[1]["lr"] / opt.param_groups[0]["lr"] - 16) < 1e-9
        opt.step()
        sch.step()
    assert abs(peak - 1.0) < 1e-6 and opt.param_groups[0]["lr"] < 1e-3
    m = nn.Linear(4, 4)
    for t in ("fused_adamw", "adamw", "schedule_free", "muon", "hybrid_muon", "8bit_adam", "adam_atan2"):
        assert create_optimizer(m, t, lr=1e-3) is not None
    for s in ("wsd", "one_cycle", "cosine", "constant"):
        assert create_scheduler(torch.optim.SGD(m.parameters(), lr=1.0), s, 10) is not None


class _Dummy(nn.Module):
    def __init__(self):
        super().__init__()
        self.base = nn.Linear(8, 8)
        self.lora_A = nn.Linear(8, 2, bias=False)
        self.lora_B = nn.Linear(2, 8, bias=False)


def test_lora_plus_groups_and_ratio():
    m = _Dummy()
    groups = LoRAPlusParameterGroups().get_param_groups(m, base_lr=2e-4, lr_ratio=16.0, weight_decay=0.01,
                                                        weight_decay_lora=0.0)
    by = {g["name"]: g for g in groups}
    assert by["lora_A"]["lr"] == 2e-4 and abs(by["lora_B"]["lr"] - 3.2e-3) < 1e-12
    assert by["other"]["weight_decay"] == 0.01 and by["lora_A"]["weight_decay"] == 0.0
    assert LoRAPlusOptimizer is LoRAPlusAdamW
    opt = create_lora_plus_optimizer(m, base_lr=2e-4, lr_ratio=16.0)
    lrs = opt.get_lr_by_group()
    assert abs(lrs["lora_B"] / lrs["lora_A"] - 16.0) < 1e-9
    with pytest.raises(ValueError):
        LoRAPlusParameterGroups().get_param_groups(m, lr_ratio=0.5)
    assert LoRAPlusParameterGroups().classify("base_model.model.layers.0.q_proj.lora_A.default.weight") == "lora_A"
    assert LoRAPlusParameterGroups().classify("model.layers.0.self_attn.qkv_proj.lora_B.q_proj") == "lora_B"


def test_optimized_lora_linear_inits_and_merge():
    torch.manual_seed(0)
    base = nn.Linear(24, 16)
    x = torch.randn(5, 24)
    y0 = base(x)
    for init in ("kaiming", "pissa", "olora"):
        lin = nn.Linear(24, 16)
        lin.load_state_dict(base.state_dict())
        l = OptimizedLoRALinear(lin, rank=4, alpha=8.0, init_method=init)
        assert l.lora_A.shape == (4, 24) and l.lora_B.shape == (16, 4)
        assert torch.allclose(l(x), y0, atol=1e-4), init            # function unchanged at initialisation
        with torch.no_grad():
            l.lora_B.add_(0.1 * torch.randn_like(l.lora_B))
        y1 = l(x)
        l.merge()
        assert torch.allclose(l(x), y1, atol=1e-4)
        l.unmerge()
        assert torch.allclose(l(x), y1, atol=1e-4)


def test_lora_on_native_model_trains_only_adapters(tmp_path):
    cfg = ChronicalsConfig.from_model_name("tiny-qwen2")
    cfg.num_hidden_layers, cfg.vocab_size = 2, 512
    m = build_model(cfg, dtype=torch.float32, seed=0)
    ids = torch.randint(0, 512, (2, 32))
    base_loss = m(ids, labels=ids).loss.item()
    apply_lora_to_model(m, rank=4, alpha=8.0)
    lora, total = count_lora_params(m)
    assert 0 < lora < 0.1 * total
    assert all(("lora_" in n) == p.requires_grad for n, p in m.named_parameters())
    assert abs(m(ids, labels=ids).loss.item() - base_loss) < 1e-5      # B = 0 at init
    opt = create_lora_plus_optimizer(m, base_lr=1e-2, lr_ratio=16.0)
    frozen = {n: p.detach().clone() for n, p in m.named_parameters() if not p.requires_grad}
    for _ in range(8):
        loss = m(ids, labels=ids).loss
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < base_loss - 0.05
    assert all(torch.equal(frozen[n], p) for n, p in m.named_parameters() if n in frozen)
    # adapter checkpoint in PEFT naming, merge keeps the function
    from chronicals_b200.checkpoint import io as ckpt
    ckpt.save_lora_adapter(m, str(tmp_path), 4, 8.0, m.lora_config["target_modules"])
    from safetensors.torch import load_file
    keys = load_file(str(tmp_path / "adapter_model.safetensors")).keys()
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in keys
    assert "base_model.model.model.layers.1.mlp.down_proj.lora_B.weight" in keys
    wrapped = LoRAModel.__new__(LoRAModel)
    nn.Module.__init__(wrapped)
    wrapped.model = m
    l1 = m(ids, labels=ids).loss.item()
    wrapped.merge_lora()
    assert abs(m(ids, labels=ids).loss.item() - l1) < 1e-4
    wrapped.unmerge_lora()
    assert abs(m(ids, labels=ids).loss.item() - l1) < 1e-4


def test_hybrid_muon_state_dict_roundtrip():
    m = nn.Sequential()
    m.add_module("q_proj", nn.Linear(8, 8))
    m.add_module("norm", nn.LayerNorm(8))
    opt = HybridMuonAdamW(m, lr=1e-3)
    m(torch.randn(2, 8)).sum().backward()
    opt.step()
    sd = opt.state_dict()
    assert set(sd) == {"muon", "adamw"}
    opt.load_state_dict(sd)
