"""Checkpoint reading and writing in HuggingFace-compatible layouts.

A checkpoint directory holds:

* ``model.safetensors`` (or ``model-0000i-of-0000n.safetensors`` plus
  ``model.safetensors.index.json`` when sharded) under HuggingFace parameter
  names, and ``config.json`` — loadable by ``transformers``;
* for LoRA runs ``adapter_model.safetensors`` + ``adapter_config.json`` with
  PEFT key names (``base_model.model.<module>.lora_A.weight`` ``[r, in]``,
  ``lora_B.weight`` ``[out, r]``);
* ``optimizer.pt``, ``scheduler.pt``, ``trainer_state.json`` (global step, epoch,
  best loss, token/time totals, RNG states, data cursor), ``training_history.json``.

The reference writes five ``torch.save`` files and restores neither RNG state
nor the data position, and never prunes old checkpoints
(chronicals/training/chronicals_trainer.py:2012-2089); ``load_model_weights``
still reads its ``model.pt`` layout.
"""
from __future__ import annotations

import json
import os
import random
import shutil
from typing import Any, Dict, List, Optional

import numpy as np
import torch

try:
    from safetensors.torch import load_file as _st_load, save_file as _st_save
    HAVE_SAFETENSORS = True
except Exception:  # pragma: no cover
    HAVE_SAFETENSORS = False

MAX_SHARD_BYTES = 5 * 2**30


def _model_hf_state(model) -> Dict[str, torch.Tensor]:
    if hasattr(model, "hf_state_dict"):
        return model.hf_state_dict()
    return {k: v.detach() for k, v in model.state_dict().items()}


def save_model(model, out_dir: str, max_shard_bytes: int = MAX_SHARD_BYTES, safe: bool = True,
               state: Optional[Dict[str, torch.Tensor]] = None) -> List[str]:
    """Write weights (+``config.json`` when the model carries a config). Returns written file names.
    ``state`` overrides the model's own state dict (used for models whose full state has to be gathered
    from several ranks first)."""
    os.makedirs(out_dir, exist_ok=True)
    sd = {k: v.detach().to("cpu").contiguous().clone() for k, v in (state or _model_hf_state(model)).items()}
    cfg = getattr(model, "config", None)
    if cfg is not None and hasattr(cfg, "to_hf_config"):
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(cfg.to_hf_config(), f, indent=2)
    if not (safe and HAVE_SAFETENSORS):
        torch.save(sd, os.path.join(out_dir, "model.pt"))
        return ["model.pt"]
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k, v in sd.items():
        nb = v.numel() * v.element_size()
        if size + nb > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][k] = v
        size += nb
    if len(shards) == 1:
        _st_save(shards[0], os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
        return ["model.safetensors"]
    names, index = [], {"metadata": {"total_size": sum(v.numel() * v.element_size() for v in sd.values())},
                        "weight_map": {}}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        _st_save(sh, os.path.join(out_dir, name), metadata={"format": "pt"})
        names.append(name)
        for k in sh:
            index["weight_map"][k] = name
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f, indent=2)
    return names


def read_weights(ckpt_dir: str) -> Dict[str, torch.Tensor]:
    """All tensors of a checkpoint directory (safetensors, sharded safetensors, or ``model.pt``)."""
    idx = os.path.join(ckpt_dir, "model.safetensors.index.json")
    single = os.path.join(ckpt_dir, "model.safetensors")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        out: Dict[str, torch.Tensor] = {}
        for name in files:
            out.update(_st_load(os.path.join(ckpt_dir, name)))
        return out
    if os.path.exists(single):
        return _st_load(single)
    pt = os.path.join(ckpt_dir, "model.pt")
    if os.path.exists(pt):
        return torch.load(pt, map_location="cpu", weights_only=True)
    raise FileNotFoundError(f"no model weights found in {ckpt_dir}")


def load_model_weights(model, ckpt_dir: str, strict: bool = True) -> List[str]:
    sd = read_weights(ckpt_dir)
    if hasattr(model, "load_hf_state_dict"):
        own_keys = set(model.state_dict().keys())
        if own_keys and own_keys.issubset(sd.keys()) and not any(k.endswith("q_proj.weight") for k in sd):
            model.load_state_dict(sd, strict=strict)      # our own fused layout saved with torch.save
            return []
        return model.load_hf_state_dict(sd, strict=strict)
    res = model.load_state_dict(sd, strict=strict)
    return list(getattr(res, "missing_keys", []))


# --------------------------------------------------------------------------------------------- LoRA adapters
def lora_state_dict(model) -> Dict[str, torch.Tensor]:
    """PEFT-named adapter tensors of a model whose projections carry LoRA."""
    out: Dict[str, torch.Tensor] = {}
    if hasattr(model, "hf_state_dict"):
        for k, v in model.hf_state_dict(include_lora=True).items():
            if ".lora_A." in k or ".lora_B." in k:
                out["base_model.model." + k] = v
        return out
    for k, v in model.state_dict().items():
        if "lora_" in k:
            out["base_model.model." + k.replace(".default", "")] = v.detach()
    return out


def save_lora_adapter(model, out_dir: str, rank: int, alpha: float, target_modules: List[str],
                      dropout: float = 0.0, base_model_name: str = "") -> None:
    os.makedirs(out_dir, exist_ok=True)
    sd = {k: v.detach().cpu().contiguous().clone() for k, v in lora_state_dict(model).items()}
    if HAVE_SAFETENSORS:
        _st_save(sd, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
    else:
        torch.save(sd, os.path.join(out_dir, "adapter_model.bin"))
    cfg = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": rank, "lora_alpha": alpha, "lora_dropout": dropout,
           "target_modules": list(target_modules), "bias": "none", "base_model_name_or_path": base_model_name,
           "inference_mode": True, "fan_in_fan_out": False}
    with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)


def load_lora_adapter(model, adapter_dir: str) -> int:
    """Copy adapter tensors into an already LoRA-equipped model; returns the number loaded."""
    path = os.path.join(adapter_dir, "adapter_model.safetensors")
    sd = _st_load(path) if os.path.exists(path) else torch.load(os.path.join(adapter_dir, "adapter_model.bin"),
                                                               map_location="cpu", weights_only=True)
    sd = {k[len("base_model.model."):] if k.startswith("base_model.model.") else k: v for k, v in sd.items()}
    sd = {k.replace(".default", ""): v for k, v in sd.items()}
    n = 0
    if hasattr(model, "hf_state_dict"):
        own = model.hf_state_dict(include_lora=True)
        with torch.no_grad():
            for k, dst in own.items():
                if k in sd and ("lora_A" in k or "lora_B" in k):
                    dst.copy_(sd[k].to(dst.dtype))
                    n += 1
        return n
    own = model.state_dict()
    with torch.no_grad():
        for k, v in sd.items():
            if k in own:
                own[k].copy_(v.to(own[k].dtype))
                n += 1
    return n


# --------------------------------------------------------------------------------------------- trainer state
def rng_state() -> Dict[str, Any]:
    st = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state_all()
    return st


def set_rng_state(st: Dict[str, Any]) -> None:
    if "python" in st:
        random.setstate(st["python"])
    if "numpy" in st:
        np.random.set_state(st["numpy"])
    if "torch" in st:
        torch.set_rng_state(st["torch"])
    if "cuda" in st and torch.cuda.is_available():
        try:
            torch.cuda.set_rng_state_all(st["cuda"])
        except Exception:
            pass


def save_training_state(out_dir: str, optimizer=None, scheduler=None, trainer_state: Optional[Dict[str, Any]] = None,
                        history: Optional[List[Dict[str, Any]]] = None, rank: int = 0, world_size: int = 1) -> None:
    os.makedirs(out_dir, exist_ok=True)
    suffix = "" if world_size == 1 else f".rank{rank}"
    if optimizer is not None:
        torch.save(optimizer.state_dict(), os.path.join(out_dir, f"optimizer{suffix}.pt"))
    if scheduler is not None:
        torch.save(scheduler.state_dict(), os.path.join(out_dir, "scheduler.pt"))
    torch.save(rng_state(), os.path.join(out_dir, f"rng_state{suffix}.pt"))
    if rank == 0:
        if trainer_state is not None:
            with open(os.path.join(out_dir, "trainer_state.json"), "w") as f:
                json.dump(trainer_state, f, indent=2, default=float)
        if history is not None:
            with open(os.path.join(out_dir, "training_history.json"), "w") as f:
                json.dump(history, f, default=float)


def _state_kind(sd: Dict[str, Any]) -> str:
    if "zero3" in sd:
        return "zero3"
    return str(sd.get("kind", "replicated"))


def _optimizer_kind(optimizer) -> str:
    name = type(optimizer).__name__
    return {"Zero3Optimizer": "zero3", "ShardedFusedAdamW": "zero1"}.get(name, "replicated")


def consolidate_optimizer_states(states: List[Dict[str, Any]]) -> Dict[str, Any]:
    """Optimizer files of all saved ranks → per-parameter exchange form: ``exp_avg`` / ``exp_avg_sq`` as lists of
    flat fp32 tensors in parameter order, ``step_count``, ``param_groups`` (hyper-parameters only)."""
    kind = _state_kind(states[0])
    if kind == "zero3":
        from ..parallel.zero3 import consolidate_zero3_states
        return consolidate_zero3_states(states)
    if kind == "zero1":
        from ..parallel.zero import consolidate_states
        return consolidate_states(states)
    sd = states[0]                                               # torch-style state dict, identical on every rank
    ids = [i for g in sd["param_groups"] for i in g["params"]]
    out: Dict[str, Any] = {"step_count": int(sd.get("step_count", 0)), "master": None,
                           "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in sd["param_groups"]]}
    for name in ("exp_avg", "exp_avg_sq"):
        out[name] = [sd["state"][i][name].reshape(-1).float() for i in ids if i in sd["state"]]
    if not out["step_count"] and ids and ids[0] in sd["state"] and "step" in sd["state"][ids[0]]:
        out["step_count"] = int(sd["state"][ids[0]]["step"])
    return out


def saved_world_size(ckpt_dir: str) -> int:
    """Number of ranks that wrote the optimizer files of a checkpoint directory (0 when there are none)."""
    if os.path.exists(os.path.join(ckpt_dir, "optimizer.pt")):
        return 1
    n = 0
    while os.path.exists(os.path.join(ckpt_dir, f"optimizer.rank{n}.pt")):
        n += 1
    return n


def load_training_state(ckpt_dir: str, optimizer=None, scheduler=None, rank: int = 0, world_size: int = 1,
                        restore_rng: bool = True) -> Dict[str, Any]:
    suffix = "" if world_size == 1 else f".rank{rank}"
    saved_world = saved_world_size(ckpt_dir)
    if optimizer is not None and saved_world:
        mine = os.path.join(ckpt_dir, f"optimizer{suffix}.pt")
        first = torch.load(mine if (saved_world == world_size and os.path.exists(mine)) else
                           os.path.join(ckpt_dir, "optimizer.pt" if saved_world == 1 else "optimizer.rank0.pt"),
                           map_location="cpu", weights_only=False)
        if saved_world == world_size and _state_kind(first) == _optimizer_kind(optimizer):
            optimizer.load_state_dict(first)
        else:
            # elastic restart (another number of ranks, or another sharding of the optimizer state): bring the
            # saved state into the per-parameter exchange form and let the optimizer lay it out for itself
            names = ["optimizer.pt"] if saved_world == 1 else [f"optimizer.rank{r}.pt" for r in range(saved_world)]
            kind = _state_kind(first)
            states = [first] if kind == "replicated" else [
                torch.load(os.path.join(ckpt_dir, n), map_location="cpu", weights_only=False) for n in names]
            if kind == _optimizer_kind(optimizer) and hasattr(optimizer, "load_resharded"):
                optimizer.load_resharded(states)
            elif hasattr(optimizer, "load_consolidated"):
                optimizer.load_consolidated(consolidate_optimizer_states(states))
            else:
                optimizer.load_state_dict(first)
            if saved_world != world_size:
                suffix = "" if saved_world == 1 else ".rank0"       # RNG: every new rank continues rank 0's stream
    p = os.path.join(ckpt_dir, "scheduler.pt")
    if scheduler is not None and os.path.exists(p):
        scheduler.load_state_dict(torch.load(p, map_location="cpu", weights_only=False))
    p = os.path.join(ckpt_dir, f"rng_state{suffix}.pt")
    if restore_rng and os.path.exists(p):
        set_rng_state(torch.load(p, map_location="cpu", weights_only=False))
    state: Dict[str, Any] = {}
    p = os.path.join(ckpt_dir, "trainer_state.json")
    if os.path.exists(p):
        with open(p) as f:
            state = json.load(f)
    else:
        p = os.path.join(ckpt_dir, "trainer_state.pt")        # the reference's layout
        if os.path.exists(p):
            state = dict(torch.load(p, map_location="cpu", weights_only=False))
    return state


def prune_checkpoints(output_dir: str, keep: int, prefix: str = "checkpoint-") -> List[str]:
    """Delete the oldest ``checkpoint-<step>`` directories beyond ``keep`` (``save_total_limit``)."""
    if keep is None or keep <= 0 or not os.path.isdir(output_dir):
        return []
    items = []
    for name in os.listdir(output_dir):
        tail = name[len(prefix):]
        if name.startswith(prefix) and tail.isdigit():
            items.append((int(tail), name))
    items.sort()
    removed = []
    for _, name in items[:-keep] if len(items) > keep else []:
        shutil.rmtree(os.path.join(output_dir, name), ignore_errors=True)
        removed.append(name)
    return removed
