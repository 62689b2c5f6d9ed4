"""Self-contained LoRA fine-tuning example on top of ``chronicals_b200``.

Reference: examples/COLAB_LORA_TRAINER.py — ``LoRAConfig`` :58-108, ``TrainerConfig`` :111-201,
``CUDATimer`` :230-253, ``LoRAPlusOptimizer.create_param_groups`` :260-335, ``apply_lora_bracketing``
:338-353, ``SequencePacker`` :360-455, ``CutCrossEntropyLoss`` :462-589, ``ChronicalsLoRATrainer``
:596-1149 (``train``, ``save_model`` :1101-1119, ``from_pretrained`` :1121-1149),
``load_alpaca_dataset`` :1156-1196.

The reference example re-implements packing, the chunked loss and LoRA+ inline because its library
trainer never applies LoRA; here the example is a thin layer over the library, which has all three:
adapters on the fused projections, the fused linear-cross-entropy kernel, packing with per-document
attention, and the fused multi-tensor AdamW with LoRA+ groups.

Run ``python examples/lora_trainer.py --model tiny-qwen2 --max_steps 10`` (synthetic data, no network),
or pass ``--weights DIR`` with a HuggingFace-format checkpoint and ``--dataset FILE.jsonl`` with
``instruction``/``input``/``output`` records.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from chronicals_b200 import ChronicalsConfig, ChronicalsTrainer, TrainingConfig, build_model  # noqa: E402
from chronicals_b200.checkpoint.io import load_lora_adapter, load_model_weights, save_lora_adapter  # noqa: E402
from chronicals_b200.data.data_loader import InstructionDataset, create_packed_dataloader  # noqa: E402
from chronicals_b200.lora import apply_lora_to_model, count_lora_params  # noqa: E402

DEFAULT_TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


@dataclass
class LoRAConfig:
    r: int = 16
    lora_alpha: float = 32.0
    lora_dropout: float = 0.0
    target_modules: List[str] = field(default_factory=lambda: list(DEFAULT_TARGETS))
    use_lora_plus: bool = True
    lora_plus_ratio: float = 16.0

    def to_peft_config(self) -> Dict[str, Any]:
        return {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": self.r, "lora_alpha": self.lora_alpha,
                "lora_dropout": self.lora_dropout, "target_modules": list(self.target_modules), "bias": "none"}


@dataclass
class TrainerConfig:
    output_dir: str = "./lora_output"
    learning_rate: float = 2e-4
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    per_device_batch_size: int = 4          # packed rows per micro-batch
    gradient_accumulation_steps: int = 1
    max_seq_length: int = 1024
    num_epochs: int = 1
    max_steps: int = -1
    warmup_ratio: float = 0.03
    lr_scheduler_type: str = "cosine"
    logging_steps: int = 10
    save_steps: int = 0
    use_packing: bool = True
    packing_strategy: str = "bfd"
    use_cuda_graphs: bool = True
    use_gradient_checkpointing: bool = False
    seed: int = 42

    def to_training_config(self, lora: LoRAConfig) -> TrainingConfig:
        cfg = TrainingConfig(
            output_dir=self.output_dir, learning_rate=self.learning_rate, weight_decay=self.weight_decay,
            max_grad_norm=self.max_grad_norm, per_device_train_batch_size=self.per_device_batch_size,
            gradient_accumulation_steps=self.gradient_accumulation_steps, max_seq_length=self.max_seq_length,
            num_train_epochs=self.num_epochs, max_steps=self.max_steps, warmup_ratio=self.warmup_ratio,
            lr_scheduler_type=self.lr_scheduler_type, logging_steps=self.logging_steps, save_steps=self.save_steps,
            use_sequence_packing=self.use_packing, use_gradient_checkpointing=self.use_gradient_checkpointing,
            use_cuda_graphs=self.use_cuda_graphs and self.gradient_accumulation_steps == 1, fp8=False,
            visual_reporting=False, seed=self.seed,
            optimizer_type="lora_plus" if lora.use_lora_plus else "fused_adamw")
        cfg.lora_plus_ratio = lora.lora_plus_ratio
        cfg.save_final = False
        return cfg


class CUDATimer:
    def __enter__(self):
        self.cuda = torch.cuda.is_available()
        if self.cuda:
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.a.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self.b.record()
            torch.cuda.synchronize()
            self.elapsed = self.a.elapsed_time(self.b) / 1e3
        else:
            self.elapsed = time.perf_counter() - self.t0
        return False


def apply_lora_bracketing(model) -> None:
    """Kept for API parity.  The evaluation order ``(x Aᵀ) Bᵀ`` is built into the adapter forward of
    this library (two skinny GEMMs instead of materialising ``B A``), so there is nothing to patch."""
    return None


class ByteTokenizer:
    """Offline stand-in tokenizer (UTF-8 bytes + 2 specials) for runs without a tokenizer directory."""
    pad_token_id, eos_token_id = 0, 1
    vocab_size = 258

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        return [b + 2 for b in text.encode("utf-8")]

    def decode(self, ids: Iterable[int]) -> str:
        return bytes(i - 2 for i in ids if i >= 2).decode("utf-8", errors="replace")


def load_alpaca_dataset(path: Optional[str] = None, max_samples: int = 1000, seed: int = 0) -> List[Dict[str, str]]:
    """Instruction records from a local ``.json``/``.jsonl`` file, or seeded synthetic ones."""
    if path:
        with open(path) as f:
            rows = json.load(f) if path.endswith(".json") else [json.loads(l) for l in f if l.strip()]
        return rows[:max_samples]
    g = torch.Generator().manual_seed(seed)
    words = ["pack", "tensor", "kernel", "gradient", "token", "adapter", "rank", "matrix", "norm", "stream", "cache", "tile"]
    def sent(n):
        return " ".join(words[int(i)] for i in torch.randint(0, len(words), (n,), generator=g))
    return [{"instruction": "Explain " + sent(4), "input": "", "output": sent(int(torch.randint(8, 60, (1,), generator=g)))}
            for _ in range(max_samples)]


class ChronicalsLoRATrainer:
    """``ChronicalsLoRATrainer(model_name, lora_config, trainer_config, tokenizer).train(dataset)``"""

    def __init__(self, model_name: str = "qwen2.5-0.5b", lora_config: Optional[LoRAConfig] = None,
                 trainer_config: Optional[TrainerConfig] = None, tokenizer=None, weights: Optional[str] = None,
                 device: Optional[str] = None):
        self.model_name = model_name
        self.lora_config = lora_config or LoRAConfig()
        self.config = trainer_config or TrainerConfig()
        self.tokenizer = tokenizer or ByteTokenizer()
        dev = torch.device(device or ("cuda:0" if torch.cuda.is_available() else "cpu"))
        self.model_config = ChronicalsConfig.from_model_name(model_name)
        self.model = build_model(self.model_config, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                                 device=dev, seed=self.config.seed)
        if weights:
            load_model_weights(self.model, weights, strict=False)
        lc = self.lora_config
        apply_lora_to_model(self.model, rank=lc.r, alpha=lc.lora_alpha, target_modules=lc.target_modules, dropout=lc.lora_dropout)
        apply_lora_bracketing(self.model)
        self.trainable, self.total = count_lora_params(self.model)
        self.history: List[Dict[str, float]] = []

    def _loader(self, dataset: Sequence[Dict[str, Any]]):
        if len(dataset) and isinstance(dataset[0], dict) and "input_ids" not in dataset[0]:
            dataset = InstructionDataset(dataset, self.tokenizer, self.config.max_seq_length)
        return create_packed_dataloader(dataset, batch_size=self.config.per_device_batch_size,
                                        max_length=self.config.max_seq_length, strategy=self.config.packing_strategy,
                                        use_packing=self.config.use_packing,
                                        pad_token_id=getattr(self.tokenizer, "pad_token_id", 0) or 0,
                                        pin_memory=torch.cuda.is_available())

    def train(self, train_dataset, eval_dataset=None, num_epochs: Optional[int] = None, max_steps: Optional[int] = None):
        if num_epochs is not None:
            self.config.num_epochs = num_epochs
        if max_steps is not None:
            self.config.max_steps = max_steps
        targs = self.config.to_training_config(self.lora_config)
        trainer = ChronicalsTrainer(self.model, targs, self._loader(train_dataset),
                                    eval_dataloader=self._loader(eval_dataset) if eval_dataset is not None else None,
                                    tokenizer=self.tokenizer, model_config=self.model_config)
        with CUDATimer() as t:
            state = trainer.train()
        self.state = state
        tokens = getattr(state, "total_tokens", 0) or getattr(state, "tokens_seen", 0)
        self.history.append({"steps": state.global_step, "seconds": t.elapsed, "tokens": float(tokens),
                             "tokens_per_sec": float(tokens) / t.elapsed if t.elapsed > 0 else 0.0})
        return state

    def save_model(self, out_dir: Optional[str] = None) -> str:
        out = out_dir or os.path.join(self.config.output_dir, "final")
        lc = self.lora_config
        save_lora_adapter(self.model, out, lc.r, lc.lora_alpha, lc.target_modules, lc.lora_dropout, self.model_name)
        with open(os.path.join(out, "trainer_config.json"), "w") as f:
            json.dump({"trainer": asdict(self.config), "lora": asdict(lc), "model_name": self.model_name}, f, indent=2)
        return out

    @classmethod
    def from_pretrained(cls, adapter_dir: str, tokenizer=None, weights: Optional[str] = None) -> "ChronicalsLoRATrainer":
        with open(os.path.join(adapter_dir, "trainer_config.json")) as f:
            saved = json.load(f)
        self = cls(saved["model_name"], LoRAConfig(**saved["lora"]), TrainerConfig(**saved["trainer"]), tokenizer, weights)
        load_lora_adapter(self.model, adapter_dir)
        return self


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-0.5b")
    ap.add_argument("--weights", default=None, help="directory with HuggingFace-format weights (optional)")
    ap.add_argument("--dataset", default=None, help="local .json/.jsonl instruction file (optional)")
    ap.add_argument("--max_samples", type=int, default=512)
    ap.add_argument("--max_steps", type=int, default=20)
    ap.add_argument("--batch_size", type=int, default=4)
    ap.add_argument("--seq_length", type=int, default=1024)
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--output_dir", default="./lora_output")
    a = ap.parse_args(argv)
    tcfg = TrainerConfig(output_dir=a.output_dir, per_device_batch_size=a.batch_size, max_seq_length=a.seq_length,
                         max_steps=a.max_steps, logging_steps=max(1, a.max_steps // 5))
    t = ChronicalsLoRATrainer(a.model, LoRAConfig(r=a.rank, lora_alpha=2.0 * a.rank), tcfg, weights=a.weights)
    print(f"trainable parameters: {t.trainable:,} of {t.total:,} ({100.0 * t.trainable / t.total:.2f} %)")
    state = t.train(load_alpaca_dataset(a.dataset, a.max_samples))
    out = t.save_model()
    print(f"finished {state.global_step} steps; adapter saved to {out}; {t.history[-1]}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
