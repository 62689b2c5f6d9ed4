"""Quick start: the same LoRA pipeline as ``examples/lora_trainer.py`` as short, copyable steps.

Reference: examples/COLAB_QUICKSTART_LORA.py (notebook cell strings of the LoRA pipeline with the
expected throughput per GPU at :55-56).  Each ``STEP_*`` string below is one cell; ``python
examples/quickstart_lora.py`` executes them in order on a tiny model with synthetic data.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

EXPECTED_TOKENS_PER_SEC = {"B200 (measured, full fine-tune 0.5B)": 180_000, "A100-40GB (published by the reference, LoRA)": 11_699}

STEP_1_BUILD = '''
import __graft_entry__ as entry          # compiles the sm_100a kernels once (nvcc); cached by content hash
entry.build()
'''

STEP_2_MODEL = '''
import torch
from chronicals_b200 import ChronicalsConfig, build_model
from chronicals_b200.lora import LoRAConfig, apply_lora
device = "cuda:0" if torch.cuda.is_available() else "cpu"
cfg = ChronicalsConfig.from_model_name(MODEL_NAME)
model = build_model(cfg, dtype=torch.bfloat16 if device != "cpu" else torch.float32, device=device, seed=0)
apply_lora(model, LoRAConfig(rank=16, alpha=32.0))
'''

STEP_3_DATA = '''
from examples.lora_trainer import ByteTokenizer, load_alpaca_dataset
from chronicals_b200.data.data_loader import InstructionDataset, create_packed_dataloader
tok = ByteTokenizer()
records = load_alpaca_dataset(None, max_samples=128)
loader = create_packed_dataloader(InstructionDataset(records, tok, 256), batch_size=2, max_length=256, pin_memory=False)
'''

STEP_4_TRAIN = '''
from chronicals_b200 import ChronicalsTrainer, TrainingConfig
args = TrainingConfig(output_dir="/tmp/quickstart_lora", learning_rate=2e-4, optimizer_type="lora_plus", max_steps=8,
                      per_device_train_batch_size=2, max_seq_length=256, logging_steps=2, save_steps=0,
                      visual_reporting=False, fp8=False, use_gradient_checkpointing=False)
args.save_final = False
state = ChronicalsTrainer(model, args, loader, tokenizer=tok, model_config=cfg).train()
'''

STEP_5_SAVE = '''
from chronicals_b200.checkpoint.io import save_lora_adapter
save_lora_adapter(model, "/tmp/quickstart_lora/adapter", 16, 32.0, model.lora_config["target_modules"])
'''


def main() -> int:
    env = {"MODEL_NAME": os.environ.get("QUICKSTART_MODEL", "tiny-qwen2")}
    steps = [STEP_2_MODEL, STEP_3_DATA, STEP_4_TRAIN, STEP_5_SAVE]
    if os.environ.get("QUICKSTART_BUILD", "0") == "1":
        steps.insert(0, STEP_1_BUILD)
    for cell in steps:
        exec(compile(cell, "<quickstart cell>", "exec"), env)
    print(f"done: {env['state'].global_step} steps; adapter in /tmp/quickstart_lora/adapter")
    return 0


if __name__ == "__main__":
    sys.exit(main())
