from .io import (load_lora_adapter, load_model_weights, load_training_state, prune_checkpoints, read_weights,
                 save_lora_adapter, save_model, save_training_state)

__all__ = ["load_lora_adapter", "load_model_weights", "load_training_state", "prune_checkpoints", "read_weights",
           "save_lora_adapter", "save_model", "save_training_state"]
