from .dora_adapter import DoRALinear, DoRAModel, apply_dora_to_model, convert_lora_to_dora, get_dora_plus_param_groups
from .gradient_checkpointing_lora import (LoRACheckpointConfig, LoRAGradientCheckpointer, UnslothCheckpointing,
                                          apply_lora_checkpointing, estimate_checkpointing_savings)
from .lora_optimized import (LoRAConfig, LoRAModel, OptimizedLoRALinear, apply_lora, apply_lora_to_model,
                             count_lora_params, get_lora_optimizer_groups, get_lora_parameters)
from .lora_presets import (GPUType, LoRAPreset, detect_gpu, get_optimal_preset, get_preset_for_hardware,
                           list_all_presets)

__all__ = ["DoRALinear", "DoRAModel", "apply_dora_to_model", "convert_lora_to_dora", "get_dora_plus_param_groups",
           "LoRACheckpointConfig", "LoRAGradientCheckpointer", "UnslothCheckpointing", "apply_lora_checkpointing",
           "estimate_checkpointing_savings", "LoRAConfig", "LoRAModel", "OptimizedLoRALinear", "apply_lora",
           "apply_lora_to_model", "count_lora_params", "get_lora_optimizer_groups", "get_lora_parameters", "GPUType",
           "LoRAPreset", "detect_gpu", "get_optimal_preset", "get_preset_for_hardware", "list_all_presets"]
