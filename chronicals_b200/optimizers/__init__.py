from .fused_adamw import FusedAdamW, FusedAdamWFP8
from .lora_plus_optimizer import (LoRAPlusAdamW, LoRAPlusOptimizer, LoRAPlusParameterGroups, create_lora_plus_optimizer,
                                  get_lora_plus_param_groups, wrap_optimizer_with_lora_plus)
from .optimizers import (Adam8bit, AdamAtan2, HybridMuonAdamW, Muon, OneCycleLR, ScheduleFreeAdamW, WSDScheduler,
                         WarmupCosineScheduler, create_optimizer, create_scheduler, newton_schulz_orthogonalize)
from .optimizers_8bit import AdamW8bit, PagedAdamW, create_8bit_optimizer

__all__ = ["FusedAdamW", "FusedAdamWFP8", "LoRAPlusAdamW", "LoRAPlusOptimizer", "LoRAPlusParameterGroups",
           "create_lora_plus_optimizer", "get_lora_plus_param_groups", "wrap_optimizer_with_lora_plus", "Adam8bit",
           "AdamAtan2", "HybridMuonAdamW", "Muon", "OneCycleLR", "ScheduleFreeAdamW", "WSDScheduler",
           "WarmupCosineScheduler", "create_optimizer", "create_scheduler", "newton_schulz_orthogonalize", "AdamW8bit",
           "PagedAdamW", "create_8bit_optimizer"]
