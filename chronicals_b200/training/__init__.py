from .chronicals_trainer import ChronicalsTrainer, TrainerState, print_chronicals_banner
from .gradient_checkpointing import (GradientCheckpointer, apply_gradient_checkpointing, enable_gradient_checkpointing,
                                     estimate_activation_memory)
from .cuda_graph_manager import CUDAGraphManager, enable_cuda_graphs

__all__ = ["ChronicalsTrainer", "TrainerState", "print_chronicals_banner", "GradientCheckpointer",
           "apply_gradient_checkpointing", "enable_gradient_checkpointing", "estimate_activation_memory",
           "CUDAGraphManager", "enable_cuda_graphs"]
