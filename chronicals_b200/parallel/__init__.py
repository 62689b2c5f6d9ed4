"""Multi-GPU support (absent from the reference): bootstrap, data-parallel reduction, peer-memory
collectives, sharded optimizer, tensor/sequence parallel layers, host-side failure detection."""
from .bootstrap import env_world, init_distributed, is_main, max_over_ranks, shutdown

__all__ = ["env_world", "init_distributed", "is_main", "max_over_ranks", "shutdown"]
