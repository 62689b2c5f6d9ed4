"""Model definitions (the reference has none of its own; it patches HF models)."""
from .decoder import (CausalLM, CausalLMOutput, DecoderLayer, FusedLinear, LlamaForCausalLM, Qwen2ForCausalLM,
                      RMSNorm, build_model)

__all__ = ["CausalLM", "CausalLMOutput", "DecoderLayer", "FusedLinear", "LlamaForCausalLM", "Qwen2ForCausalLM",
           "RMSNorm", "build_model"]
