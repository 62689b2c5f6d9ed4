"""Public names of the reference's modules resolve here (same module paths under ``chronicals_b200`` and
under the ``chronicals`` alias)."""
import importlib

import pytest

INVENTORY = {
    "config.config": ["ChronicalsConfig", "TrainingConfig", "BenchmarkConfig", "MODEL_REGISTRY", "DATASET_REGISTRY",
                      "get_model_config", "get_optimal_config_for_gpu", "Qwen05BOptimalConfig", "ROOFLINE_ANALYSIS",
                      "BenchmarkOptimizedConfig", "get_benchmark_config", "HF_READ_TOKEN", "HF_WRITE_TOKEN"],
    "config.sota_config": ["TheoreticalPerformance", "OPTIMIZATION_SYNERGY", "MaxPerformanceConfig", "OptimizationStatus",
                           "OptimizationChecklist", "print_diagnostic_report", "IntegrationTestConfig",
                           "BENCHMARK_COMPARISON", "get_sota_config_for_gpu", "UNSLOTH_BENCHMARKS",
                           "print_comprehensive_diagnostic", "verify_optimization_synergy", "print_synergy_report"],
    "kernels.triton_kernels": ["fused_cross_entropy_triton", "rmsnorm_forward", "rmsnorm_backward", "LigerRMSNormFunction",
                               "rmsnorm_triton", "rmsnorm_with_grad", "FusedRMSNorm", "swiglu_forward", "swiglu_backward",
                               "LigerSwiGLUFunction", "fused_swiglu_triton", "FusedSwiGLU", "FusedSiLUMul", "geglu_forward",
                               "geglu_backward", "LigerGeGLUFunction", "FusedGeGLU", "fused_geglu", "fused_qk_rope_inplace",
                               "FusedQKRoPEFunction", "fused_qk_rope", "fused_rope", "fused_cross_entropy", "rmsnorm",
                               "fused_swiglu", "precompute_rope_cache", "DEFAULT_CHUNK_SIZE",
                               "fused_linear_cross_entropy_forward", "fused_linear_cross_entropy",
                               "FusedLinearCrossEntropyFunction", "chunked_cross_entropy", "FusedLinearCrossEntropyLoss",
                               "ChunkedCrossEntropyLoss", "liger_cross_entropy_forward", "LigerCrossEntropyFunction",
                               "liger_cross_entropy", "triton_fused_linear_cross_entropy_forward",
                               "TritonFusedLinearCrossEntropyFunction", "triton_fused_linear_cross_entropy",
                               "TritonFusedLinearCrossEntropyLoss", "LigerFusedLinearCrossEntropyLoss", "fused_rmsnorm_linear",
                               "FusedRMSNormLinear", "fused_embedding_rope", "FusedEmbeddingRoPE", "fused_gqa_attention"],
    "kernels.cut_cross_entropy": ["get_optimal_chunk_size", "CutCrossEntropyForward", "CutCrossEntropyBackward",
                                  "CutCrossEntropyFunction", "TritonCCEFunction", "cut_cross_entropy", "CutCrossEntropyLoss"],
    "kernels.fused_qk_rope": ["fused_qk_rope_forward", "FusedQKRoPEFunction", "fused_qk_rope", "fused_qkv_rope_inplace",
                              "precompute_rope_cache", "FusedQKRoPE", "apply_rope"],
    "kernels.fused_rope": ["FusedQKRoPEFunction", "fused_qk_rope", "precompute_rope_cache", "FusedRotaryEmbedding",
                           "benchmark_rope"],
    "kernels.fused_lora_kernels": ["fused_lora_down_dropout", "fused_lora_linear", "FusedLoRALinearFunction", "FusedLoRALinear",
                                   "FusedLoRAAdapter", "apply_lora_to_model", "get_lora_params", "count_lora_params",
                                   "benchmark_lora"],
    "kernels.flash_attention_optimizer": ["get_flash_attn_info", "GPU_SPECS", "FlashAttentionConfig", "get_gpu_specs",
                                          "create_cu_seqlens", "create_cu_seqlens_from_attention_mask",
                                          "create_cu_seqlens_from_position_ids", "is_packed_sequence",
                                          "unpack_sequence_to_padded", "pack_padded_to_varlen",
                                          "create_position_ids_for_packed", "flash_attn_varlen_wrapper",
                                          "FP8BlockQuantConfig", "quantize_to_fp8_block", "dequantize_from_fp8_block",
                                          "patch_model"],
    "kernels": ["fused_rmsnorm", "fused_swiglu", "fused_cross_entropy", "fused_qk_rope"],
    "optimizers.fused_adamw": ["FusedAdamW", "FusedAdamWFP8", "benchmark_optimizer"],
    "optimizers.lora_plus_optimizer": ["LoRAPlusParameterGroups", "LoRAPlusAdamW", "LoRAPlusOptimizer",
                                       "create_lora_plus_optimizer", "get_lora_plus_param_groups",
                                       "wrap_optimizer_with_lora_plus"],
    "optimizers.optimizers": ["ScheduleFreeAdamW", "Muon", "Adam8bit", "AdamAtan2", "HybridMuonAdamW", "WSDScheduler",
                              "OneCycleLR", "create_optimizer", "create_scheduler"],
    "optimizers.optimizers_8bit": ["get_bnb_info", "AdamW8bit", "Adam8bit", "PagedAdamW", "OptimizerStateConverter",
                                   "HybridPrecisionOptimizer", "create_8bit_optimizer"],
    "optimizers": ["FusedAdamW", "create_lora_plus_optimizer", "Adam8bit", "LoRAPlusAdamW", "LoRAPlusOptimizer",
                   "LoRAPlusParameterGroups"],
    "lora.lora_optimized": ["OptimizedLoRALinear", "LoRAModel", "apply_lora_to_model", "get_lora_optimizer_groups",
                            "benchmark_bracketing"],
    "lora.dora_adapter": ["DoRALinear", "DoRAModel", "apply_dora_to_model", "convert_lora_to_dora",
                          "get_dora_plus_param_groups"],
    "lora.gradient_checkpointing_lora": ["LoRAGradientCheckpointer", "LoRACheckpointConfig", "UnslothCheckpointing",
                                         "apply_lora_checkpointing", "estimate_checkpointing_savings"],
    "lora.lora_presets": ["GPUType", "GPUSpec", "GPU_SPECS", "detect_gpu", "detect_hardware", "LoRAPreset", "PRESET_REGISTRY",
                          "get_model_size", "get_preset_for_hardware", "get_optimal_preset",
                          "get_optimization_recommendations", "compare_presets", "list_all_presets"],
    "lora": ["LoRAConfig", "apply_lora"],
    "data.sequence_packer": ["PackedBatch", "BinPackingAlgorithm", "Bin", "FixedShapeSequencePacker", "SequencePacker",
                             "create_cu_seqlens", "create_cu_seqlens_from_position_ids", "apply_flash_attention_varlen",
                             "DataPrefetcher", "DoubleBufferPrefetcher", "PackedDataset", "PackedDataLoader",
                             "compute_padding_free_loss", "compute_tokens_per_second", "DynamicBatchSizeAdjuster",
                             "analyze_dataset_for_packing"],
    "data.sequence_packer_v2": ["PackedBatchV2", "compute_cu_seqlens", "cu_seqlens_to_sequence_lengths",
                                "compute_cu_seqlens_from_position_ids", "is_packed_sequence", "flash_attention_varlen",
                                "SequencePackerV2", "create_block_causal_mask", "create_4d_attention_mask",
                                "compute_packed_loss", "compute_packing_statistics"],
    "data.data_loader": ["DataCollator", "DataCollatorWithFlattening", "PackingDataCollator", "InstructionDataset",
                         "StreamingInstructionDataset", "LengthAwareSampler", "CurriculumSampler", "load_dataset_hf",
                         "load_alpaca", "load_dolly", "load_slimorca", "create_dataloader", "create_packed_dataloader",
                         "get_tokenizer", "analyze_dataset", "estimate_training_throughput", "ChronicalsDataPipeline",
                         "create_optimized_dataloader"],
    "data": ["SequencePacker", "PackedBatch", "DataPrefetcher", "create_dataloader"],
    "training.chronicals_trainer": ["ChronicalsTrainer", "TrainerState", "print_chronicals_banner",
                                    "setup_torch_compile_for_training"],
    "training.gradient_checkpointing": ["GradientCheckpointer", "CheckpointedLayer", "SelectiveCheckpointing",
                                        "apply_gradient_checkpointing", "estimate_activation_memory"],
    "training.cuda_graph_manager": ["CUDAGraphConfig", "GraphStatistics", "CUDAGraphMemoryPool", "CapturedGraph",
                                    "CUDAGraphManager", "create_cuda_graph_training_step", "cuda_graph_capture"],
    "training.async_activation_offload": ["OffloadConfig", "OffloadStats", "CUDAStreamManager", "PinnedMemoryPool",
                                          "ActivationOffloadManager", "OffloadActivations", "CheckpointWithOffload",
                                          "estimate_offload_bandwidth", "estimate_activation_memory",
                                          "create_offload_manager"],
    "training": ["ChronicalsTrainer", "apply_gradient_checkpointing", "enable_gradient_checkpointing", "enable_cuda_graphs"],
    "utils.fp8_utils": ["FP8Format", "FP8Handler", "FP8Linear", "compute_fp8_memory_savings"],
    "utils.fp8_deepseek": ["FP8Spec", "FP8GradScaler", "FP8GradientAccumulator", "quantize_block_e4m3", "quantize_block_e5m2",
                           "dequantize_block", "AmaxHistory", "FP8LinearFunction", "FP8Linear", "DEFAULT_FP8_EXCLUDE_PATTERNS",
                           "should_convert_to_fp8", "convert_linear_to_fp8", "convert_model_to_fp8", "FP8Context",
                           "compute_fp8_memory_savings", "apply_fp8_to_huggingface_model", "FP8AttentionConfig",
                           "prepare_fp8_attention_inputs", "fp8_flash_attention_forward"],
    "utils.profiling_utils": ["GPU_SPECS", "detect_gpu_specs", "TimingBreakdown", "MemorySnapshot", "PerformanceMetrics",
                              "MFUTracker", "ThroughputMonitor", "PerformanceProfiler", "MixedPrecisionManager",
                              "generate_performance_report", "print_performance_report"],
    "utils.compile_utils": ["get_compile_info", "CompileConfig", "GraphBreakPrevention", "LoRAHotswapManager",
                            "CompiledLoRAModel", "compile_model_with_lora", "get_optimal_compile_mode"],
    "utils.visual_reporter": ["TrainingMetrics", "VisualReporter", "create_progress_bar"],
    "": ["ChronicalsTrainer", "ChronicalsConfig", "LoRAPlusOptimizer", "SequencePacker", "get_version", "get_device_info",
         "print_info"],
}


# names added after the first inventory pass (same modules as above)
INVENTORY_ADDED = {
    "kernels.flash_attention_optimizer": ["get_hadamard_matrix", "apply_hadamard_transform",
                                          "apply_inverse_hadamard_transform", "get_fp8_max", "compute_arithmetic_intensity",
                                          "estimate_tokens_per_second", "FlashAttnVarlenOutput", "OptimizationResult"],
    "kernels.fused_rope": ["fused_qk_rope_inplace", "fused_qk_rope_inplace_backward", "precompute_rope_cache_extended"],
    "kernels.fused_kernels": ["swiglu_with_grad", "fused_cross_entropy_pytorch", "fused_swiglu_pytorch",
                              "fused_rope_pytorch", "liger_cross_entropy_backward"],
    "kernels.triton_kernels": ["swiglu_with_grad", "fused_cross_entropy_pytorch", "liger_cross_entropy_backward"],
    "kernels.fused_lora_kernels": ["fused_lora_linear_with_grad"],
    "lora.gradient_checkpointing_lora": ["SelectiveCheckpoint"],
}


def _missing(root: str):
    out = []
    for mod, names in list(INVENTORY.items()) + list(INVENTORY_ADDED.items()):
        m = importlib.import_module(root + ("." + mod if mod else ""))
        out += [f"{mod}.{n}" for n in names if not hasattr(m, n)]
    return out


@pytest.mark.parametrize("root", ["chronicals_b200", "chronicals"])
def test_reference_public_names_resolve(root):
    missing = _missing(root)
    assert not missing, f"{len(missing)} names missing: {missing}"


def test_functional_forward_backward_pairs_match_autograd():
    import torch
    import importlib
    cce = importlib.import_module("chronicals_b200.kernels.cut_cross_entropy")
    fk = importlib.import_module("chronicals_b200.kernels.fused_kernels")
    flk = importlib.import_module("chronicals_b200.kernels.fused_lora_kernels")
    torch.manual_seed(0)
    x = torch.randn(6, 32, requires_grad=True)
    w = torch.randn(32).abs().requires_grad_(True)
    y, rstd = fk.rmsnorm_forward(x, w)
    dy = torch.randn_like(y)
    dx, dw = fk.rmsnorm_backward(dy, x, w, rstd)
    ref = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)) * w
    gx, gw = torch.autograd.grad(ref, (x, w), dy)
    assert torch.allclose(y, ref, atol=1e-5) and torch.allclose(dx, gx, atol=1e-5) and torch.allclose(dw, gw, atol=1e-4)
    assert torch.allclose(fk.LigerRMSNormFunction.apply(x, w, 1e-6), ref, atol=1e-5)

    g, u = torch.randn(4, 16, requires_grad=True), torch.randn(4, 16, requires_grad=True)
    out = fk.LigerSwiGLUFunction.apply(g, u)
    want = torch.nn.functional.silu(g) * u
    assert torch.allclose(out, want, atol=1e-6)
    dg, du = fk.swiglu_backward(torch.ones_like(out), g, u)
    wg, wu = torch.autograd.grad(want.sum(), (g, u))
    assert torch.allclose(dg, wg, atol=1e-5) and torch.allclose(du, wu, atol=1e-5)
    assert torch.allclose(fk.LigerGeGLUFunction.apply(g, u), torch.nn.functional.gelu(g, approximate="tanh") * u, atol=1e-5)

    q, k = torch.randn(2, 8, 4, 16, requires_grad=True), torch.randn(2, 8, 2, 16, requires_grad=True)
    cos, sin = fk.precompute_rope_cache(8, 16)
    qr, kr = fk.FusedQKRoPEFunction.apply(q, k, cos, sin)
    q2, k2 = fk.fused_qk_rope(q, k, cos, sin)
    assert torch.allclose(qr, q2) and torch.allclose(kr, k2)
    (gq,) = torch.autograd.grad(qr.sum() + kr.sum(), (q,), retain_graph=True)
    (gq2,) = torch.autograd.grad(q2.sum() + k2.sum(), (q,))
    assert torch.allclose(gq, gq2, atol=1e-5)

    h = torch.randn(10, 24, requires_grad=True)
    W = (0.1 * torch.randn(50, 24)).requires_grad_(True)
    lab = torch.randint(0, 50, (10,))
    lab[3] = -100
    loss = cce.CutCrossEntropyFunction.apply(h, W, lab)
    want = torch.nn.functional.cross_entropy(h @ W.t(), lab, ignore_index=-100)
    assert abs(float(loss) - float(want)) < 1e-5
    gh, gW = torch.autograd.grad(loss, (h, W))
    wh, wW = torch.autograd.grad(want, (h, W))
    assert torch.allclose(gh, wh, atol=1e-5) and torch.allclose(gW, wW, atol=1e-5)
    l2, lse, tgt, valid = cce.CutCrossEntropyForward.forward(h, W, lab)
    assert torch.allclose(lse[valid], torch.logsumexp(h @ W.t(), -1)[valid].detach(), atol=1e-4)
    l3, z, g_h, g_w = fk.fused_linear_cross_entropy_forward(h, W, lab)
    assert torch.allclose(g_h, wh, atol=1e-5) and abs(float(l3) - float(want)) < 1e-5
    l4 = fk.LigerCrossEntropyFunction.apply((h @ W.t()).detach().requires_grad_(True), lab)
    assert abs(float(l4) - float(want)) < 1e-5

    xx = torch.randn(5, 24, requires_grad=True)
    A = torch.randn(4, 24, requires_grad=True)
    B = torch.randn(50, 4, requires_grad=True)
    yy = flk.FusedLoRALinearFunction.apply(xx, W.detach(), A, B, None, 0.5)
    want = xx @ W.detach().t() + 0.5 * (xx @ A.t()) @ B.t()
    assert torch.allclose(yy, want, atol=1e-4)
    g1 = torch.autograd.grad(yy.sum(), (xx, A, B))
    g2 = torch.autograd.grad(want.sum(), (xx, A, B))
    assert all(torch.allclose(a, b, atol=1e-3) for a, b in zip(g1, g2))


def test_alias_package_shares_module_objects():
    import chronicals.config.config as a
    import chronicals_b200.config.config as b
    from chronicals_b200.models import decoder
    assert a is b and a.ChronicalsConfig is decoder.ChronicalsConfig
