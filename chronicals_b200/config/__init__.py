from .config import (BenchmarkConfig, BenchmarkOptimizedConfig, ChronicalsConfig, DATASET_REGISTRY, HF_READ_TOKEN,
                     HF_WRITE_TOKEN, MODEL_REGISTRY, ParallelConfig, Qwen05BOptimalConfig, ROOFLINE_ANALYSIS,
                     TrainingConfig, get_benchmark_config, get_model_config, get_optimal_config_for_gpu,
                     measured_peaks, roofline_analysis)

__all__ = ["BenchmarkConfig", "BenchmarkOptimizedConfig", "ChronicalsConfig", "DATASET_REGISTRY", "HF_READ_TOKEN",
           "HF_WRITE_TOKEN", "MODEL_REGISTRY", "ParallelConfig", "Qwen05BOptimalConfig", "ROOFLINE_ANALYSIS",
           "TrainingConfig", "get_benchmark_config", "get_model_config", "get_optimal_config_for_gpu",
           "measured_peaks", "roofline_analysis"]
