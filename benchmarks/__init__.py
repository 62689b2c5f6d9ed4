"""Benchmark scripts (``python -m benchmarks.run_benchmark`` or run the files directly)."""
