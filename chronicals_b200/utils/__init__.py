"""Utilities: FP8, profiling, reporting, adapter hot-swap (imported lazily by name)."""
import importlib

_MODULES = ("compile_utils", "profiling_utils", "visual_reporter", "fp8_utils", "fp8_deepseek", "native")


def __getattr__(name):
    if name in _MODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
