"""Import-path alias: code written against ``chronicals`` (the reference's package name) imports this
framework.  ``chronicals.X.Y`` is the same module object as ``chronicals_b200.X.Y``."""
import importlib
import sys

import chronicals_b200 as _impl
from chronicals_b200 import *  # noqa: F401,F403
from chronicals_b200 import __version__, get_device_info, get_version, print_info  # noqa: F401

_SUBPACKAGES = ("config", "training", "data", "optimizers", "lora", "kernels", "utils", "models", "ops", "parallel",
                "checkpoint")


class _AliasFinder:
    """Resolves ``chronicals.<sub>...`` to the already imported ``chronicals_b200.<sub>...`` module."""

    @staticmethod
    def find_spec(fullname, path=None, target=None):
        if not fullname.startswith("chronicals."):
            return None
        real = "chronicals_b200." + fullname[len("chronicals."):]
        try:
            mod = importlib.import_module(real)
        except ImportError:
            return None
        # (sys.modules[fullname] must not be set here: the import system would then take the real module's
        # own spec and execute the real module a second time)
        return importlib.util.spec_from_loader(fullname, loader=_AliasLoader(mod))


class _AliasLoader:
    def __init__(self, mod):
        self.mod = mod

    def create_module(self, spec):
        return self.mod

    def exec_module(self, module):
        pass


import importlib.util  # noqa: E402

if not any(isinstance(f, type) and f.__name__ == "_AliasFinder" for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder)


def __getattr__(name):
    if name in _SUBPACKAGES:
        return importlib.import_module(f"chronicals.{name}")
    return getattr(_impl, name)
