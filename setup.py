"""Packaging for chronicals_b200.

Reference: setup.py:1-115 / pyproject.toml (pure-Python distribution, extras per optional dependency,
console script ``chronicals-bench``).  Here the distribution also carries CUDA and C++ sources; the
``build_kernels`` command (run automatically by ``build_py``) compiles them with nvcc / g++ into
``chronicals_b200/_cb_kernels.so`` and ``chronicals_b200/_cb_host.so`` inside the package, for sm_100a
only.  ``pip install -e .`` followed by ``python -m chronicals_b200.csrc.build`` does the same in place.
"""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class build_kernels(Command):
    description = "compile the sm_100a CUDA kernels and the C++ host helpers in-tree"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        sys.path.insert(0, HERE)
        from chronicals_b200.csrc import build as kernels
        from chronicals_b200.utils import native
        print("built", kernels.build())
        print("built", native.build())


class build_py_with_kernels(build_py):
    def run(self):
        if os.environ.get("CHRONICALS_SKIP_KERNEL_BUILD", "0") != "1":
            self.run_command("build_kernels")
        super().run()


setup(
    name="chronicals-b200",
    version="0.1.0",
    description="Blackwell-native (sm_100a) LLM fine-tuning framework with the Chronicals API",
    packages=find_packages(include=["chronicals_b200", "chronicals_b200.*", "chronicals", "benchmarks", "examples"]),
    package_data={"chronicals_b200": ["_cb_kernels.so", "_cb_host.so", "csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "csrc/host/*.cpp"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy"],
    extras_require={
        "hf": ["transformers>=4.36", "safetensors", "sentencepiece"],
        "data": ["datasets", "pyarrow"],
        "logging": ["tqdm", "rich"],
        "dev": ["pytest", "pytest-timeout", "hypothesis"],
    },
    entry_points={"console_scripts": ["chronicals-bench=benchmarks.run_benchmark:main"]},
    cmdclass={"build_kernels": build_kernels, "build_py": build_py_with_kernels},
)
