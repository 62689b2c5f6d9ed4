"""Import-path alias: the reference keeps its fused ops in ``chronicals.kernels.triton_kernels``.
This framework has no Triton; the same names live in ``fused_kernels`` and are re-exported here."""
from .fused_kernels import *  # noqa: F401,F403
from .fused_kernels import __all__  # noqa: F401
