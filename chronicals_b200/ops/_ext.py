"""ctypes binding of the in-tree CUDA kernel library.

The kernels expose a plain C ABI (raw device pointers + a stream handle) so the
library builds with nothing but ``nvcc`` and loads without a C++ binding layer.
On a machine with a GPU the library is required: ``lib()`` raises instead of
letting callers fall back silently to PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LOCK = threading.Lock()
_STATUS = {}

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "_cb_kernels.so")

P = c_void_p
I = c_int
L = c_longlong
F = c_float

_PROTOTYPES = {
    "cb_gemm_bf16": [P, P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, I, P, P],
    "cb_cce_num_splits": [I, I],
    "cb_cce_forward": [P, P, P, I, I, I, L, L, I, P, P, P, P, P, P],
    "cb_cce_combine": [P, P, P, P, P, I, I, I, F, F, L, I, P, P, P, P, P],
    "cb_cce_dlogits": [P, P, P, P, P, P, P, I, I, I, L, L, L, I, I, F, F, P, P],
    "cb_rmsnorm_max_n": [],
    "cb_rmsnorm_bwd_blocks": [I, I],
    "cb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, F, P],
    "cb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, F, I, P],
    "cb_colsum_blocks": [L],
    "cb_colsum_bf16": [P, P, P, L, I, L, P],
    "cb_glu_fwd": [P, P, P, L, I, L, L, I, P],
    "cb_glu_bwd": [P, P, P, P, P, L, I, L, L, L, I, P],
    "cb_qk_rope": [P, P, P, P, P, L, I, I, I, L, L, I, I, L, P],
    "cb_debug_word": [P],
    "cb_embedding_fwd": [P, P, P, L, I, L, P],
    "cb_embedding_bwd": [P, P, P, P, L, I, L, I, P],
    "cb_ce_logits": [P, P, L, L, I, I, L, F, F, P, P, P],
    "cb_ce_logits_grad": [P, P, P, P, P, P, L, L, I, I, L, F, F, P],
    "cb_attn_fwd": [P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, F, P, P],
    "cb_attn_bwd": [P, P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, F, P, P, P, P, P, L, P, P, I],
    "cb_gemm2sm_bf16": [P, P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, P, P],
    "cb_gemm2sm_supported": [P, L, I],
    "cb_gemm2sm_bf16_ex": [P, P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, I, P, P],
    "cb_gemm2sm_cost_milli": [I, I, I, I],
    "cb_gemm2sm_bf16_dual": [P, P, P, P, P, P, P, I, I, I, I, L, L, L, L, L, L, I, P, P],
    "cb_gemm2sm_bf16_glu": [P, P, P, P, P, I, I, I, L, L, L, L, P, P],
    "cb_lora_pack": [P, P, P, P, P, P, I, I, I, P, P, P],
    "cb_lora_unpack": [P, P, P, P, I, I, I, P, P, P, P],
    "cb_gemm2sm_fp8": [P, P, P, P, P, P, I, I, I, L, L, L, P, P],
    "cb_rowquant_e4m3": [P, P, P, L, I, L, L, P],
    "cb_gemm_bf16_splitk": [P, P, P, I, I, I, L, L, L, I, I, P, P],
    "cb_adamw8bit": [P, P, P, P, P, P, L, I, F, F, F, F, F, F, F, P],
    "cb_opt_chunk": [],
    "cb_adamw_multi": [P, P, P, P, P, P, P, P, I, I, P, P, I, P],
    "cb_grad_clip_coef": [P, P, P, I, I, P, P, F, P, I, P],
}


def available() -> bool:
    return os.path.exists(LIB_PATH)


_FORCE_REFERENCE = False


class force_reference:
    """Context manager that routes every op in ``chronicals_b200.ops`` through its plain-PyTorch
    formula (the test oracle), also on CUDA.  Used to time or compare the library-only execution of
    the same model; never enabled by default."""

    def __enter__(self):
        global _FORCE_REFERENCE
        self._prev = _FORCE_REFERENCE
        _FORCE_REFERENCE = True
        return self

    def __exit__(self, *exc):
        global _FORCE_REFERENCE
        _FORCE_REFERENCE = self._prev
        return False


def debug_word():
    """``(compiled_with_checks, code, value)`` of the optional index checks (``CHRONICALS_DEBUG_BOUNDS=1`` build):
    code 401 = token id, 402 = rotary position, 403 = label out of range; reading clears the word."""
    buf = (ctypes.c_longlong * 2)()
    rc = lib().cb_debug_word(buf)
    code, value = int(buf[0]), int(buf[1])
    if code == 0:
        # checks of the kernels that carry the status words (GEMM epilogues, attention, collectives: codes 411-431)
        # leave their finding in status[8:10] of the device they ran on
        for st in _STATUS.values():
            vals = st[8:10].tolist()
            if vals[0] != 0:
                code, value = int(vals[0]), int(vals[1])
                st[8:10].zero_()
                break
    return rc == 1, code, value


def reference_forced() -> bool:
    return _FORCE_REFERENCE


def lib() -> ctypes.CDLL:
    """The loaded kernel library; builds it first when the sources are newer."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        from ..csrc import build as _build
        if not _build.is_current():
            _build.build()
        handle = ctypes.CDLL(LIB_PATH)
        proxy = _Library(handle)
        for name, argtypes in _PROTOTYPES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue
            fn.argtypes = argtypes
            fn.restype = c_int
            n = _KERNELS_PER_CALL.get(name, 1)
            setattr(proxy, name, _Counted(fn, n) if n else fn)
        _LIB = proxy
    return _LIB


# device kernels launched by one call of each entry point (0: host-only query)
_KERNELS_PER_CALL = {"cb_gemm2sm_supported": 0, "cb_gemm2sm_cost_milli": 0, "cb_cce_num_splits": 0, "cb_rmsnorm_max_n": 0, "cb_rmsnorm_bwd_blocks": 0, "cb_opt_chunk": 0,
                     "cb_cce_combine": 2, "cb_rmsnorm_bwd": 2, "cb_grad_clip_coef": 2, "cb_attn_bwd": 3}
LAUNCH_COUNT = [0]


class _Counted:
    """Callable wrapper that counts the kernels this process launched through the library."""
    __slots__ = ("fn", "n")

    def __init__(self, fn, n):
        self.fn, self.n = fn, n

    def __call__(self, *args):
        LAUNCH_COUNT[0] += self.n
        return self.fn(*args)


class _Library:
    def __init__(self, handle):
        self._handle = handle

    def __getattr__(self, name):           # symbols without a prototype entry (looked up lazily)
        return getattr(self._handle, name)


def launches() -> int:
    return LAUNCH_COUNT[0]


def count_launch(n: int = 1) -> None:
    """Account for kernels launched through entry points that are bound outside the prototype table."""
    LAUNCH_COUNT[0] += n


def has_symbol(name: str) -> bool:
    return hasattr(lib(), name)


class KernelError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: kernel launch rejected/failed with code {code}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_buffer(device: Optional[torch.device] = None) -> torch.Tensor:
    """Per-device int32[16] status words shared by every kernel that can wait.
    ``status[0] != 0`` after a step means a bounded device-side wait gave up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _STATUS.get(key)
    if buf is None:
        buf = torch.zeros(16, dtype=torch.int32, device=torch.device("cuda", key))
        _STATUS[key] = buf
        _register_gemm_workspace(key)
    return buf


_GEMM_WS = {}


def _register_gemm_workspace(index: int) -> None:
    """Zero-filled scratch for the CTA-pair GEMM's split tiles (fp32 tile slots + arrival counters, about 41 MB per
    GPU), allocated together with the device's status words on first use and kept for the life of the process.
    The kernels leave it zero-filled.  ``CHRONICALS_GEMM_STREAMK=0`` runs whole tiles only."""
    if os.environ.get("CHRONICALS_GEMM_STREAMK", "1") == "0" or not has_symbol("cb_gemm2sm_set_workspace"):
        return
    L_ = lib()
    fn_bytes = L_.cb_gemm2sm_workspace_bytes
    fn_bytes.restype, fn_bytes.argtypes = ctypes.c_ulonglong, []
    fn_set = L_.cb_gemm2sm_set_workspace
    fn_set.restype, fn_set.argtypes = c_int, [c_int, c_void_p, ctypes.c_ulonglong]
    n = int(fn_bytes())
    ws = torch.zeros(n + 1024, dtype=torch.uint8, device=torch.device("cuda", index))
    off = (-ws.data_ptr()) % 1024
    _GEMM_WS[index] = ws
    code = fn_set(index, ws.data_ptr() + off, n)
    if code != 0:
        raise KernelError(f"cb_gemm2sm_set_workspace failed with code {code}")


_STATUS_NAMES = {101: "TMA stage never filled", 102: "smem stage never drained", 103: "accumulator never completed",
                 104: "accumulator never released", 201: "peer flag never arrived", 301: "wait abandoned"}


def check_status(device: Optional[torch.device] = None, reset: bool = True) -> None:
    """Host-side check (synchronises).  Raises ``KernelError`` when a device wait timed out."""
    buf = status_buffer(device)
    vals = buf.tolist()
    if vals[0] != 0:
        if reset:
            buf.zero_()
        raise KernelError(f"device-side wait timed out: code {vals[0]} ({_STATUS_NAMES.get(vals[0], '?')}), "
                          f"block {vals[1]}, thread {vals[2]}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()
