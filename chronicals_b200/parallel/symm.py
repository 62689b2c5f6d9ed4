"""Symmetric (peer-mapped) device buffers and the collectives built on them.

Every rank allocates a buffer of the same size, exports it as a CUDA IPC handle, and maps all
peers' buffers into its own address space, giving each rank a table of W device pointers per
buffer.  Kernels in ``csrc/comm.cu`` then move data with ordinary loads and stores on those
pointers — NVLink 5 through NVSwitch gives every GPU a direct path to every peer's HBM — and
synchronise through epoch flags in a small per-rank flag pad.  NCCL is only used once, at set-up,
to exchange the handles.

The reference has no multi-GPU code; nothing here has a counterpart there.

Safety: every device-side wait is bounded (``wait_budget_us``); when it expires the kernel records
an error in the status word and returns, and :func:`chronicals_b200.ops._ext.check_status` raises
on the host.  Epochs only ever increase, so a stale flag can never satisfy a later barrier.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext

_P, _I, _L, _F, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_ulonglong
_PROTOS = {
    "cb_comm_max_ranks": [], "cb_comm_pad_bytes": [], "cb_comm_payload_floats": [], "cb_comm_grid": [],
    "cb_symm_barrier": [_P, _I, _I, _P, _P, _P, _U, _P, _P],
    "cb_rs_reduce_sqnorm": [_P, _I, _L, _L, _P, _P, _P, _P, _P],
    "cb_adamw_shard_allgather": [_P, _I, _I, _L, _L, _P, _P, _P, _P, _P, _P, _P, _F, _P, _P, _P],
    "cb_allreduce_pull": [_P, _I, _L, _F, _P, _P, _P],
}
_BOUND = False


def _lib():
    global _BOUND
    lib = _ext.lib()
    if not _BOUND:
        for name, args in _PROTOS.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int
        _BOUND = True
    return lib


_PEER_ENABLED = set()


def enable_peer_access(my_device: int, peer_device: int) -> None:
    """Let kernels running on ``my_device`` dereference pointers into ``peer_device``'s memory."""
    if my_device == peer_device or (my_device, peer_device) in _PEER_ENABLED:
        return
    lib = _lib()
    fn = lib.cb_enable_peer_access
    fn.argtypes = [_I, _I]
    fn.restype = ctypes.c_int
    code = fn(my_device, peer_device)
    if code != 0:
        raise RuntimeError(f"cudaDeviceEnablePeerAccess({my_device} -> {peer_device}) failed with CUDA error {code}")
    _PEER_ENABLED.add((my_device, peer_device))


def peer_access_available(group=None) -> bool:
    """True when every pair of local GPUs can address each other's memory."""
    if not torch.cuda.is_available():
        return False
    n = torch.cuda.device_count()
    me = torch.cuda.current_device()
    return all(torch.cuda.can_device_access_peer(me, j) for j in range(n) if j != me)


class _DeviceBlock:
    """A cudaMalloc block exposed through ``__cuda_array_interface__`` so torch can alias it."""

    def __init__(self, ptr: int, nbytes: int, owner: bool):
        self.ptr, self.nbytes, self.owner = ptr, nbytes, owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}

    def release(self) -> None:
        if self.ptr:
            lib = _lib()
            (lib.cb_symm_free if self.owner else lib.cb_ipc_close)(ctypes.c_void_p(self.ptr))
            self.ptr = 0


def _bind_ipc(lib) -> None:
    lib.cb_symm_alloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_ulonglong]
    lib.cb_symm_free.argtypes = [ctypes.c_void_p]
    lib.cb_ipc_export.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    lib.cb_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.cb_ipc_close.argtypes = [ctypes.c_void_p]
    for n in ("cb_symm_alloc", "cb_symm_free", "cb_ipc_export", "cb_ipc_open", "cb_ipc_close"):
        getattr(lib, n).restype = ctypes.c_int


class SymmetricBuffer:
    """A tensor present on every rank, with all peers' copies mapped locally.

    ``local`` is this rank's tensor; ``ptrs`` a host array of the W device pointers for kernel
    launches (``ptrs[rank] == local.data_ptr()``).  The block comes from ``cudaMalloc`` directly, is
    exported as a CUDA IPC handle and opened by each peer on its own device with lazy peer access,
    so every mapping lives in the opening rank's context.  Peer memory is only ever touched by the
    kernels of ``csrc/comm.cu`` through ``ptrs``; it is never handed to a library kernel.
    """

    def __init__(self, numel: int, dtype: torch.dtype, group=None, zero: bool = True):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("SymmetricBuffer needs an initialised process group")
        lib = _lib()
        _bind_ipc(lib)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        esz = torch.empty((), dtype=dtype).element_size()
        used = numel * esz
        nbytes = max(2 << 20, (used + (2 << 20) - 1) // (2 << 20) * (2 << 20))
        torch.cuda.synchronize(dev)
        with torch.cuda.device(dev):
            out = ctypes.c_void_p()
            code = lib.cb_symm_alloc(ctypes.byref(out), nbytes)        # zero-filled
            if code != 0:
                raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed with CUDA error {code}")
            self._block = _DeviceBlock(out.value, nbytes, True)
            raw = torch.as_tensor(self._block, device=dev)
            self.local = raw[:used].view(dtype)
            # canary words behind the payload: a peer kernel that writes past the end of this buffer
            # shows up in canary_ok() (checked on the host, between steps)
            guard_at = (used + 255) // 256 * 256
            self._guard = raw[guard_at:guard_at + 256] if guard_at + 256 <= nbytes else None
            if self._guard is not None:
                self._guard.fill_(0xA5)
            handle = ctypes.create_string_buffer(64)
            code = lib.cb_ipc_export(ctypes.c_void_p(self._block.ptr), handle)
            if code != 0:
                raise RuntimeError(f"cudaIpcGetMemHandle failed with CUDA error {code}")
            gathered: List[object] = [None] * self.world
            dist.all_gather_object(gathered, handle.raw, group=group)
            self._peer_blocks: List[_DeviceBlock] = []
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(self._block.ptr)
                    continue
                p = ctypes.c_void_p()
                code = lib.cb_ipc_open(gathered[r], ctypes.byref(p))
                if code != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r}'s buffer failed with CUDA error {code}")
                self._peer_blocks.append(_DeviceBlock(p.value, nbytes, False))
                ptrs.append(p.value)
        self.ptrs = (ctypes.c_ulonglong * self.world)(*ptrs)
        dist.barrier(group=group)

    def canary_ok(self) -> bool:
        """True while the 256 guard bytes behind the payload still hold their pattern (host-side check)."""
        return self._guard is None or bool((self._guard == 0xA5).all().item())

    def close(self) -> None:
        """Unmap the peers' blocks and free the local one (after a barrier, so nobody still reads it)."""
        if getattr(self, "_block", None) is None:
            return
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for b in self._peer_blocks:
            b.release()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        self.local = None
        self._block.release()
        self._block = None


class SymmetricContext:
    """Flag pad + barrier shared by all symmetric collectives of one process group."""

    def __init__(self, group=None, wait_budget_us: int = 2_000_000):
        lib = _lib()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > lib.cb_comm_max_ranks():
            raise ValueError(f"at most {lib.cb_comm_max_ranks()} ranks per symmetric group")
        self.pad = SymmetricBuffer(lib.cb_comm_pad_bytes(), torch.uint8, group, zero=True)
        self.payload_floats = lib.cb_comm_payload_floats()
        self.epoch_ctr = torch.zeros(1, dtype=torch.int64, device=self.pad.local.device)   # advanced on the device
        self.wait_ns = int(wait_budget_us) * 1000
        dev = self.pad.local.device
        self.gathered = torch.zeros(self.world * self.payload_floats, dtype=torch.float32, device=dev)
        self.status = _ext.status_buffer(dev)
        self.grid = lib.cb_comm_grid()

    def barrier(self, payload: Optional[torch.Tensor] = None, gather: bool = False) -> Optional[torch.Tensor]:
        """All-rank barrier on the current stream (a kernel, not a host wait).  With ``payload``
        (4 floats on the device) every rank receives all ranks' payloads in ``self.gathered``."""
        code = _lib().cb_symm_barrier(self.pad.ptrs, self.rank, self.world, self.epoch_ctr.data_ptr(), _ext.ptr(payload),
                                      self.gathered.data_ptr() if (gather or payload is not None) else None,
                                      self.wait_ns, self.status.data_ptr(), _ext.stream_ptr())
        _ext.check(code, "symm_barrier")
        return self.gathered if (gather or payload is not None) else None


class FusedAllReduce:
    """Bucket all-reduce by peer loads (``allreduce_pull_kernel``): every rank reads all W copies of
    the bucket and writes the average locally.  Used by ``GradientReducer(backend="fused")`` for
    small buckets (adapter gradients); large buckets go through the sharded optimizer instead."""

    def __init__(self, buckets, group=None, wait_budget_us: int = 2_000_000):
        if not peer_access_available(group):
            raise RuntimeError("peer access between the local GPUs is not available")
        self.ctx = SymmetricContext(group, wait_budget_us)
        self.world = self.ctx.world
        self.bufs = {}
        for b in buckets:
            if b.flat.dtype != torch.bfloat16 or b.flat.numel() % 8 != 0:
                raise RuntimeError("fused all-reduce handles bf16 buckets whose size is a multiple of 8")
            sb = SymmetricBuffer(b.flat.numel(), torch.bfloat16, group)
            self.bufs[id(b)] = sb

    def all_reduce(self, bucket) -> None:
        sb = self.bufs[id(bucket)]
        sb.local.copy_(bucket.flat)
        self.ctx.barrier()                      # every rank's copy is in place
        code = _lib().cb_allreduce_pull(sb.ptrs, self.world, bucket.flat.numel(), 1.0 / self.world,
                                        bucket.flat.data_ptr(), self.ctx.status.data_ptr(), _ext.stream_ptr())
        _ext.check(code, "allreduce_pull")
        self.ctx.barrier()                      # nobody overwrites its copy while a peer still reads it
