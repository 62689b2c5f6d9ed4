"""C++ host helpers (bin packing, packed-row assembly) behind a ctypes binding.

The sources live in ``csrc/host``; :func:`build` compiles them with ``g++`` into
``chronicals_b200/_cb_host.so`` (in-tree, content-hashed like the kernel library).  The reference
has no native code; its packer is Python (chronicals/data/sequence_packer.py:94-322).  The Python
packer in ``data/sequence_packer.py`` stays the oracle: both produce identical bins.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
from typing import List, Optional, Sequence

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
SRC_DIR = os.path.join(PKG, "csrc", "host")
LIB_PATH = os.path.join(PKG, "_cb_host.so")
HASH_PATH = os.path.join(PKG, "_cb_host.hash")
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=default"]
STRATEGY_IDS = {"ffd": 0, "bfd": 1, "bfd_heap": 2, "spfhp": 3, "greedy": 4}

_LIB: Optional[ctypes.CDLL] = None


def _sources() -> List[str]:
    return sorted(os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR) if f.endswith(".cpp"))


def _hash() -> str:
    h = hashlib.sha256()
    for p in _sources():
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(CXX_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(HASH_PATH)):
        return False
    with open(HASH_PATH) as f:
        return f.read().strip() == _hash()


def build(force: bool = False) -> str:
    if not force and is_current():
        return LIB_PATH
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found for the host helpers")
    r = subprocess.run([cxx, *CXX_FLAGS, *_sources(), "-o", LIB_PATH], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the host helpers failed:\n{r.stderr}")
    with open(HASH_PATH, "w") as f:
        f.write(_hash())
    return LIB_PATH


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not is_current():
            build()
        L = ctypes.CDLL(LIB_PATH)
        pll, ll, pi = ctypes.POINTER(ctypes.c_longlong), ctypes.c_longlong, ctypes.POINTER(ctypes.c_int)
        L.cb_pack_bins.argtypes = [pll, ll, ll, ctypes.c_int, pll, pll]
        L.cb_pack_bins.restype = ll
        L.cb_fill_rows.argtypes = [pll, pll, pll, pll, pll, ll, ll, ll, ll, ctypes.c_int, ll, pll, pll, pll, pll, pi, pi]
        L.cb_fill_rows.restype = ctypes.c_int
        _LIB = L
    return _LIB


def _pll(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))


def native_pack(lengths: Sequence[int], capacity: int, strategy: str = "bfd") -> Optional[List[List[int]]]:
    """Bins (lists of item indices) for ``lengths``; None when the strategy is unknown to the C++ side."""
    if strategy not in STRATEGY_IDS:
        return None
    L = lib()
    n = len(lengths)
    if n == 0:
        return []
    arr = np.ascontiguousarray(np.asarray(lengths, dtype=np.int64))
    bin_of = np.empty(n, dtype=np.int64)
    slot = np.empty(n, dtype=np.int64)
    nb = L.cb_pack_bins(_pll(arr), n, int(capacity), STRATEGY_IDS[strategy], _pll(bin_of), _pll(slot))
    if nb < 0:
        raise RuntimeError(f"cb_pack_bins failed with code {nb}")
    bins: List[List[int]] = [[] for _ in range(nb)]
    order = np.lexsort((slot, bin_of))
    for i in order.tolist():
        bins[int(bin_of[i])].append(i)
    return bins


def native_fill_rows(items: Sequence[Sequence[int]], bins: Sequence[Sequence[int]], capacity: int, pad_id: int = 0,
                     ignore_index: int = -100, labels: Optional[Sequence[Optional[Sequence[int]]]] = None,
                     mask_first_label: bool = True, max_docs: Optional[int] = None, pin_memory: bool = False):
    """Assemble packed rows from token lists.

    Returns a dict of tensors: ``input_ids``, ``position_ids``, ``labels``, ``sequence_ids``
    (``[rows, capacity]`` int64), ``cu_seqlens`` (``[rows, max_docs + 1]`` int32, padded with the row's
    token count) and ``n_docs`` (``[rows]`` int32).  With ``pin_memory`` the outputs are page-locked so
    the following host→device copy can be asynchronous.
    """
    L = lib()
    n = len(items)
    lens = np.fromiter((len(x) for x in items), dtype=np.int64, count=n)
    offsets = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(lens, out=offsets[1:])
    tokens = np.empty(int(offsets[-1]), dtype=np.int64)
    lab = np.empty_like(tokens) if labels is not None else None
    for i, x in enumerate(items):
        tokens[offsets[i]:offsets[i + 1]] = np.asarray(x, dtype=np.int64)
        if lab is not None:
            li = labels[i]
            lab[offsets[i]:offsets[i + 1]] = np.asarray(li if li is not None else x, dtype=np.int64)
    rows = len(bins)
    row_starts = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(np.fromiter((len(b) for b in bins), dtype=np.int64, count=rows), out=row_starts[1:])
    row_items = np.fromiter((i for b in bins for i in b), dtype=np.int64, count=int(row_starts[-1]))
    md = int(max_docs or max((len(b) for b in bins), default=1) or 1)

    def out(shape, dtype):
        return torch.empty(shape, dtype=dtype, pin_memory=pin_memory and torch.cuda.is_available())
    ids, pos, labs, sid = (out((rows, capacity), torch.int64) for _ in range(4))
    cu, nd = out((rows, md + 1), torch.int32), out((rows,), torch.int32)
    as_ll = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_longlong))
    as_i = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_int))
    code = L.cb_fill_rows(_pll(tokens), _pll(lab) if lab is not None else None, _pll(offsets), _pll(row_items),
                          _pll(row_starts), rows, int(capacity), int(pad_id), int(ignore_index), int(mask_first_label), md,
                          as_ll(ids), as_ll(pos), as_ll(labs), as_ll(sid), as_i(cu), as_i(nd))
    if code != 0:
        raise RuntimeError(f"cb_fill_rows failed with code {code}")
    return {"input_ids": ids, "position_ids": pos, "labels": labs, "sequence_ids": sid, "cu_seqlens": cu, "n_docs": nd}
