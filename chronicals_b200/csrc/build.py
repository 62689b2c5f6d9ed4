"""Builds the CUDA kernels into ``chronicals_b200/_cb_kernels.so`` (in-tree).

Plain ``nvcc`` per ``.cu`` file (sm_100a only), objects linked into one shared
library with a C ABI that ``chronicals_b200.ops._ext`` loads with ctypes.  A
content hash of the sources is stored beside the library so an unchanged tree
is never rebuilt (modification times do not survive copying the tree to
another machine).

Run ``python -m chronicals_b200.csrc.build`` or call :func:`build`.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_PATH = os.path.join(PKG, "_cb_kernels.so")
HASH_PATH = os.path.join(PKG, "_cb_kernels.hash")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def _flags() -> List[str]:
    """``CHRONICALS_DEBUG_BOUNDS=1`` in the environment compiles the extra index checks in."""
    extra = ["-DCHRONICALS_DEBUG_BOUNDS"] if os.environ.get("CHRONICALS_DEBUG_BOUNDS", "0") == "1" else []
    return NVCC_FLAGS + extra


def sources() -> List[str]:
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(_flags()).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(HASH_PATH)):
        return False
    with open(HASH_PATH) as f:
        return f.read().strip() == source_hash()


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    return cand


def _compile_one(nvcc: str, src: str, verbose: bool, obj_dir: str = OBJ_DIR) -> str:
    obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
    cmd = [nvcc, *_flags(), "-I", HERE, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile (if needed) and return the path of the shared library."""
    if not force and is_current():
        return LIB_PATH
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    # Several ranks of one job may find a stale library at the same time: one of them builds, the others wait for
    # the lock and then see a current hash.  Objects and the linked library go to names private to this process
    # and are moved into place atomically, so nobody ever loads a half-written file.
    import fcntl
    with open(os.path.join(OBJ_DIR, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and is_current():
                return LIB_PATH
            obj_dir = os.path.join(OBJ_DIR, f"p{os.getpid()}")
            os.makedirs(obj_dir, exist_ok=True)
            srcs = sources()
            with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
                objs = list(ex.map(lambda s: _compile_one(nvcc, s, verbose, obj_dir), srcs))
            tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
            cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp, *objs]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, LIB_PATH)
            tmp_hash = f"{HASH_PATH}.{os.getpid()}.tmp"
            with open(tmp_hash, "w") as f:
                f.write(source_hash())
            os.replace(tmp_hash, HASH_PATH)
            shutil.rmtree(obj_dir, ignore_errors=True)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
