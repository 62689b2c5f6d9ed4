"""Host-side failure detection for multi-rank jobs.

Nothing in the reference corresponds to this (it is single-process).  The design follows one
rule: a GPU is never made to fault, trap or hang — failures are noticed on the host, between
steps, and a rank stops *launching* work as soon as it knows a peer is gone, so no kernel is ever
left waiting on a dead peer.

* ``Heartbeat``: every rank bumps a counter in the job's key-value store (the ``torch.distributed``
  TCPStore, or any object with ``set/get``) once per step from the training thread and from a
  background thread every ``interval`` seconds.
* ``Watchdog.check()``: called before each step's first launch; raises ``PeerFailure`` when a
  peer's heartbeat is older than ``timeout`` seconds or when a peer has published an error.
* ``Watchdog.report_failure(exc)``: a rank that catches an exception publishes it so that its
  peers leave at their next ``check()`` instead of timing out inside a collective.
* device-side waits are bounded separately (status word, ``ops._ext.check_status``).

Recovery is restart-from-checkpoint, possibly with a different number of ranks: optimizer shards
are stored per rank and can be consolidated and re-sliced (``parallel.zero.consolidate_states`` /
``reshard_state``).
"""
from __future__ import annotations

import json
import threading
import time
from typing import Any, Callable, Dict, List, Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class DictStore:
    """In-process stand-in for a distributed key-value store (tests, single-process runs)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            if key not in self._d:
                raise KeyError(key)
            return self._d[key]

    def check(self, keys: List[str]) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


def _get(store, key: str) -> Optional[bytes]:
    try:
        if hasattr(store, "check") and not store.check([key]):
            return None
        return store.get(key)
    except Exception:
        return None


_LIVE: "weakref.WeakSet[Heartbeat]" = None  # type: ignore[assignment]


def stop_all() -> None:
    """Stop every running heartbeat thread of this process.  Called before the process group (and with it the
    store the threads write to) is destroyed: a thread caught inside a store call while the interpreter shuts
    down would take the whole process with it."""
    if _LIVE is not None:
        for hb in list(_LIVE):
            hb.stop()


class Heartbeat:
    def __init__(self, store, rank: int, interval: float = 1.0, prefix: str = "cb/hb", clock: Callable[[], float] = time.time):
        self.store, self.rank, self.interval, self.prefix, self.clock = store, rank, interval, prefix, clock
        self.step = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def key(self, rank: Optional[int] = None) -> str:
        return f"{self.prefix}/{self.rank if rank is None else rank}"

    def beat(self, step: Optional[int] = None) -> None:
        if step is not None:
            self.step = step
        self.store.set(self.key(), json.dumps({"t": self.clock(), "step": self.step}))

    def start(self) -> "Heartbeat":
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return

        self._stop.clear()
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        global _LIVE
        if _LIVE is None:
            import atexit
            import weakref
            _LIVE = weakref.WeakSet()
            atexit.register(stop_all)
        _LIVE.add(self)
        return self

    @property
    def running(self) -> bool:
        return self._thread is not None and self._thread.is_alive()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
            self._thread = None


class Watchdog:
    def __init__(self, store, rank: int, world_size: int, timeout: float = 30.0, interval: float = 1.0,
                 prefix: str = "cb", clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world, self.timeout, self.prefix, self.clock = store, rank, world_size, timeout, prefix, clock
        self.heartbeat = Heartbeat(store, rank, interval, f"{prefix}/hb", clock)
        self.failed: Optional[PeerFailure] = None

    def start(self) -> "Watchdog":
        self.heartbeat.start()
        return self

    def stop(self) -> None:
        self.heartbeat.stop()

    def report_failure(self, exc: BaseException) -> None:
        """Publish this rank's failure so peers stop launching work that would wait for it."""
        try:
            self.store.set(f"{self.prefix}/err/{self.rank}", json.dumps({"t": self.clock(), "error": repr(exc)[:500]}))
        except Exception:
            pass

    def peer_status(self) -> List[Dict[str, Any]]:
        now = self.clock()
        out = []
        for r in range(self.world):
            hb = _get(self.store, f"{self.prefix}/hb/{r}")
            err = _get(self.store, f"{self.prefix}/err/{r}")
            info = json.loads(hb.decode()) if hb else None
            out.append({"rank": r, "age": (now - info["t"]) if info else None, "step": info["step"] if info else None,
                        "error": json.loads(err.decode())["error"] if err else None})
        return out

    def check(self, step: Optional[int] = None) -> None:
        """Call between steps, before the first launch of the next step."""
        self.heartbeat.beat(step)
        for st in self.peer_status():
            if st["rank"] == self.rank:
                continue
            if st["error"] is not None:
                self.failed = PeerFailure(st["rank"], f"reported {st['error']}")
            elif st["age"] is not None and st["age"] > self.timeout:
                self.failed = PeerFailure(st["rank"], f"no heartbeat for {st['age']:.1f} s (last step {st['step']})")
            if self.failed is not None:
                raise self.failed

    def guard(self, fn: Callable, *a, **kw):
        """Run ``fn``; on any exception publish it for the peers and re-raise."""
        try:
            return fn(*a, **kw)
        except BaseException as e:
            self.report_failure(e)
            raise


def watchdog_from_process_group(timeout: float = 30.0, interval: float = 1.0) -> Optional[Watchdog]:
    """A watchdog on the default process group's store (None when not distributed)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return None
    store = dist.distributed_c10d._get_default_store()
    return Watchdog(store, dist.get_rank(), dist.get_world_size(), timeout, interval)
