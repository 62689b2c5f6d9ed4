"""Failure detection is exercised on the host only: a rank that stops beating, a rank that
publishes an error, a gloo rank that leaves between steps.  No GPU is involved."""
import json
import os
import subprocess
import sys

import pytest

from chronicals_b200.parallel.watchdog import DictStore, PeerFailure, Watchdog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _Clock:
    def __init__(self):
        self.t = 1000.0

    def __call__(self):
        return self.t


def test_stale_heartbeat_is_detected():
    store, clock = DictStore(), _Clock()
    a = Watchdog(store, 0, 2, timeout=5.0, clock=clock)
    b = Watchdog(store, 1, 2, timeout=5.0, clock=clock)
    a.heartbeat.beat(0)
    b.heartbeat.beat(0)
    a.check(1)                      # both fresh
    clock.t += 3
    b.heartbeat.beat(1)
    a.check(2)
    clock.t += 6                    # rank 1 never beats again
    with pytest.raises(PeerFailure) as e:
        a.check(3)
    assert e.value.rank == 1 and "no heartbeat" in e.value.reason


def test_reported_error_reaches_peers():
    store = DictStore()
    a, b = Watchdog(store, 0, 2), Watchdog(store, 1, 2)
    a.heartbeat.beat()
    b.heartbeat.beat()

    def boom():
        raise ValueError("bad batch")

    with pytest.raises(ValueError):
        b.guard(boom)
    with pytest.raises(PeerFailure) as e:
        a.check()
    assert e.value.rank == 1 and "bad batch" in e.value.reason


def test_background_thread_keeps_beating():
    import time
    store = DictStore()
    w = Watchdog(store, 0, 1, interval=0.05).start()
    t0 = json.loads(store.get("cb/hb/0"))["t"]
    time.sleep(0.3)
    w.stop()
    assert json.loads(store.get("cb/hb/0"))["t"] > t0


def test_gloo_rank_leaves_between_steps(tmp_path):
    """Rank 1 raises after step 2 and publishes it; rank 0 notices at its next check, before it would
    enter another collective, and exits cleanly."""
    out = os.path.join(str(tmp_path), "res.json")
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29547", os.path.join(ROOT, "tests", "_watchdog_worker.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    res = json.load(open(out))
    assert res["detected_rank"] == 1 and res["steps_done"] == 2, (res, r.stderr[-1500:])


def test_trainer_stops_launching_after_peer_failure(tmp_path):
    """A rank that raises between steps publishes the error; the surviving rank notices at its next pre-step
    check, writes an emergency state directory and raises ``PeerFailure`` instead of hanging in a collective."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = os.path.join(str(tmp_path), "wd")
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29549", os.path.join(root, "tests", "_trainer_watchdog_worker.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert os.path.exists(out + ".0.json") and os.path.exists(out + ".1.json"), r.stdout[-1500:] + r.stderr[-3000:]
    r0, r1 = json.load(open(out + ".0.json")), json.load(open(out + ".1.json"))
    assert r1["outcome"].startswith("raised:injected")
    assert r0["outcome"] == "peer_failure" and r0["failed_rank"] == 1 and r0["step"] == 2, r0
    assert any(n.startswith("emergency-") for n in r0["emergency"]), r0
