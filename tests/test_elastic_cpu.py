"""Elastic restart: a checkpoint written by 2 ranks resumes on 1 and on 4 ranks with the same next losses
(replicated, ZeRO-1 and ZeRO-3 optimizer layouts; gloo ranks on CPU)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "_elastic_worker.py")


def _run(world, port, *args):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), WORKER, *args]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("mode,port", [("dp", 29601), ("zero1", 29611), ("zero3", 29621)])
def test_checkpoint_from_two_ranks_resumes_on_one_and_four(tmp_path, mode, port):
    root = str(tmp_path)
    _run(2, port, root, mode, "save")
    want = json.load(open(os.path.join(root, "save_2.json")))
    for i, world in enumerate((1, 4)):
        _run(world, port + 1 + i, root, mode, "resume")
        got = json.load(open(os.path.join(root, f"resume_{world}.json")))
        assert got["step_count"] == want["step_count"], (got, want)
        # first loss: the weights came back; second loss: the AdamW moments and the step counter came back
        assert max(abs(a - b) for a, b in zip(got["losses"], want["losses"])) < 2e-5, (mode, world, got, want)
