"""Tensor + sequence parallel model over gloo equals the single-process model (loss, gradients, state)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("tied", ["tied", "untied"])
def test_tp2_gloo_matches_single_process(tmp_path, tied):
    out = os.path.join(str(tmp_path), "tp.json")
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    port = "29541" if tied == "tied" else "29542"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", port, os.path.join(ROOT, "tests", "_tp_worker.py"), out, "gloo", tied]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert max(abs(a - b) for a, b in zip(res["loss_tp"], res["loss_full"])) < 1e-4, res
    assert res["grad_rel_err_max"] < 1e-3, res
    assert res["state_dict_ok"], res
