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


def test_trainer_with_tp2_matches_single_process(tmp_path):
    """``parallel.tp = 2`` inside ChronicalsTrainer: same losses and parameters as one process, including
    global-norm clipping across shards and the gathered HuggingFace-format checkpoint."""
    out = os.path.join(str(tmp_path), "tpt.json")
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29546", os.path.join(ROOT, "tests", "_tp_trainer_worker.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert max(abs(a - b) for a, b in zip(res["tp_losses"], res["single_losses"])) < 1e-4, res
    assert res["max_param_diff"] < 1e-4, res
    assert res["saved_diff"] < 1e-6, res
