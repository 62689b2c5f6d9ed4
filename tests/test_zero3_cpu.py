"""ZeRO-3 bookkeeping (units, gather/release, gradient slots, sharded AdamW) over gloo equals plain AdamW."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_zero3_gloo_matches_single_process(tmp_path):
    out = os.path.join(str(tmp_path), "z3.json")
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29547", os.path.join(ROOT, "tests", "_zero3_worker.py"), out, "gloo"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert max(abs(a - b) for a, b in zip(res["zero3_losses"], res["ref_losses"])) < 1e-4, res
    assert res["max_param_diff"] < 2e-5, res


def test_trainer_zero_stage_3_matches_single_process(tmp_path):
    """``parallel.zero_stage = 3`` inside ChronicalsTrainer (gloo, 2 ranks) equals one process on the joint batch."""
    out = os.path.join(str(tmp_path), "z3t.json")
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29551", os.path.join(ROOT, "tests", "_dp_worker.py"), out, "zero3"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert max(abs(a - b) for a, b in zip(res["dp_losses"], res["single_losses"])) < 1e-4, res
    assert res["max_param_diff"] < 1e-4, res


def test_trainer_zero_stage_1_matches_single_process(tmp_path):
    """``parallel.zero_stage = 1`` (bucketed sharded AdamW, reduce-scatter queued from the gradient hooks) on 2 gloo
    ranks equals one process on the joint batch."""
    out = os.path.join(str(tmp_path), "z1t.json")
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29553", os.path.join(ROOT, "tests", "_dp_worker.py"), out, "zero1"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["optimizer"] == "ShardedFusedAdamW" and res["buckets"] >= 3, res
    assert max(abs(a - b) for a, b in zip(res["dp_losses"], res["single_losses"])) < 1e-4, res
    assert res["max_param_diff"] < 1e-4, res
