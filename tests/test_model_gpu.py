"""The benchmark's segmentation model on the C++ host layer (neuzephyr_b200/host/tools/seg_model.cpp):
a sharded data-parallel step must equal the same step on the full batch. With one visible GPU the
check runs with world size 1 (shard == full batch); with two or more it launches one process per
GPU over NCCL (NVLS disabled, plain ring/tree collectives)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tool():
    from neuzephyr_b200 import build as B
    B.build()
    return B.build_tools()[0]


def _last_json(text):
    for line in reversed(text.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    raise AssertionError("no JSON line in:\n" + text[-2000:])


def test_single_process_step_matches_itself():
    r = subprocess.run([_tool(), "check", "4", "48"], capture_output=True, text=True, timeout=300)
    out = _last_json(r.stdout)
    assert r.returncode == 0 and out["ok"], r.stdout[-2000:] + r.stderr[-2000:]
    assert out["max_abs_param_diff"] < 1e-6


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_data_parallel_step_matches_full_batch():
    port = "29533"
    idf = "/tmp/nz_dp_%s.id" % port
    if os.path.exists(idf):
        os.remove(idf)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", port, "--no-python", _tool(), "check", "8",
                        "64"], capture_output=True, text=True, timeout=600, env=env)
    out = _last_json(r.stdout)
    assert r.returncode == 0 and out["ok"] and out["world"] == 2, r.stdout[-2000:] + r.stderr[-2000:]
    assert abs(out["loss_sharded"] - out["loss_full"]) < 1e-5
