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
@pytest.mark.parametrize("shard_optimizer", ["1", "0"])
def test_two_rank_data_parallel_step_matches_full_batch(shard_optimizer):
    """Both forms of the exchange: all-reduce + replicated Adam, and reduce-scatter + Adam on each rank's
    slice + all-gather of the updated weights (the default)."""
    port = "29533" if shard_optimizer == "1" else "29534"
    idf = "/tmp/nz_dp_%s.id" % port
    if os.path.exists(idf):
        os.remove(idf)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NZ_DP_SHARD_OPTIMIZER=shard_optimizer)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", port, "--no-python", _tool(), "check", "8",
                        "64"], capture_output=True, text=True, timeout=600, env=env)
    out = _last_json(r.stdout)
    assert r.returncode == 0 and out["ok"] and out["world"] == 2, r.stdout[-2000:] + r.stderr[-2000:]
    assert abs(out["loss_sharded"] - out["loss_full"]) < 1e-5


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_gradients_against_fp64_host_gradient(tmp_path, world):
    """The data-parallel arithmetic on one GPU (shards run one after the other, gradients averaged on the
    host) measured against an fp64 host gradient of the same step: the sharded average and the full-batch
    gradient must both sit inside the contract's bound, and sharding may not be worse than twice the
    full batch. This is the measurement behind the 2e-3 sharded-versus-full tolerance of `seg_model check`:
    both differ from the truth by fp16 operand rounding, so they differ from each other by as much."""
    import numpy as np
    from oracle import model_step as MS
    B, S = 8, 48
    r = subprocess.run([_tool(), "check", str(B), str(S), "emulate", str(world), str(tmp_path)], capture_output=True,
                       text=True, timeout=300)
    out = _last_json(r.stdout)
    assert r.returncode == 0 and out["ok"] and out["world"] == world, r.stdout[-2000:] + r.stderr[-2000:]
    hp = (S - 5) // 2 + 1
    shapes = [(1, 1, 27, 16), (1, 1, S * S, 16), (1, 1, 144, 16), (1, 1, S * S, 16), (1, 1, 16, 16 * hp * hp), (1, 1, 16, 1)]
    ld = lambda n, shp: np.fromfile(str(tmp_path / (n + ".bin")), dtype=np.float32).reshape(shp)
    x, t = ld("x", (B, 3, S, S)), ld("t", (B, 1, 16, 1))
    params = [ld("p%d" % i, shp) for i, shp in enumerate(shapes)]
    _, truth = MS.seg_model_gradients(x, t, params, exact=True)
    _, rounded = MS.seg_model_gradients(x, t, params, exact=False)
    worst = 0.0
    for i, shp in enumerate(shapes):
        den = np.max(np.abs(truth[i]))
        e_sh = float(np.max(np.abs(ld("sharded_g%d" % i, shp) - truth[i])) / den)
        e_full = float(np.max(np.abs(ld("full_g%d" % i, shp) - truth[i])) / den)
        # what the reference's own arithmetic (fp16-rounded GEMM operands, no loss scaling) loses on this
        # tensor: gradients that reach the first layers are 1e-5 and below, in fp16's subnormal range
        e_alg = float(np.max(np.abs(rounded[i] - truth[i])) / den)
        worst = max(worst, e_sh, e_full)
        bound = max(1e-2, 2 * e_alg)
        assert e_sh <= bound and e_full <= bound, (i, e_sh, e_full, e_alg)
        assert e_sh <= 2 * e_full + 2e-4, (i, e_sh, e_full)
    # the tool's own tolerance between the two is of the size of their distance to the truth
    assert out["max_rel_grad_diff"] <= 2e-3 and out["max_rel_grad_diff"] <= 2 * worst + 2e-4


_DP_CHILD = r"""
import ctypes, os, sys, torch
rank, world, idf, root = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
torch.cuda.set_device(rank)
H = ctypes.CDLL(os.path.join(root, "neuzephyr_b200", "libneuzephyr_host.so"))
H.nzb_dp_init.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_double,
                          ctypes.POINTER(ctypes.c_void_p)]
H.nzb_dp_allreduce_avg.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
H.nzb_dp_finalize.argtypes = [ctypes.c_void_p]
H.nzb_dp_last_error_string.restype = ctypes.c_char_p
comm = ctypes.c_void_p()
rc = H.nzb_dp_init(rank, world, idf.encode(), rank, 60.0, ctypes.byref(comm))
assert rc == 0, H.nzb_dp_last_error_string()
g = torch.full((1000003,), float(rank + 1), device="cuda")
s = torch.cuda.current_stream()
for _ in range(2):  # the second call averages values that are already equal
    assert H.nzb_dp_allreduce_avg(comm, ctypes.c_void_p(g.data_ptr()), g.numel(), ctypes.c_void_p(s.cuda_stream)) == 0
torch.cuda.synchronize()
want = sum(range(1, world + 1)) / world
assert torch.all(g == want).item(), (g[:4], want)
H.nzb_dp_finalize(comm)
print("dp ok", rank)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_dp_c_abi_two_ranks():
    """include/nzb_dp.h through ctypes: two processes, one GPU each, average a gradient buffer in place."""
    idf = "/tmp/nz_dp_abi_%d.id" % os.getpid()
    if os.path.exists(idf):
        os.remove(idf)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", _DP_CHILD, str(r), "2", idf, ROOT], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, env=env) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    if os.path.exists(idf):
        os.remove(idf)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and ("dp ok %d" % r) in o, o[-2000:]
