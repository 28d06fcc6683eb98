"""Failure paths, exercised without faulting or hanging any GPU.

CPU (no GPU needed): the file rendezvous behind nzb_dp_init times out with a clear message when no
record appears, and refuses a stale record (older than the launch) or a record of another launch
(different nonce); the collective watchdog aborts on an injected error and on a host deadline and
leaves a healthy collective alone. GPU: a bounded device-side wait is made to run out (a barrier
nothing arrives at, with a one-millisecond budget) and the kernel must return with
NZB_ERR_DEVICE_TIMEOUT in the status word, after which the context keeps working.
"""
import ctypes
import os
import struct
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_LIB = os.path.join(ROOT, "neuzephyr_b200", "libneuzephyr_host.so")


@pytest.fixture(scope="module")
def H():
    h = ctypes.CDLL(HOST_LIB)
    h.nzb_dp_last_error_string.restype = ctypes.c_char_p
    h.nzb_dp_rendezvous_publish.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64]
    h.nzb_dp_rendezvous_wait.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64,
                                         ctypes.c_double, ctypes.c_double]
    h.nzb_dp_watchdog_run.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_double,
                                      ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    return h


def test_rendezvous_times_out_without_a_record(H, tmp_path):
    buf = ctypes.create_string_buffer(128)
    t0 = time.time()
    rc = H.nzb_dp_rendezvous_wait(str(tmp_path / "none.id").encode(), buf, 128, 7, 0.5, 60.0)
    assert rc != 0 and 0.4 <= time.time() - t0 < 3.0
    assert b"timed out" in H.nzb_dp_last_error_string() and b"no file" in H.nzb_dp_last_error_string()


def test_rendezvous_accepts_fresh_rejects_stale_and_foreign(H, tmp_path):
    f = str(tmp_path / "run.id").encode()
    payload = bytes(range(128))
    src = ctypes.create_string_buffer(payload, 128)
    assert H.nzb_dp_rendezvous_publish(f, src, 128, 42) == 0
    got = ctypes.create_string_buffer(128)
    assert H.nzb_dp_rendezvous_wait(f, got, 128, 42, 1.0, 60.0) == 0 and got.raw == payload
    # another launch's record
    assert H.nzb_dp_rendezvous_wait(f, got, 128, 43, 0.3, 60.0) != 0
    assert b"nonce" in H.nzb_dp_last_error_string()
    # the same record, but written long before this "launch" began waiting: rewrite its time stamp
    raw = bytearray(open(f, "rb").read())
    magic, nonce, created, nbytes = struct.unpack_from("<QQqQ", raw, 0)
    struct.pack_into("<QQqQ", raw, 0, magic, nonce, created - int(3600e9), nbytes)
    open(f, "wb").write(raw)
    assert H.nzb_dp_rendezvous_wait(f, got, 128, 42, 0.3, 60.0) != 0
    assert b"stale" in H.nzb_dp_last_error_string()
    # a truncated / foreign file is not a record
    open(f, "wb").write(b"garbage")
    assert H.nzb_dp_rendezvous_wait(f, got, 128, 42, 0.3, 60.0) != 0
    # publishing again replaces whatever was there
    assert H.nzb_dp_rendezvous_publish(f, src, 128, 42) == 0
    assert H.nzb_dp_rendezvous_wait(f, got, 128, 42, 1.0, 60.0) == 0


def test_rendezvous_between_two_processes(tmp_path):
    f = str(tmp_path / "two.id")
    child = r"""
import ctypes, sys, time
h = ctypes.CDLL(sys.argv[1])
h.nzb_dp_rendezvous_publish.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64]
time.sleep(0.5)
buf = ctypes.create_string_buffer(b"x" * 128, 128)
sys.exit(h.nzb_dp_rendezvous_publish(sys.argv[2].encode(), buf, 128, 99))
"""
    p = subprocess.Popen([sys.executable, "-c", child, HOST_LIB, f])
    h = ctypes.CDLL(HOST_LIB)
    h.nzb_dp_rendezvous_wait.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64,
                                         ctypes.c_double, ctypes.c_double]
    got = ctypes.create_string_buffer(128)
    assert h.nzb_dp_rendezvous_wait(f.encode(), got, 128, 99, 10.0, 60.0) == 0 and got.raw == b"x" * 128
    assert p.wait(timeout=10) == 0


def _watch(H, script, deadline):
    arr = (ctypes.c_int * len(script))(*script)
    polls, aborted = ctypes.c_int(0), ctypes.c_int(0)
    out = H.nzb_dp_watchdog_run(arr, len(script), deadline, ctypes.byref(polls), ctypes.byref(aborted))
    return out, polls.value, aborted.value


def test_watchdog_injected_error_deadline_and_success(H):
    # finishes: no abort
    assert _watch(H, [1, 1, 0], 5.0) == (0, 3, 0)
    # a peer failed: the poll reports an error code -> abort exactly once, outcome "failed"
    out, polls, aborted = _watch(H, [1, 1, 1, 106], 5.0)
    assert (out, polls, aborted) == (1, 4, 1)
    # a peer never joined: still in progress when the host deadline passes -> abort, outcome "timed out"
    t0 = time.time()
    out, polls, aborted = _watch(H, [1], 0.2)
    assert out == 2 and aborted == 1 and polls > 5 and time.time() - t0 < 2.0


@pytest.mark.gpu
def test_bounded_device_wait_runs_out_and_reports():
    """In a child process (the status word is per process): the wait gives up after ~1 ms of cycles."""
    child = r"""
import ctypes, sys, torch
sys.path.insert(0, %r)
import neuzephyr_b200 as nz
from neuzephyr_b200 import _capi as C
L = C.lib()
assert nz.device_status() == 0
roles = torch.zeros(1, dtype=torch.int32, device="cuda")
s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
assert L.nzb_selftest_wait_timeout(2_000_000, ctypes.c_void_p(roles.data_ptr()), s) == C.OK
torch.cuda.synchronize()                       # the kernel RETURNED
assert nz.device_status() == C.ERR_DEVICE_TIMEOUT
assert int(roles.item()) == 2                  # both warps left through the abort path
assert L.nzb_device_status_reset() == C.OK and nz.device_status() == 0
# the context is intact: a GEMM still runs and is right
a = torch.rand(300, 200, device="cuda"); b = torch.rand(200, 150, device="cuda")
c = nz.gemm(a, b); torch.cuda.synchronize()
assert torch.allclose(c, a.half().float() @ b.half().float(), rtol=1e-3, atol=1e-3) and nz.device_status() == 0
# out-of-range budgets are refused on the host
assert L.nzb_selftest_wait_timeout(1 << 40, ctypes.c_void_p(roles.data_ptr()), s) == C.ERR_BAD_ARG
print("wait timeout ok")
""" % ROOT
    r = subprocess.run([sys.executable, "-c", child], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "wait timeout ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
