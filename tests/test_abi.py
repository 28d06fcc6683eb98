"""CPU-side checks of the C-ABI boundary: the library loads and exports every symbol
include/nzb.h declares; descriptor validation and workspace sizing need no GPU."""
import ctypes
import os
import re

from neuzephyr_b200 import _capi as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# counters of the in-kernel operand staging that follow the two fp16 copies in a GEMM workspace
SYNC = 16384


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nzb.h")).read()
    return sorted(set(re.findall(r"NZB_API\s+[\w\s\*]+?\b(nzb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = C.lib()
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(L, n), n
    assert sorted(C.EXPORTS) == names


def test_desc_layout_matches_header():
    # 3+3 int64, 2 int32, 2 int32, 6 int64, 2 int32, int64, 2 int32
    assert ctypes.sizeof(C.GemmDesc) == 48 + 8 + 8 + 48 + 8 + 8 + 8


def test_workspace_sizing_and_validation():
    L = C.lib()
    d = C.GemmDesc()
    d.M, d.N, d.K = 127, 129, 131
    d.lda, d.ldb, d.ldc = 131, 129, 129
    d.batch[0] = d.batch[1] = 1
    n = ctypes.c_size_t(0)
    assert L.nzb_gemm_workspace_bytes(ctypes.byref(d), ctypes.byref(n)) == C.OK
    # A (M x K) is staged K-major [M][Kp]; B (K x N, N > 32) keeps its layout, MN-major [K][Np]
    kp, np_ = 192, 192
    assert n.value == (127 * kp * 2 + 255) // 256 * 256 + (131 * np_ * 2 + 255) // 256 * 256 + SYNC
    d.batch[0], d.batch[1] = 4, 3
    d.strideA[0], d.strideA[1] = 3 * 127 * 131, 127 * 131
    d.strideB[0], d.strideB[1] = 0, 131 * 129
    assert L.nzb_gemm_workspace_bytes(ctypes.byref(d), ctypes.byref(n)) == C.OK
    assert n.value == (12 * 127 * kp * 2 + 255) // 256 * 256 + (3 * 131 * np_ * 2 + 255) // 256 * 256 + SYNC
    d.transB = 1  # B stored N x K: K-major copy [N][Kp]
    d.ldb = 131
    assert L.nzb_gemm_workspace_bytes(ctypes.byref(d), ctypes.byref(n)) == C.OK
    assert n.value == (12 * 127 * kp * 2 + 255) // 256 * 256 + (3 * 129 * kp * 2 + 255) // 256 * 256 + SYNC
    d.transB = 0
    d.ldb = 129
    d.ldc = 5
    assert L.nzb_gemm_workspace_bytes(ctypes.byref(d), ctypes.byref(n)) == C.ERR_BAD_ARG
    assert b"leading dimension" in L.nzb_last_error_string()
    d.ldc = 129
    d.batch[0] = 0
    assert L.nzb_gemm_workspace_bytes(ctypes.byref(d), ctypes.byref(n)) == C.ERR_BAD_ARG
    assert L.nzb_gemm_workspace_bytes(None, ctypes.byref(n)) == C.ERR_BAD_ARG


def test_shape_entry_points_validate_without_a_device():
    L = C.lib()
    n = ctypes.c_size_t(0)
    sa, sb, sc = C.shape4((2, 1, 8, 16)), C.shape4((1, 3, 16, 4)), C.shape4((2, 3, 8, 4))
    assert L.nzb_tensorcore_gemm_workspace_bytes(sa, sb, sc, ctypes.byref(n)) == C.OK
    assert n.value == (2 * 8 * 64 * 2 + 255) // 256 * 256 + (3 * 4 * 64 * 2 + 255) // 256 * 256 + SYNC
    bad = C.shape4((2, 3, 8, 5))
    assert L.nzb_tensorcore_gemm_workspace_bytes(sa, sb, bad, ctypes.byref(n)) == C.ERR_BAD_ARG
    incompatible = C.shape4((3, 1, 8, 16))
    sb2 = C.shape4((2, 3, 16, 4))
    assert L.nzb_tensorcore_gemm_workspace_bytes(incompatible, sb2, sc, ctypes.byref(n)) == C.ERR_BAD_ARG


def test_version():
    assert C.lib().nzb_version() >= 100


def test_dp_library_exports_and_validates():
    """include/nzb_dp.h: every declared symbol is exported by libneuzephyr_host.so, and argument
    errors are reported before any device or NCCL call."""
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = open(os.path.join(root, "include", "nzb_dp.h")).read()
    names = re.findall(r"NZB_API\s+[\w\s\*]+?\b(nzb_dp_\w+)\s*\(", hdr)
    assert sorted(names) == sorted(["nzb_dp_init", "nzb_dp_allreduce_avg", "nzb_dp_world", "nzb_dp_finalize", "nzb_dp_wait_healthy",
                                    "nzb_dp_rendezvous_publish", "nzb_dp_rendezvous_wait", "nzb_dp_watchdog_run",
                                    "nzb_dp_last_error_string"])
    lib_path = os.path.join(root, "neuzephyr_b200", "libneuzephyr_host.so")
    assert os.path.exists(lib_path), "build the host layer first (python -c 'import __graft_entry__ as g; g.build()')"
    H = ctypes.CDLL(lib_path)
    for n in names:
        assert hasattr(H, n), n
    H.nzb_dp_init.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_double,
                              ctypes.POINTER(ctypes.c_void_p)]
    H.nzb_dp_last_error_string.restype = ctypes.c_char_p
    out = ctypes.c_void_p()
    assert H.nzb_dp_init(2, 2, b"/tmp/unused.id", 0, 1.0, ctypes.byref(out)) == C.ERR_BAD_ARG
    assert b"rank" in H.nzb_dp_last_error_string()
    assert H.nzb_dp_init(0, 2, None, 0, 1.0, ctypes.byref(out)) == C.ERR_BAD_ARG
    H.nzb_dp_allreduce_avg.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    assert H.nzb_dp_allreduce_avg(None, None, 4, None) == C.ERR_BAD_ARG
