"""Parity of the sm_100a GEMM path (through the C ABI) against the host oracle.

Error metric: e_max = max|x - x64| / max|x64| per output tensor.
  * against the fp64 product of the fp16-rounded operands (what the reference's WMMA
    kernel approximates): e_max <= 2e-5 -- only fp32 accumulation order differs;
  * against the fp64 product of the raw fp32 operands: e_max <= 1e-2, the bound the
    baseline contract states for this path.
"""
import ctypes
import json
import os

import numpy as np
import pytest
import torch

from oracle import nz_oracle as O

pytestmark = pytest.mark.gpu

TOL_ROUNDED = 2e-5
TOL_RAW = 1e-2
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kat.json")))


@pytest.fixture(scope="module")
def nz():
    import neuzephyr_b200 as nz
    return nz


def emax(x, ref):
    ref = np.asarray(ref, dtype=np.float64)
    den = np.max(np.abs(ref))
    return float(np.max(np.abs(np.asarray(x, dtype=np.float64) - ref)) / (den if den > 0 else 1.0))


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def check_status(nz):
    torch.cuda.synchronize()
    assert nz.device_status() == 0


SHAPES = [
    (1, 1, 1), (16, 16, 16), (15, 17, 16), (17, 15, 33), (127, 129, 131), (128, 256, 64), (129, 257, 65),
    (300, 40, 700), (1, 512, 640), (640, 1, 512), (256, 512, 1), (1024, 1024, 1024), (3, 1000, 7),
    (513, 72, 1030), (200, 130, 48), (2000, 24, 200),
]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_shapes(nz, M, N, K):
    rng = np.random.default_rng(M * 1000003 + N * 1009 + K)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    C = nz.gemm(dev(A), dev(B)).cpu().numpy()
    check_status(nz)
    assert emax(C, O.gemm_f64(A, B, True)) <= TOL_ROUNDED
    assert emax(C, O.gemm_f64(A, B, False)) <= TOL_RAW


def test_config1_seed0_1024(nz):
    """The headline configuration's CPU-runnable case: 1024^3, uniform[-1,1], seed 0."""
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (1024, 1024)).astype(np.float32)
    B = rng.uniform(-1, 1, (1024, 1024)).astype(np.float32)
    C = nz.gemm(dev(A), dev(B)).cpu().numpy()
    check_status(nz)
    e_r = emax(C, O.gemm_f64(A, B, True))
    e_raw = emax(C, O.gemm_f64(A, B, False))
    assert e_r <= TOL_ROUNDED and e_raw <= TOL_RAW


@pytest.mark.parametrize("M,N,K", [(150, 90, 210), (300, 520, 130), (64, 40, 100), (1, 33, 70), (257, 24, 65),
                                   (520, 300, 1000)])
@pytest.mark.parametrize("tA,tB", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_transposed_operands(nz, tA, tB, M, N, K):
    """Every storage combination: stored K x M / K x N operands are read MN-major by the tensor core
    (no transposing pass), N <= 32 takes the transposing staging pass."""
    rng = np.random.default_rng(42 + M)
    A = rng.normal(0, 1, (M, K)).astype(np.float32)
    B = rng.normal(0, 1, (K, N)).astype(np.float32)
    As = np.ascontiguousarray(A.T) if tA else A
    Bs = np.ascontiguousarray(B.T) if tB else B
    C = nz.gemm(dev(As), dev(Bs), transA=tA, transB=tB).cpu().numpy()
    check_status(nz)
    assert emax(C, O.gemm_f64(A, B, True)) <= TOL_ROUNDED


def test_gemm_epilogue_bias_relu_accumulate(nz):
    from neuzephyr_b200 import _capi as C
    rng = np.random.default_rng(7)
    for (M, N, K) in [(130, 96, 200), (77, 33, 50)]:
        A = rng.normal(0, 1, (M, K)).astype(np.float32)
        B = rng.normal(0, 1, (K, N)).astype(np.float32)
        ref = O.gemm_f64(A, B, True)
        brow = rng.normal(0, 1, N).astype(np.float32)
        bcol = rng.normal(0, 1, M).astype(np.float32)
        bmat = rng.normal(0, 1, (M, N)).astype(np.float32)
        got = nz.gemm(dev(A), dev(B), bias=dev(brow), bias_mode=C.BIAS_ROW).cpu().numpy()
        assert emax(got, ref + brow[None, :]) <= TOL_ROUNDED
        got = nz.gemm(dev(A), dev(B), bias=dev(bcol), bias_mode=C.BIAS_COL, relu=True).cpu().numpy()
        assert emax(got, np.maximum(ref + bcol[:, None], 0)) <= TOL_ROUNDED
        got = nz.gemm(dev(A), dev(B), bias=dev(bmat), bias_mode=C.BIAS_MATRIX, relu=True).cpu().numpy()
        assert emax(got, np.maximum(ref + bmat, 0)) <= TOL_ROUNDED
        c0 = rng.normal(0, 1, (M, N)).astype(np.float32)
        out = dev(c0)
        nz.gemm(dev(A), dev(B), out=out, accumulate=True)
        assert emax(out.cpu().numpy(), ref + c0) <= TOL_ROUNDED
    check_status(nz)


@pytest.mark.parametrize("M,N,K", [(16, 5000, 16), (7, 300, 5000), (32, 129, 100), (1, 4096, 4096), (3, 70, 33),
                                   (16, 16, 40000)])
@pytest.mark.parametrize("tA,tB", [(False, False), (True, True)])
def test_gemm_tiny_m_and_split_k_epilogues(nz, M, N, K, tA, tB):
    """A few rows against a wide output run with the operands swapped and a transposed epilogue; few
    tiles with a long contraction are shared among CTAs along k (the first slice adds the bias)."""
    from neuzephyr_b200 import _capi as C
    rng = np.random.default_rng(M * 7919 + N + K)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    As = dev(np.ascontiguousarray(A.T) if tA else A)
    Bs = dev(np.ascontiguousarray(B.T) if tB else B)
    ref = O.gemm_f64(A, B, True)
    # one accumulator chain over a very long contraction carries fp32 accumulation error that grows with K
    tol = max(TOL_ROUNDED, 5e-9 * K)
    brow = rng.normal(0, 1, N).astype(np.float32)
    bcol = rng.normal(0, 1, M).astype(np.float32)
    bmat = rng.normal(0, 1, (M, N)).astype(np.float32)
    got = nz.gemm(As, Bs, transA=tA, transB=tB).cpu().numpy()
    assert emax(got, ref) <= tol
    got = nz.gemm(As, Bs, transA=tA, transB=tB, bias=dev(brow), bias_mode=C.BIAS_ROW).cpu().numpy()
    assert emax(got, ref + brow[None, :]) <= tol
    got = nz.gemm(As, Bs, transA=tA, transB=tB, bias=dev(bcol), bias_mode=C.BIAS_COL, relu=True).cpu().numpy()
    assert emax(got, np.maximum(ref + bcol[:, None], 0)) <= tol
    got = nz.gemm(As, Bs, transA=tA, transB=tB, bias=dev(bmat), bias_mode=C.BIAS_MATRIX).cpu().numpy()
    assert emax(got, ref + bmat) <= tol
    c0 = rng.normal(0, 1, (M, N)).astype(np.float32)
    out = dev(c0)
    nz.gemm(As, Bs, transA=tA, transB=tB, out=out, accumulate=True)
    assert emax(out.cpu().numpy(), ref + c0) <= tol
    out = dev(c0)
    nz.gemm(As, Bs, transA=tA, transB=tB, out=out, accumulate=True, bias=dev(brow), bias_mode=C.BIAS_ROW)
    assert emax(out.cpu().numpy(), ref + c0 + brow[None, :]) <= tol
    check_status(nz)


def test_reference_kat_matmul_forward(nz):
    """TensorCore.TensorCoreGEMMTest / NodeBasic.MatMulForward literals; integers are exact in fp16."""
    g = GOLD["matmul_forward"]
    A = np.array(g["A"], np.float32).reshape(g["shapeA"])
    B = np.array(g["B"], np.float32).reshape(g["shapeB"])
    C = nz.tensorcore_gemm(dev(A), dev(B)).cpu().numpy()
    check_status(nz)
    assert C.shape == tuple(g["shapeC"])
    assert np.array_equal(C, np.array(g["C"], np.float32).reshape(g["shapeC"]))


def test_reference_kat_matmul_backward(nz):
    """NodeBasic.MatMulBackwardSpecial / MatMulBackwardNormal: dA = dC B^T, dB = A^T dC, summed over broadcast dims."""
    g = GOLD["matmul_backward_normal"]
    A = np.array(g["A"], np.float32).reshape(g["shapeA"])
    B = np.array(g["B"], np.float32).reshape(g["shapeB"])
    dC = np.array(g["dC"], np.float32).reshape(2, 3, 2, 2)
    dA = torch.zeros(g["shapeA"], device="cuda")
    dB = torch.zeros(g["shapeB"], device="cuda")
    nz.gemm_backward(dev(dC), dev(O.transpose(B)), dA)
    nz.gemm_backward(dev(O.transpose(A)), dev(dC), dB)
    check_status(nz)
    assert np.array_equal(dA.cpu().numpy().ravel(), np.array(g["dA"], np.float32))
    assert np.array_equal(dB.cpu().numpy().ravel(), np.array(g["dB"], np.float32))
    s = GOLD["matmul_backward_special"]
    A1 = torch.ones(s["shapeA"], device="cuda")
    B1 = torch.ones(s["shapeB"], device="cuda")
    dC1 = torch.ones((2, 3, 2, 2), device="cuda")
    dA1 = torch.zeros(s["shapeA"], device="cuda")
    dB1 = torch.zeros(s["shapeB"], device="cuda")
    nz.gemm_backward(dC1, dev(O.transpose(B1.cpu().numpy())), dA1)
    nz.gemm_backward(dev(O.transpose(A1.cpu().numpy())), dC1, dB1)
    assert torch.all(dA1 == s["dA_fill"]) and torch.all(dB1 == s["dB_fill"])


@pytest.mark.parametrize("sa,sb", [((2, 1, 40, 70), (1, 3, 70, 50)), ((3, 2, 33, 17), (3, 2, 17, 65)),
                                   ((1, 1, 20, 30), (4, 1, 30, 10)), ((2, 3, 130, 64), (1, 1, 64, 24))])
def test_batched_broadcast_forward(nz, sa, sb):
    rng = np.random.default_rng(sum(sa) * 31 + sum(sb))
    A = rng.uniform(-1, 1, sa).astype(np.float32)
    B = rng.uniform(-1, 1, sb).astype(np.float32)
    C = nz.tensorcore_gemm(dev(A), dev(B)).cpu().numpy()
    check_status(nz)
    assert emax(C, O.gemm_forward(A, B, True, f64=True)) <= TOL_ROUNDED


@pytest.mark.parametrize("sa,sb,sc", [
    ((2, 3, 20, 30), (1, 3, 30, 10), (2, 3, 20, 10)),   # no reduction
    ((2, 3, 30, 20), (2, 3, 20, 10), (1, 3, 30, 10)),   # sum over N
    ((4, 2, 16, 100), (4, 2, 100, 8), (1, 1, 16, 8)),   # sum over N and C
    ((2, 3, 30, 20), (2, 3, 20, 10), (2, 1, 30, 10)),   # sum over C
])
def test_batched_backward_accumulate_and_reduce(nz, sa, sb, sc):
    rng = np.random.default_rng(sum(sa) * 17 + sum(sc))
    A = rng.uniform(-1, 1, sa).astype(np.float32)
    B = rng.uniform(-1, 1, sb).astype(np.float32)
    C0 = rng.uniform(-1, 1, sc).astype(np.float32)
    ref = C0.astype(np.float64)
    O.gemm_backward(A, B, ref, True)
    out = dev(C0)
    nz.gemm_backward(dev(A), dev(B), out)
    check_status(nz)
    assert emax(out.cpu().numpy(), ref) <= TOL_ROUNDED


@pytest.mark.parametrize("M,N,K,acc", [(16, 24, 20000, False), (100, 300, 9000, False), (200, 130, 30000, True),
                                       (576, 128, 12544, True), (1, 16, 70000, False)])
def test_split_k_long_contraction(nz, M, N, K, acc):
    """Few output tiles and a long contraction: k is split across CTAs and partial sums are added
    with fp32 atomics (as the reference's CuttingAndCompress does), so only the tolerance applies."""
    rng = np.random.default_rng(M + N + K)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (M, N)).astype(np.float32) if acc else np.zeros((M, N), np.float32)
    out = dev(c0) if acc else torch.full((M, N), float("nan"), device="cuda")
    nz.gemm(dev(A), dev(B), out=out, accumulate=acc)
    check_status(nz)
    assert emax(out.cpu().numpy(), O.gemm_f64(A, B, True) + c0) <= TOL_ROUNDED


def test_split_k_with_batch_reduction(nz):
    rng = np.random.default_rng(77)
    A = rng.uniform(-1, 1, (6, 1, 40, 3000)).astype(np.float32)
    B = rng.uniform(-1, 1, (6, 1, 3000, 24)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (1, 1, 40, 24)).astype(np.float32)
    ref = C0.astype(np.float64)
    O.gemm_backward(A, B, ref, True)
    out = dev(C0)
    nz.gemm_backward(dev(A), dev(B), out)
    check_status(nz)
    assert emax(out.cpu().numpy(), ref) <= TOL_ROUNDED


def test_cast_matches_oracle_bits(nz):
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.uniform(-1, 1, 3000), rng.normal(0, 300, 3000), rng.uniform(-1e-5, 1e-5, 2000),
                        [65504, 65519, 65520, 7e4, -7e4, 2.0 ** -24, 2.0 ** -25, 0.0]]).astype(np.float32)
    x = x[: (x.size // 77) * 77].reshape(-1, 77)
    got = nz.cast_f32_f16(dev(x)).cpu().numpy()
    assert got.shape[1] == 128 and np.all(got[:, 77:] == 0)
    assert np.array_equal(got[:, :77].view(np.uint16), O.f16_bits(x))
    gt = nz.cast_f32_f16(dev(x), transpose=True).cpu().numpy()
    assert np.array_equal(gt[:, : x.shape[0]].view(np.uint16), O.f16_bits(x.T.copy()))
    assert np.all(gt[:, x.shape[0]:] == 0)


def test_linearity_large(nz):
    """Size-independent property at a size the CPU oracle does not check in full:
    (A1 + A2) B == A1 B + A2 B for operands whose sums are exact in fp16 (small integers),
    plus sampled rows against the fp64 oracle."""
    M, N, K = 2048, 2304, 4096
    rng = np.random.default_rng(99)
    A1 = rng.integers(-4, 5, (M, K)).astype(np.float32)
    A2 = rng.integers(-4, 5, (M, K)).astype(np.float32)
    B = rng.integers(-4, 5, (K, N)).astype(np.float32)
    Bd = dev(B)
    c12 = nz.gemm(dev(A1 + A2), Bd)
    c1 = nz.gemm(dev(A1), Bd)
    c2 = nz.gemm(dev(A2), Bd)
    check_status(nz)
    assert torch.equal(c12, c1 + c2)  # all partial sums are integers below 2^24: exact
    rows = np.array([0, 1, 127, 128, 1000, 2047])
    assert np.array_equal(c1.cpu().numpy()[rows], O.gemm_f64_rows(A1, B, rows, True).astype(np.float32))


def test_argument_errors(nz):
    from neuzephyr_b200 import _capi as C
    L = C.lib()
    d = C.GemmDesc()
    d.M, d.N, d.K = 4, 4, 4
    d.lda = d.ldb = d.ldc = 4
    d.batch[0] = d.batch[1] = 1
    a = torch.zeros(16, device="cuda")
    p = ctypes.c_void_p(a.data_ptr())
    assert L.nzb_gemm(ctypes.byref(d), p, p, p, None, None, 0, None) == C.ERR_WORKSPACE
    assert L.nzb_gemm(ctypes.byref(d), None, p, p, None, p, 1 << 20, None) == C.ERR_BAD_ARG
    d.lda = 2
    assert L.nzb_gemm(ctypes.byref(d), p, p, p, None, p, 1 << 20, None) == C.ERR_BAD_ARG
    bad = C.shape4((1, 1, 4, 5))
    ok = C.shape4((1, 1, 4, 4))
    assert L.nzb_tensorcore_gemm(p, p, p, bad, ok, ok, p, 1 << 20, None) == C.ERR_BAD_ARG
    assert b"B.H" in L.nzb_last_error_string()


@pytest.mark.parametrize("M,N,K,tB", [(1300, 700, 520, False), (2048, 512, 256, True), (40, 33, 70, False),
                                     (5000, 136, 64, False)])
def test_gemm_host_pipeline_matches_device_call(nz, M, N, K, tB):
    """nzb_gemm_host (host operands, copies and row blocks pipelined on three streams) gives exactly
    what nzb_gemm gives on device-resident copies of the same data, bias / ReLU included."""
    from neuzephyr_b200 import _capi as C
    rng = np.random.default_rng(M + N + K)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    Bs = np.ascontiguousarray(B.T) if tB else B
    brow = rng.normal(0, 1, N).astype(np.float32)
    bcol = rng.normal(0, 1, M).astype(np.float32)
    hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(Bs).pin_memory()
    for bias, mode, relu in [(None, C.BIAS_NONE, False), (brow, C.BIAS_ROW, True), (bcol, C.BIAS_COL, False)]:
        hb = torch.from_numpy(bias).pin_memory() if bias is not None else None
        hC = nz.gemm_host(hA, hB, transB=tB, bias=hb, bias_mode=mode, relu=relu)
        torch.cuda.synchronize()
        ref = nz.gemm(dev(A), dev(Bs), transB=tB, bias=dev(bias) if bias is not None else None, bias_mode=mode,
                      relu=relu).cpu().numpy()
        assert np.array_equal(hC.numpy(), ref)
    # pageable buffers work too (no overlap), and two calls in a row reuse the pipe's events safely
    hC1 = nz.gemm_host(torch.from_numpy(A), torch.from_numpy(Bs), transB=tB)
    hC2 = nz.gemm_host(hA, hB, transB=tB)
    torch.cuda.synchronize()
    assert np.array_equal(hC1.numpy(), hC2.numpy())
    check_status(nz)
    assert emax(hC2.numpy(), O.gemm_f64(A, B, True)) <= TOL_ROUNDED


@pytest.mark.parametrize("tA,tB", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_in_kernel_staging_odd_shapes(nz, tA, tB):
    """One matrix product with 148 or more 256x256 tiles takes the CTA-pair kernel with its own converter
    warps (fp32 -> fp16 staging inside the GEMM kernel, panel by panel behind counters): extents that are
    not multiples of the tile or chunk sizes, every storage combination, a second call on the same
    workspace (the counters are cleared per call), and the fused epilogue."""
    from neuzephyr_b200 import _capi as C
    M, N, K = 3100, 3332, 1000
    rng = np.random.default_rng(77)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    As = np.ascontiguousarray(A.T) if tA else A
    Bs = np.ascontiguousarray(B.T) if tB else B
    Ad, Bd = dev(As), dev(Bs)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    out = None
    for _ in range(2):
        out = nz.gemm(Ad, Bd, transA=tA, transB=tB, bias=dev(bias), bias_mode=C.BIAS_ROW, relu=True).cpu().numpy()
    check_status(nz)
    rows = np.unique(np.concatenate([[0, 255, 256, M - 1], rng.integers(0, M, 40)]))
    cols = np.unique(np.concatenate([[0, 255, 256, N - 1], rng.integers(0, N, 40)]))
    ref_r = np.maximum(O.gemm_f64_rows(A, B, rows, True) + bias[None, :], 0)
    ref_c = np.maximum(O.gemm_f64_rows(np.ascontiguousarray(B.T), np.ascontiguousarray(A.T), cols, True)
                       + bias[cols][:, None], 0)
    assert emax(out[rows], ref_r) <= TOL_ROUNDED
    assert emax(out[:, cols].T, ref_c) <= TOL_ROUNDED
