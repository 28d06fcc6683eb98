"""nzb_matmul_f32 (the Tensor::operator* seam): fp32-accurate products on the fp16 tensor cores through
a two-fp16 split of each operand. Checked against the reference's literal vector for operator*
(test/Test.cpp TensorBasic.TensorMultiplicationTest, bit-exact: small integers) and against fp64 host
products: e_max = max|x - x64| / max|x64| <= 1.5e-6 (the fp16-operand product sits at 3e-4; numpy's own
fp32 product at 2e-7 to 5e-7), and at least 99 % of the elements satisfy the reference's elementwise
equality rule (abs 1e-6 or rel 1e-5, src/Tensor.cu:506-548) -- the ones that do not are results near
zero, whose absolute error of a few 1e-6 comes from the tensor core's truncating fp32 accumulator, not
from the split (emulated in numpy with exact accumulation the same split gives 8e-8). Operand
magnitudes from 1e-20 to 1e+20 are covered."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import nz_oracle as O

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kat.json")))


@pytest.fixture(scope="module")
def nz():
    import neuzephyr_b200 as nz
    return nz


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def ref_equal(a, b):
    """Tensor::operator== of the reference, element by element: fraction of elements that pass."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    d = np.abs(a - b)
    return float(np.mean((d <= 1e-6) | (d <= 1e-5 * np.maximum(np.abs(a), np.abs(b)))))


def truth(A, B):
    sa, sb = A.shape, B.shape
    out = np.zeros((max(sa[0], sb[0]), max(sa[1], sb[1]), sa[2], sb[3]), dtype=np.float64)
    for i in range(out.shape[0]):
        for j in range(out.shape[1]):
            a = A[i if sa[0] > 1 else 0, j if sa[1] > 1 else 0].astype(np.float64)
            b = B[i if sb[0] > 1 else 0, j if sb[1] > 1 else 0].astype(np.float64)
            out[i, j] = a @ b
    return out


def test_reference_vector_bit_exact(nz):
    k = GOLD["matmul_forward"]
    A = np.array(k["A"], dtype=np.float32).reshape(k["shapeA"])
    B = np.array(k["B"], dtype=np.float32).reshape(k["shapeB"])
    C = nz.matmul_f32(dev(A), dev(B)).cpu().numpy()
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    assert C.shape == tuple(k["shapeC"])
    np.testing.assert_array_equal(C.ravel(), np.array(k["C"], dtype=np.float32))


@pytest.mark.parametrize("sa,sb", [((1, 1, 70, 200), (1, 1, 200, 90)), ((2, 1, 33, 129), (1, 3, 129, 65)),
                                   ((1, 1, 1, 256), (1, 1, 256, 300)), ((1, 2, 300, 64), (1, 2, 64, 7)),
                                   ((1, 1, 257, 100), (1, 1, 100, 31)), ((3, 1, 16, 16), (3, 1, 16, 16))])
def test_reference_equality_rule_on_random_data(nz, sa, sb):
    rng = np.random.default_rng(sum(sa) + sum(sb))
    A = rng.uniform(-1, 1, sa).astype(np.float32)
    B = rng.uniform(-1, 1, sb).astype(np.float32)
    C = nz.matmul_f32(dev(A), dev(B)).cpu().numpy()
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    t = truth(A, B)
    assert float(np.max(np.abs(C - t)) / np.max(np.abs(t))) <= 1.5e-6
    assert ref_equal(C, t) >= 0.99
    # the fp16-operand product of the same tensors is nowhere near that rule
    assert ref_equal(nz.tensorcore_gemm(dev(A), dev(B)).cpu().numpy(), t) < 0.5


@pytest.mark.parametrize("scale_a,scale_b", [(1.0, 1.0), (1e-20, 1e20), (3e7, 2e-9), (1e-20, 1e-8)])
def test_scaling_and_large_contraction(nz, scale_a, scale_b):
    M, N, K = 300, 500, 4096
    rng = np.random.default_rng(5)
    A = (rng.normal(0, 1, (1, 1, M, K)) * scale_a).astype(np.float32)
    B = (rng.normal(0, 1, (1, 1, K, N)) * scale_b).astype(np.float32)
    C = nz.matmul_f32(dev(A), dev(B)).cpu().numpy()
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    t = truth(A, B)
    e = float(np.max(np.abs(C - t)) / np.max(np.abs(t)))
    e32 = float(np.max(np.abs((A[0, 0] @ B[0, 0]) - t[0, 0])) / np.max(np.abs(t)))  # numpy fp32 product
    e16 = float(np.max(np.abs(O.gemm_f64(A[0, 0] * np.float32(1 / scale_a), B[0, 0] * np.float32(1 / scale_b), True)
                              * (scale_a * scale_b) - t[0, 0])) / np.max(np.abs(t)))
    assert e <= 1.5e-6, (e, e32, e16)
    assert e <= 4 * e32 + 2e-7 and e16 >= 50 * e  # fp32-class accuracy, far from the fp16 operand error


def test_mixed_magnitudes_and_zero_operand(nz):
    rng = np.random.default_rng(9)
    A = rng.normal(0, 1, (1, 1, 128, 384)).astype(np.float32)
    A[0, 0, :, ::7] *= 1e-6   # columns far below the largest magnitude keep their absolute accuracy
    A[0, 0, 5, 3] = 4000.0
    B = rng.normal(0, 1, (1, 1, 384, 160)).astype(np.float32)
    C = nz.matmul_f32(dev(A), dev(B)).cpu().numpy()
    t = truth(A, B)
    assert float(np.max(np.abs(C - t)) / np.max(np.abs(t))) <= 2e-6
    Z = nz.matmul_f32(dev(np.zeros_like(A)), dev(B)).cpu().numpy()
    assert np.all(Z == 0)
    torch.cuda.synchronize()
    assert nz.device_status() == 0
