"""Pins the host oracle against the known answers of NeuZephyr's own tests (test/Test.cpp).

Literal vectors come from tests/golden/reference_kat.json; where the reference test
derives its expectation from a host formula over random data, the formula is restated
here in numpy (independently of the C++ oracle) with correctly sized buffers.
"""
import json
import os

import numpy as np
import pytest

from oracle import nz_oracle as O

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kat.json")))


def tensor_eq(a, b):
    """Tensor::operator== of the reference: abs 1e-6 or rel 1e-5 (src/Tensor.cu:506-548)."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    d = np.abs(a - b)
    return bool(np.all((d <= 1e-6) | (d <= 1e-5 * np.maximum(np.abs(a), np.abs(b)))))


def test_f16_rounding_matches_numpy():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.uniform(-1, 1, 20000), rng.normal(0, 100, 20000), rng.uniform(-1e-7, 1e-7, 2000),
        rng.uniform(-7e-5, 7e-5, 5000), np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e6, -1e6, 2.0 ** -24,
                                                   2.0 ** -25, 1.5 * 2.0 ** -25, 2.0 ** -14, 1.0009765625,
                                                   1.00048828125, 1.00146484375])]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    got = O.f16_bits(x)
    assert np.array_equal(got, want.view(np.uint16))
    assert np.array_equal(O.round_f16(x), want.astype(np.float32))


def test_matmul_forward_literals():
    g = GOLD["matmul_forward"]
    A = np.array(g["A"], np.float32).reshape(g["shapeA"])
    B = np.array(g["B"], np.float32).reshape(g["shapeB"])
    want = np.array(g["C"], np.float32).reshape(g["shapeC"])
    for f64 in (False, True):
        for rnd in (False, True):
            C = O.gemm_forward(A, B, round_operands=rnd, f64=f64)
            assert C.shape == tuple(g["shapeC"])
            assert tensor_eq(C, want)


def test_matmul_backward_special():
    g = GOLD["matmul_backward_special"]
    A = np.full(g["shapeA"], g["fillA"], np.float32)
    B = np.full(g["shapeB"], g["fillB"], np.float32)
    dC = np.full((2, 3, 2, 2), g["fill_dC"], np.float32)
    dA = np.zeros(g["shapeA"], np.float32)
    dB = np.zeros(g["shapeB"], np.float32)
    O.matmul_node_backward(A, B, dC, dA, dB)
    assert tensor_eq(dA, np.full(g["shapeA"], g["dA_fill"]))
    assert tensor_eq(dB, np.full(g["shapeB"], g["dB_fill"]))


def test_matmul_backward_normal():
    g = GOLD["matmul_backward_normal"]
    A = np.array(g["A"], np.float32).reshape(g["shapeA"])
    B = np.array(g["B"], np.float32).reshape(g["shapeB"])
    dC = np.array(g["dC"], np.float32).reshape(2, 3, 2, 2)
    for dt in (np.float32, np.float64):
        dA = np.zeros(g["shapeA"], dt)
        dB = np.zeros(g["shapeB"], dt)
        O.matmul_node_backward(A, B, dC, dA, dB)
        assert tensor_eq(dA, np.array(g["dA"]))
        assert tensor_eq(dB, np.array(g["dB"]))


def test_backward_accumulates():
    """GEMMBackwardParallel adds into the gradient buffer (CuttingAndCompress)."""
    rng = np.random.default_rng(1)
    A = rng.integers(-3, 4, (2, 1, 3, 4)).astype(np.float32)
    B = rng.integers(-3, 4, (2, 1, 4, 5)).astype(np.float32)
    C = np.full((2, 1, 3, 5), 7.0, np.float32)
    O.gemm_backward(A, B, C)
    assert np.array_equal(C, 7.0 + np.matmul(A, B))


def test_add_forward_and_backward():
    g = GOLD["add_backward_special"]
    rng = np.random.default_rng(2)
    a = rng.uniform(-10, 10, g["shape1"]).astype(np.float32)
    b = rng.uniform(-10, 10, g["shape2"]).astype(np.float32)
    assert tensor_eq(O.add_broadcast(a, b), a + b)  # NodesBasic.AddForward, test/Test.cpp:615-649
    gout = np.full((2, 3, 4, 5), g["fill_dOut"], np.float32)
    assert tensor_eq(O.add_backward(gout, g["shape1"]), np.full(g["shape1"], g["grad1_fill"]))
    assert tensor_eq(O.add_backward(gout, g["shape2"]), np.full(g["shape2"], g["grad2_fill"]))
    # NodesBasic.AddBackwardNormal, test/Test.cpp:673-706
    gout = rng.uniform(-10, 10, (2, 3, 4, 5)).astype(np.float32)
    assert np.array_equal(O.add_backward(gout, (2, 3, 4, 5)), gout)
    assert tensor_eq(O.add_backward(gout, (1, 3, 4, 5)), gout.sum(axis=0, keepdims=True))


def _im2col_numpy(x, kh, kw, s, p):
    """Index rule of TensorBasic.img2colTest (test/Test.cpp:2880-2944)."""
    n, c, h, w = x.shape
    ho, wo = (h + 2 * p - kh) // s + 1, (w + 2 * p - kw) // s + 1
    out = np.zeros((n, 1, ho * wo, c * kh * kw), np.float32)
    for b in range(n):
        for i in range(ho):
            for j in range(wo):
                for r in range(kh):
                    for t in range(kw):
                        hi, wi = i * s - p + r, j * s - p + t
                        if 0 <= hi < h and 0 <= wi < w:
                            out[b, 0, i * wo + j, np.arange(c) * kh * kw + r * kw + t] = x[b, :, hi, wi]
    return out


@pytest.mark.parametrize("shape,k,s,p", [((2, 3, 4, 5), 3, 1, 1), ((1, 2, 7, 6), 3, 2, 0), ((2, 1, 5, 5), 2, 1, 1)])
def test_img2col_forward_backward(shape, k, s, p):
    rng = np.random.default_rng(3)
    x = rng.uniform(0.1, 0.9, shape).astype(np.float32)
    col = O.img2col(x, k, k, s, p)
    want = _im2col_numpy(x, k, k, s, p)
    assert np.array_equal(col, want)
    # NodeBasic.img2colBackward (test/Test.cpp:3012-3072): scatter-add of the column gradient.
    g = rng.uniform(0.1, 0.9, col.shape).astype(np.float32)
    dx = O.img2col_backward(g, shape, k, k, s, p)
    n, c, h, w = shape
    ho, wo = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    ref = np.zeros(shape, np.float64)
    for b in range(n):
        for pos in range(ho * wo):
            for m in range(c * k * k):
                ci, r, t = m // (k * k), (m % (k * k)) // k, m % k
                hi, wi = (pos // wo) * s - p + r, (pos % wo) * s - p + t
                if 0 <= hi < h and 0 <= wi < w:
                    ref[b, ci, hi, wi] += g[b, 0, pos, m]
    assert tensor_eq(dx, ref)


def test_col2img_roundtrip():
    """TenorBasic.col2imgTest / NodeBasic.col2imgForward/Col2imgBackward (test/Test.cpp:3074-3177)."""
    rng = np.random.default_rng(4)
    n, c, h, w = 2, 3, 4, 5
    x = rng.uniform(0.1, 0.9, (n, 1, h * w, c)).astype(np.float32)
    y = O.col2img(x, h, w, c)
    assert np.array_equal(y, x.reshape(n, h, w, c).transpose(0, 3, 1, 2))
    assert np.array_equal(O.col2img_backward(y), x)


def test_relu():
    """NodeBasic.ReLUForward/Backward (test/Test.cpp:1054-1108)."""
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, 1000).astype(np.float32)
    g = rng.uniform(-1, 1, 1000).astype(np.float32)
    assert np.array_equal(O.relu(x), np.maximum(x, 0))
    assert np.array_equal(O.relu_backward(x, g), np.where(x > 0, g, 0))


@pytest.mark.parametrize("pool,s,p", [(2, 2, 0), (3, 2, 1), (5, 2, 0)])
def test_avgpool(pool, s, p):
    """TensorBasic.AveragePooling, NodeBasic.AveragePoolingForward/Backward (test/Test.cpp:3179-3385)."""
    rng = np.random.default_rng(6)
    n, c, h, w = 2, 3, 8, 9
    x = rng.uniform(0.1, 0.9, (n, c, h, w)).astype(np.float32)
    ho, wo = (h + 2 * p - pool) // s + 1, (w + 2 * p - pool) // s + 1
    want = np.zeros((n, c, ho, wo), np.float64)
    cnt = np.zeros((ho, wo))
    for k in range(ho):
        for l in range(wo):
            for r in range(pool):
                for t in range(pool):
                    hi, wi = k * s - p + r, l * s - p + t
                    if 0 <= hi < h and 0 <= wi < w:
                        want[:, :, k, l] += x[:, :, hi, wi]
                        cnt[k, l] += 1
    want /= cnt
    assert tensor_eq(O.avgpool(x, pool, s, p), want)
    g = rng.uniform(0.1, 0.9, (n, c, ho, wo)).astype(np.float32)
    ref = np.zeros((n, c, h, w), np.float64)
    for k in range(ho):
        for l in range(wo):
            div = cnt[k, l] if p else pool * pool
            for r in range(pool):
                for t in range(pool):
                    hi, wi = k * s - p + r, l * s - p + t
                    if 0 <= hi < h and 0 <= wi < w:
                        ref[:, :, hi, wi] += g[:, :, k, l] / div
    assert tensor_eq(O.avgpool_backward(g, (n, c, h, w), pool, s, p), ref)


@pytest.mark.parametrize("pool,s,p", [(2, 2, 0), (3, 2, 1), (3, 1, 0)])
def test_maxpool(pool, s, p):
    """NodeBasic.MaxPoolingForward / MaxPoolingBackward (test/Test.cpp:3460-3617): the expected values are the
    test's own host loops (first strict maximum of the window wins, an empty window gives 0, the gradient goes
    to the position of the maximum), restated here on seeded inputs of the test's shape and a larger one."""
    rng = np.random.default_rng(8)
    for (n, c, h, w) in ((2, 3, 4, 5), (2, 2, 9, 11)):
        x = rng.uniform(0.1, 0.9, (n, c, h, w)).astype(np.float32)
        ho, wo = (h + 2 * p - pool) // s + 1, (w + 2 * p - pool) // s + 1
        want = np.zeros((n, c, ho, wo), np.float32)
        idx = np.zeros((n, c, ho, wo), np.int64)
        for i in range(n):
            for j in range(c):
                for k in range(ho):
                    for l in range(wo):
                        best, bi = -1e20, 0
                        for r in range(pool):
                            for t in range(pool):
                                hi, wi = k * s - p + r, l * s - p + t
                                if 0 <= hi < h and 0 <= wi < w and x[i, j, hi, wi] > best:
                                    best, bi = x[i, j, hi, wi], r * pool + t
                        want[i, j, k, l] = 0.0 if best == -1e20 else best
                        idx[i, j, k, l] = bi
        out, pos = O.maxpool(x, pool, s, p)
        assert np.array_equal(out, want)
        assert np.array_equal(pos.astype(np.int64), idx)
        g = rng.uniform(0.1, 0.9, (n, c, ho, wo)).astype(np.float32)
        ref = np.zeros((n, c, h, w), np.float64)
        for i in range(n):
            for j in range(c):
                for k in range(ho):
                    for l in range(wo):
                        hi, wi = k * s - p + idx[i, j, k, l] // pool, l * s - p + idx[i, j, k, l] % pool
                        if 0 <= hi < h and 0 <= wi < w:
                            ref[i, j, hi, wi] += g[i, j, k, l]
        assert tensor_eq(O.maxpool_backward(g, pos, (n, c, h, w), pool, s, p), ref)


def test_softmax_and_jacobian():
    """NodeBasic.SoftmaxForward, TensorBasic.SoftmaxJacobianTest, NodeBasic.SoftmaxBackwardRow (test/Test.cpp:1735-1870)."""
    rng = np.random.default_rng(7)
    x = rng.uniform(-1, 1, (2, 3, 8, 1)).astype(np.float32)
    y = O.softmax(x)
    e = np.exp(x.astype(np.float64))
    assert tensor_eq(y, e / e.sum(axis=(2, 3), keepdims=True))
    y0 = y[0, 0].ravel()
    J = O.softmax_jacobian(y0)
    assert tensor_eq(J, np.diag(y0) - np.outer(y0, y0))
    g = rng.uniform(-1, 1, x.shape).astype(np.float32)
    dx = O.softmax_backward(y, g, round_operands=False)
    yy = y.astype(np.float64)
    gg = g.astype(np.float64)
    want = yy * (gg - (yy * gg).sum(axis=(2, 3), keepdims=True))
    assert np.allclose(dx, want, rtol=1e-5, atol=1e-7)


def test_bce():
    """NodeLoss.BCEForward/BCEBackward (test/Test.cpp:1937-2000): mean over all elements; loss compared to 1e-2."""
    rng = np.random.default_rng(8)
    p = rng.uniform(0.1, 0.9, 240).astype(np.float32)
    t = (rng.uniform(0, 1, 240) > 0.5).astype(np.float32)
    want = np.mean(-t * np.log(p.astype(np.float64)) - (1 - t) * np.log(1 - p.astype(np.float64)))
    assert abs(O.bce(p, t) - want) < 1e-6
    gw = (p.astype(np.float64) - t) / (p.astype(np.float64) * (1 - p.astype(np.float64))) / p.size
    assert tensor_eq(O.bce_backward(p, t), gw)


def test_adam_two_steps():
    """OptimizerBasic.AdamTest (test/Test.cpp:2398-2451): two steps, eps 1e-6, t = 1, 2."""
    rng = np.random.default_rng(9)
    n = 2 * 3 * 3 * 4
    data = rng.uniform(-10, 10, n).astype(np.float32)
    grad = rng.uniform(-10, 10, n).astype(np.float32)
    lr, b1, b2, eps = np.float32(0.01), np.float32(0.9), np.float32(0.999), np.float32(1e-6)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    exp = data.copy()
    for it in (1, 2):
        m = b1 * m + (1 - b1) * grad
        v = b2 * v + (1 - b2) * grad * grad
        mm = m / np.float32(1 - np.power(b1, it))
        vv = v / np.float32(1 - np.power(b2, it))
        exp = exp - (lr / (np.sqrt(vv) + eps)) * mm
    d, m2, v2 = data.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.adam(d, m2, v2, grad, 0.01, 0.9, 0.999, 1e-6, 1)
    O.adam(d, m2, v2, grad, 0.01, 0.9, 0.999, 1e-6, 2)
    assert tensor_eq(d, exp)
    assert tensor_eq(m2, m) and tensor_eq(v2, v)


def test_conv_composition_equals_direct():
    """Model::Conv2d = Img2Col -> MatMul -> Bias -> Col2Img (src/Model.cu:244-263): the fused
    oracle entry must equal the node-by-node composition, forward and backward."""
    rng = np.random.default_rng(10)
    n, c, h, w, co, k, s, p = 2, 3, 6, 5, 4, 3, 1, 1
    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
    for wn in (1, n):
        wt = rng.normal(0, 0.3, (wn, 1, c * k * k, co)).astype(np.float32)
        ho, wo = O.conv_out_hw(h, w, k, k, s, p)
        bias = rng.normal(0, 1, (1, 1, ho * wo, co)).astype(np.float32)
        col = O.img2col(x, k, k, s, p)
        mm = O.gemm_forward(col, wt, round_operands=True, f64=True).astype(np.float32)
        want = O.col2img(O.add_broadcast(mm, bias), ho, wo, co)
        got = O.conv2d_forward(x, wt, bias, k, k, s, p, round_operands=True)
        assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
        # backward
        dy = rng.normal(0, 1, (n, co, ho, wo)).astype(np.float32)
        dmm = O.col2img_backward(dy)
        db_w = O.add_backward(dmm, bias.shape)
        dcol = np.zeros(col.shape, np.float64)
        dw_w = np.zeros(wt.shape, np.float64)
        O.matmul_node_backward(col, wt, dmm, dcol, dw_w, round_operands=True)
        dx_w = O.img2col_backward(dcol.astype(np.float32), x.shape, k, k, s, p)
        dx, dw, db = O.conv2d_backward(dy, x, wt, k, k, s, p)
        assert np.allclose(db, db_w, rtol=1e-5, atol=1e-5)
        assert np.allclose(dw, dw_w, rtol=1e-5, atol=1e-4)
        assert np.allclose(dx, dx_w, rtol=1e-5, atol=1e-4)


def test_gemm_f32_baseline_agrees_with_f64():
    rng = np.random.default_rng(11)
    A = rng.uniform(-1, 1, (70, 131)).astype(np.float32)
    B = rng.uniform(-1, 1, (131, 45)).astype(np.float32)
    c64 = O.gemm_f64(A, B, True)
    c32 = O.gemm_f32(A, B, True)
    assert np.max(np.abs(c32 - c64)) / np.max(np.abs(c64)) < 1e-5
    rows = np.array([0, 5, 69])
    assert np.array_equal(O.gemm_f64_rows(A, B, rows, True), c64[rows])
    want = O.round_f16(A).astype(np.float64) @ O.round_f16(B).astype(np.float64)
    assert np.allclose(c64, want, rtol=1e-12, atol=1e-12)
