"""Node operations around the contraction (im2col, col2img, bias add, ReLU, pooling, softmax,
BCE, Adam) through the C ABI against the host oracle. Copies and permutations are bit-exact;
sums are compared with the reference's own Tensor::operator== rule (abs 1e-6 or rel 1e-5),
transcendental paths with rtol 1e-5."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import nz_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from neuzephyr_b200 import _capi as C
    return C.lib()


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def P(t):
    return ctypes.c_void_p(t.data_ptr())


def S():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def sh(s):
    return (ctypes.c_int64 * 4)(*[int(v) for v in s])


def tensor_eq(a, b, abs_tol=1e-6, rel_tol=1e-5):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    d = np.abs(a - b)
    return bool(np.all((d <= abs_tol) | (d <= rel_tol * np.maximum(np.abs(a), np.abs(b)))))


@pytest.mark.parametrize("shape,k,s,p", [((2, 3, 4, 5), 3, 1, 1), ((3, 5, 17, 13), 3, 2, 0), ((2, 2, 9, 9), 5, 2, 2),
                                         ((1, 16, 40, 33), 3, 1, 1), ((2, 4, 8, 8), 2, 2, 0)])
def test_img2col_forward_backward(L, shape, k, s, p):
    rng = np.random.default_rng(sum(shape) + k)
    x = rng.uniform(0.1, 0.9, shape).astype(np.float32)
    n, c, h, w = shape
    ho, wo = O.conv_out_hw(h, w, k, k, s, p)
    out = torch.empty((n, 1, ho * wo, c * k * k), device="cuda")
    assert L.nzb_img2col(P(out), P(dev(x)), ho, wo, c, k, k, s, p, h, w, n, S()) == 0
    assert np.array_equal(out.cpu().numpy(), O.img2col(x, k, k, s, p))
    g = rng.uniform(0.1, 0.9, out.shape).astype(np.float32)
    dx0 = rng.uniform(-1, 1, shape).astype(np.float32)
    dx = dev(dx0)
    assert L.nzb_img2col_backward(P(dx), P(dev(g)), ho, wo, c, k, k, s, p, h, w, n, S()) == 0
    want = O.img2col_backward(g, shape, k, k, s, p, dx=dx0.copy())
    assert tensor_eq(dx.cpu().numpy(), want, abs_tol=1e-5)


@pytest.mark.parametrize("n,c,h,w", [(2, 3, 4, 5), (3, 16, 33, 31), (1, 128, 7, 9)])
def test_col2img_roundtrip(L, n, c, h, w):
    rng = np.random.default_rng(n * c * h)
    x = rng.uniform(-1, 1, (n, 1, h * w, c)).astype(np.float32)
    y = torch.empty((n, c, h, w), device="cuda")
    assert L.nzb_col2img(P(y), P(dev(x)), h, w, c, n, S()) == 0
    assert np.array_equal(y.cpu().numpy(), O.col2img(x, h, w, c))
    back = torch.empty((n, 1, h * w, c), device="cuda")
    assert L.nzb_col2img_backward(P(back), P(y), h, w, c, n, S()) == 0
    assert np.array_equal(back.cpu().numpy(), x)


def test_add_broadcast_and_backward(L):
    rng = np.random.default_rng(1)
    for sa, sb in [((2, 1, 4, 5), (1, 3, 4, 5)), ((4, 3, 6, 7), (1, 1, 6, 7)), ((2, 3, 5, 5), (2, 3, 5, 5))]:
        a = rng.uniform(-10, 10, sa).astype(np.float32)
        b = rng.uniform(-10, 10, sb).astype(np.float32)
        so = (max(sa[0], sb[0]), max(sa[1], sb[1]), sa[2], sa[3])
        out = torch.empty(so, device="cuda")
        assert L.nzb_add_broadcast(P(out), P(dev(a)), P(dev(b)), sh(sa), sh(sb), S()) == 0
        assert np.array_equal(out.cpu().numpy(), O.add_broadcast(a, b))
        g = rng.uniform(-10, 10, so).astype(np.float32)
        for sin in (sa, sb):
            g0 = rng.uniform(-1, 1, sin).astype(np.float32)
            gin = dev(g0)
            assert L.nzb_add_backward(P(gin), P(dev(g)), sh(sin), sh(so), S()) == 0
            want = O.add_backward(g, sin, gin=g0.copy())
            assert tensor_eq(gin.cpu().numpy(), want, abs_tol=1e-5)


def test_relu(L):
    rng = np.random.default_rng(2)
    x = rng.uniform(-1, 1, 100003).astype(np.float32)
    g = rng.uniform(-1, 1, 100003).astype(np.float32)
    out = torch.empty(x.size, device="cuda")
    assert L.nzb_relu(P(out), P(dev(x)), x.size, S()) == 0
    assert np.array_equal(out.cpu().numpy(), O.relu(x))
    assert L.nzb_relu_backward(P(out), P(dev(x)), P(dev(g)), x.size, S()) == 0
    assert np.array_equal(out.cpu().numpy(), O.relu_backward(x, g))


@pytest.mark.parametrize("pool,s,p,h,w", [(2, 2, 0, 4, 5), (3, 2, 1, 8, 9), (5, 2, 0, 30, 31), (3, 1, 1, 7, 7),
                                          (4, 3, 2, 13, 11),
                                          # widths that are multiples of 4 take the four-column backward kernels,
                                          # (5|3|2, stride 2, no padding) the compile-time-window kernels
                                          (5, 2, 0, 30, 32), (5, 2, 0, 21, 68), (3, 2, 0, 17, 40), (2, 2, 0, 10, 36),
                                          (4, 3, 0, 20, 24), (3, 1, 0, 9, 16), (5, 2, 0, 5, 8)])
def test_avgpool(L, pool, s, p, h, w):
    rng = np.random.default_rng(pool * 7 + h)
    n, c = 2, 3
    x = rng.uniform(0.1, 0.9, (n, c, h, w)).astype(np.float32)
    ho, wo = (h + 2 * p - pool) // s + 1, (w + 2 * p - pool) // s + 1
    out = torch.empty((n, c, ho, wo), device="cuda")
    assert L.nzb_avgpool(P(out), P(dev(x)), pool, s, p, n, c, h, w, ho, wo, S()) == 0
    assert tensor_eq(out.cpu().numpy(), O.avgpool(x, pool, s, p))
    g = rng.uniform(0.1, 0.9, (n, c, ho, wo)).astype(np.float32)
    g0 = rng.uniform(-1, 1, x.shape).astype(np.float32)
    gin = dev(g0)
    assert L.nzb_avgpool_backward(P(gin), P(dev(g)), pool, s, p, n, c, h, w, ho, wo, S()) == 0
    want = O.avgpool_backward(g, x.shape, pool, s, p, gin=g0.copy())
    assert tensor_eq(gin.cpu().numpy(), want, abs_tol=1e-5)


def test_softmax_forward_backward(L):
    rng = np.random.default_rng(3)
    for n in (16, 8, 100):
        x = rng.uniform(-2, 2, (5, 1, n, 1)).astype(np.float32)
        y = torch.empty(x.shape, device="cuda")
        assert L.nzb_softmax(P(y), P(dev(x)), 5, n, S()) == 0
        yo = O.softmax(x)
        assert np.allclose(y.cpu().numpy(), yo, rtol=1e-5, atol=1e-7)
        g = rng.uniform(-1, 1, x.shape).astype(np.float32)
        gin = torch.empty(x.shape, device="cuda")
        for rnd in (0, 1):
            assert L.nzb_softmax_backward(P(gin), P(dev(yo)), P(dev(g)), 5, n, rnd, S()) == 0
            want = O.softmax_backward(yo, g, round_operands=bool(rnd))
            assert np.allclose(gin.cpu().numpy(), want, rtol=1e-4, atol=1e-6)


def test_bce(L):
    rng = np.random.default_rng(4)
    p = rng.uniform(0.05, 0.95, 5000).astype(np.float32)
    t = (rng.uniform(0, 1, 5000) > 0.5).astype(np.float32)
    loss = torch.zeros(1, device="cuda")
    assert L.nzb_bce(P(loss), P(dev(p)), P(dev(t)), p.size, S()) == 0
    assert abs(loss.item() - O.bce(p, t)) < 1e-5  # the reference's tests compare losses to 1e-2
    g = torch.empty(p.size, device="cuda")
    assert L.nzb_bce_backward(P(g), P(dev(p)), P(dev(t)), p.size, S()) == 0
    assert np.allclose(g.cpu().numpy(), O.bce_backward(p, t), rtol=1e-5, atol=1e-9)


def test_adam_two_steps(L):
    rng = np.random.default_rng(5)
    n = 10007
    data = rng.uniform(-10, 10, n).astype(np.float32)
    grad = rng.uniform(-10, 10, n).astype(np.float32)
    d, m, v = dev(data), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    dh, mh, vh = data.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t in (1, 2):
        assert L.nzb_adam(P(d), P(m), P(v), P(dev(grad)), 0.01, 0.9, 0.999, 1e-6, t, n, S()) == 0
        O.adam(dh, mh, vh, grad, 0.01, 0.9, 0.999, 1e-6, t)
    assert tensor_eq(d.cpu().numpy(), dh, rel_tol=2e-5)
    assert tensor_eq(m.cpu().numpy(), mh) and tensor_eq(v.cpu().numpy(), vh)


def test_fill_expand_scale(L):
    a = torch.empty(1000, device="cuda")
    assert L.nzb_fill(P(a), 2.5, 1000, S()) == 0
    assert torch.all(a == 2.5)
    src = torch.arange(12, dtype=torch.float32, device="cuda")
    out = torch.empty(5 * 12, device="cuda")
    assert L.nzb_expand(P(out), P(src), 12, 5, S()) == 0
    assert torch.equal(out.view(5, 12), src.expand(5, 12))
    assert L.nzb_scale(P(out), 0.5, 60, S()) == 0
    assert torch.equal(out.view(5, 12), (src * 0.5).expand(5, 12))
