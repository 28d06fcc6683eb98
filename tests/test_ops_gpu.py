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
    # overwrite form: whatever gin held is replaced by the gradient alone
    gin2 = dev(g0 * 1e6)
    assert L.nzb_avgpool_backward_ex(P(gin2), P(dev(g)), pool, s, p, n, c, h, w, ho, wo, 1, S()) == 0
    assert tensor_eq(gin2.cpu().numpy(), O.avgpool_backward(g, x.shape, pool, s, p), abs_tol=1e-5)


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


def test_adam_multi_matches_per_tensor_adam_and_writes_fp16_copies(L):
    """nzb_adam_multi: one launch over tensors of different sizes, alignments and time steps equals
    nzb_adam tensor by tensor (bit for bit) and the oracle; the optional fp16 copy is the RN rounding of
    the updated weights."""
    from neuzephyr_b200 import _capi as C
    rng = np.random.default_rng(6)
    sizes = [10007, 16, 4096 * 3, 1, 70001]
    ts = [1, 3, 7, 10, 15]
    base = [torch.empty(n + 3, device="cuda") for n in sizes]  # slices at offset 1 or 3: unaligned tensors
    offs = [0, 1, 0, 3, 0]
    data_h = [rng.uniform(-10, 10, n).astype(np.float32) for n in sizes]
    grad_h = [rng.uniform(-10, 10, n).astype(np.float32) for n in sizes]
    d = [b[o:o + n] for b, o, n in zip(base, offs, sizes)]
    for t_, h in zip(d, data_h):
        t_.copy_(torch.from_numpy(h))
    m = [torch.zeros(n, device="cuda") for n in sizes]
    v = [torch.zeros(n, device="cuda") for n in sizes]
    g = [dev(h) for h in grad_h]
    shadows = [torch.empty(n, dtype=torch.float16, device="cuda") if i % 2 == 0 else None for i, n in enumerate(sizes)]
    d2 = [dev(h) for h in data_h]
    m2 = [torch.zeros(n, device="cuda") for n in sizes]
    v2 = [torch.zeros(n, device="cuda") for n in sizes]
    for step in range(2):
        arr = (C.AdamTensor * len(sizes))()
        for i, n in enumerate(sizes):
            arr[i].data, arr[i].m, arr[i].v, arr[i].grad = d[i].data_ptr(), m[i].data_ptr(), v[i].data_ptr(), g[i].data_ptr()
            arr[i].shadow_f16 = shadows[i].data_ptr() if shadows[i] is not None else None
            arr[i].n, arr[i].t = n, ts[i] + 20 * step
        assert L.nzb_adam_multi(arr, len(sizes), 0.01, 0.9, 0.999, 1e-6, S()) == 0
        for i, n in enumerate(sizes):
            assert L.nzb_adam(P(d2[i]), P(m2[i]), P(v2[i]), P(g[i]), 0.01, 0.9, 0.999, 1e-6, ts[i] + 20 * step, n, S()) == 0
    torch.cuda.synchronize()
    for i, n in enumerate(sizes):
        assert torch.equal(d[i], d2[i]) and torch.equal(m[i], m2[i]) and torch.equal(v[i], v2[i])
        if shadows[i] is not None:
            assert np.array_equal(shadows[i].view(torch.int16).cpu().numpy().view(np.uint16), O.f16_bits(d[i].cpu().numpy()))
        dh, mh, vh = data_h[i].copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        for step in range(2):
            O.adam(dh, mh, vh, grad_h[i], 0.01, 0.9, 0.999, 1e-6, ts[i] + 20 * step)
        assert tensor_eq(d[i].cpu().numpy(), dh, rel_tol=2e-5)


def test_softmax_bce_head(L):
    """The fused head equals softmax -> BCE and BCE backward -> softmax backward (both rounding modes)."""
    rng = np.random.default_rng(8)
    for batches, n in ((5, 16), (64, 16), (3, 100), (1000, 7)):
        x = rng.uniform(-2, 2, (batches, 1, n, 1)).astype(np.float32)
        t = (rng.uniform(0, 1, x.shape) > 0.5).astype(np.float32)
        probs = torch.empty(x.shape, device="cuda")
        loss = torch.full((1,), 0.25, device="cuda")  # the loss scalar accumulates
        assert L.nzb_softmax_bce_forward(P(probs), P(loss), P(dev(x)), P(dev(t)), batches, n, S()) == 0
        yo = O.softmax(x)
        assert np.allclose(probs.cpu().numpy(), yo, rtol=1e-5, atol=1e-7)
        assert abs(loss.item() - 0.25 - O.bce(yo, t)) < 1e-5
        dl = torch.empty(x.shape, device="cuda")
        for rnd in (0, 1):
            assert L.nzb_softmax_bce_backward(P(dl), P(dev(yo)), P(dev(t)), batches, n, rnd, S()) == 0
            want = O.softmax_backward(yo, O.bce_backward(yo, t), round_operands=bool(rnd))
            scale = np.max(np.abs(want))
            assert np.max(np.abs(dl.cpu().numpy() - want)) <= 1e-5 * scale + 1e-9


@pytest.mark.parametrize("pool,s,p,h,w", [(2, 2, 0, 4, 5), (3, 2, 1, 8, 9), (5, 2, 0, 30, 31), (3, 1, 1, 7, 7),
                                          (4, 3, 2, 13, 11), (2, 2, 0, 64, 64), (3, 3, 0, 9, 12)])
def test_maxpool(L, pool, s, p, h, w):
    rng = np.random.default_rng(pool * 11 + h)
    n, c = 2, 3
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    x[0, 0, :2, :2] = 0.5  # ties: the first maximum in window order must win
    ho, wo = (h + 2 * p - pool) // s + 1, (w + 2 * p - pool) // s + 1
    out = torch.empty((n, c, ho, wo), device="cuda")
    pos = torch.empty((n, c, ho, wo), device="cuda")
    assert L.nzb_maxpool(P(out), P(pos), P(dev(x)), pool, s, p, n, c, h, w, ho, wo, S()) == 0
    o_out, o_pos = O.maxpool(x, pool, s, p)
    assert np.array_equal(out.cpu().numpy(), o_out) and np.array_equal(pos.cpu().numpy(), o_pos)
    g = rng.uniform(0.1, 0.9, (n, c, ho, wo)).astype(np.float32)
    g0 = rng.uniform(-1, 1, x.shape).astype(np.float32)
    gin = dev(g0)
    assert L.nzb_maxpool_backward(P(gin), P(pos), P(dev(g)), pool, s, p, n, c, h, w, ho, wo, S()) == 0
    want = O.maxpool_backward(g, o_pos, x.shape, pool, s, p, gin=g0.copy())
    assert tensor_eq(gin.cpu().numpy(), want, abs_tol=1e-5)
