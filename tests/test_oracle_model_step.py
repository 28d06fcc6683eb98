"""Pins oracle/model_step.py (the composed training step of the segmentation model) on the CPU:
its layers against the C oracle functions that the reference's own vectors pin
(tests/test_oracle_kat.py), its gradient against central differences of its own loss in float64,
and its Adam update against the C oracle's AdamKernel restatement."""
import numpy as np

from oracle import model_step as MS
from oracle import nz_oracle as O


def _params(rng, N, S, per_sample=False, scale=0.2):
    hp = (S - 5) // 2 + 1
    shapes = [(N if per_sample else 1, 1, 27, 16), (1, 1, S * S, 16), (N if per_sample else 1, 1, 144, 16),
              (1, 1, S * S, 16), (1, 1, 16, 16 * hp * hp), (1, 1, 16, 1)]
    return [rng.uniform(-scale, scale, s).astype(np.float32) for s in shapes]


def test_conv_layer_matches_c_oracle():
    rng = np.random.default_rng(0)
    for per_sample in (False, True):
        N, C, S, Co = 3, 5, 9, 7
        x = rng.normal(0, 1, (N, C, S, S)).astype(np.float32)
        w = rng.normal(0, 0.3, (N if per_sample else 1, 1, C * 9, Co)).astype(np.float32)
        b = rng.normal(0, 1, (1, 1, S * S, Co)).astype(np.float32)
        dy = rng.normal(0, 1, (N, Co, S, S)).astype(np.float32)
        conv = MS._Conv(x.shape, 3, 1, Co, O.round_f16, np.float32)
        y = conv.forward(x, w, b)
        np.testing.assert_allclose(y, O.conv2d_forward(x, w, b, 3, 3, 1, 1), rtol=1e-5, atol=1e-5)
        dx, dw, db = conv.backward(dy, w, True)
        rdx, rdw, rdb = O.conv2d_backward(dy, x, w, 3, 3, 1, 1)
        np.testing.assert_allclose(dx, rdx, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(dw, rdw, rtol=1e-5, atol=1e-4)
        np.testing.assert_allclose(db, rdb, rtol=1e-5, atol=1e-5)


def test_pool_softmax_bce_adam_match_c_oracle():
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, (2, 3, 13, 13)).astype(np.float32)
    np.testing.assert_allclose(MS._avgpool(x, 5, 2), O.avgpool(x, 5, 2, 0), rtol=1e-6, atol=1e-6)
    g = rng.normal(0, 1, (2, 3, 5, 5)).astype(np.float32)
    np.testing.assert_allclose(MS._avgpool_backward(g, x.shape, 5, 2), O.avgpool_backward(g, x.shape, 5, 2, 0),
                               rtol=1e-6, atol=1e-6)
    p = rng.normal(0, 1, 1000).astype(np.float32)
    grad = rng.normal(0, 1e-3, 1000).astype(np.float32)
    for t in (1, 3, 17, 37):
        a, m, v = p.copy(), np.zeros_like(p), np.zeros_like(p)
        b, m2, v2 = p.copy(), np.zeros_like(p), np.zeros_like(p)
        MS.adam_step(a, m, v, grad, 0.01, 0.9, 0.999, 1e-6, t)
        O.adam(b, m2, v2, grad, 0.01, 0.9, 0.999, 1e-6, t)
        np.testing.assert_allclose(a, b, rtol=2e-7, atol=2e-7)  # one fp32 ulp: data - step is rounded once in each
        np.testing.assert_allclose(m, m2, rtol=1e-6)


def test_gradient_matches_central_differences():
    """float64, no rounding: d(loss)/d(parameter) from the composed backward equals a central difference."""
    rng = np.random.default_rng(2)
    N, S = 2, 9
    x = rng.normal(0, 1, (N, 3, S, S))
    t = (rng.uniform(0, 1, (N, 1, 16, 1)) < 0.5).astype(np.float64)
    params = [p.astype(np.float64) for p in _params(rng, N, S)]
    loss, grads = MS.seg_model_gradients(x, t, params, exact=True)
    assert np.isfinite(loss)
    for i, (p, g) in enumerate(zip(params, grads)):
        flat = p.reshape(-1)
        for k in rng.choice(flat.size, 6, replace=False):
            old = flat[k]
            h = 1e-5
            flat[k] = old + h
            lp, _ = MS.seg_model_gradients(x, t, params, exact=True)
            flat[k] = old - h
            lm, _ = MS.seg_model_gradients(x, t, params, exact=True)
            flat[k] = old
            num = (lp - lm) / (2 * h)
            assert abs(num - g.reshape(-1)[k]) <= 1e-6 + 1e-4 * abs(num), (i, k, num, g.reshape(-1)[k])


def test_rounded_mode_stays_close_to_exact_and_time_steps():
    rng = np.random.default_rng(3)
    N, S = 2, 12
    x = rng.uniform(-1, 1, (N, 3, S, S)).astype(np.float32)
    t = (rng.uniform(0, 1, (N, 1, 16, 1)) < 0.5).astype(np.float32)
    params = _params(rng, N, S)
    l32, g32 = MS.seg_model_gradients(x, t, params, exact=False)
    l64, g64 = MS.seg_model_gradients(x, t, params, exact=True)
    assert abs(l32 - l64) <= 1e-3 * abs(l64)
    for a, b in zip(g32, g64):
        assert np.max(np.abs(a - b)) <= 1e-2 * np.max(np.abs(b))
    # the first update moves parameter i by the Adam step of time ts[i]; for t = 1 that is lr * g / (|g| + eps)
    losses, first, after = MS.seg_model_steps(x, t, params, 2)
    assert len(after) == 2 and MS.REF_T == (1, 3, 7, 10, 15, 17)
    g = first[0]
    want = params[0] - 0.01 * g / (np.abs(g) + 1e-6)
    np.testing.assert_allclose(after[0][0], want, rtol=0, atol=1e-6)
