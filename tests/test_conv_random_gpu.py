"""Seeded random sweep of the convolution entry points against the host oracle: kernel sizes 1..5, strides 1
and 2, every pad below the kernel size, channel counts on both sides of every kernel-selection boundary
(16 / 32 / 64 / 128), widths from a few pixels to several 128-pixel segments, shared and per-sample weights,
with and without ReLU. Forward, then the whole backward (the one-call form where the library takes it, the
separate calls otherwise; the fused data gradient is defined for stride 1 only). Tolerances as in
test_conv_gpu.py: fp32 accumulation order is the only difference from the fp64 result on rounded operands."""
import numpy as np
import pytest
import torch

from oracle import nz_oracle as O

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def emax(x, ref):
    ref = np.asarray(ref, np.float64)
    den = np.max(np.abs(ref))
    return float(np.max(np.abs(np.asarray(x, np.float64) - ref)) / (den if den > 0 else 1.0))


@pytest.mark.parametrize("seed", [1, 2])
def test_random_convolutions(seed):
    import neuzephyr_b200 as nz
    rng = np.random.default_rng(seed)
    done = 0
    for _ in range(40):
        k = int(rng.choice([1, 2, 3, 3, 3, 4, 5]))
        s = int(rng.choice([1, 1, 1, 2]))
        p = int(rng.integers(0, k))
        n = int(rng.integers(1, 4))
        c = int(rng.choice([1, 3, 8, 16, 17, 32, 40, 64, 70]))
        co = int(rng.choice([1, 7, 16, 20, 32, 33, 64, 65, 100, 128, 140]))
        h = int(rng.integers(max(k, 3), 14))
        w = int(rng.choice([rng.integers(max(k, 5), 40), rng.integers(32, 80), rng.integers(100, 300), 64, 128, 224, 256]))
        per, relu = bool(rng.integers(0, 4) == 0), bool(rng.integers(0, 2))
        ho, wo = O.conv_out_hw(h, w, k, k, s, p)
        if ho < 1 or wo < 1:
            continue
        tag = (n, c, h, w, co, k, s, p, per, relu)
        x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
        wt = (rng.normal(0, 1, (n if per else 1, 1, c * k * k, co)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
        bias = rng.normal(0, 1, (1, 1, ho * wo, co)).astype(np.float32)
        y = nz.conv2d_forward(dev(x), dev(wt), dev(bias), k, k, s, p, relu=relu).cpu().numpy()
        assert emax(y, O.conv2d_forward(x, wt, bias, k, k, s, p, True, relu=relu)) <= 2e-5, ("forward", tag)
        dy = rng.normal(0, 1, (n, co, ho, wo)).astype(np.float32)
        dy_eff = dy * (y > 0) if relu else dy
        dx_ref, dw_ref, db_ref = O.conv2d_backward(dy_eff, x, wt, k, k, s, p)
        dx = torch.zeros(x.shape, device="cuda")
        dw = torch.zeros(wt.shape, device="cuda")
        db = torch.zeros((1, 1, ho * wo, co), device="cuda")
        try:
            nz.conv2d_backward(dev(x), dev(wt), dev(dy), k, k, s, p, dx=dx, dw=dw, dbias=db, y=dev(y) if relu else None)
        except Exception:  # shapes the one-call form does not take
            dx.zero_(), dw.zero_(), db.zero_()
            if s == 1:
                nz.conv2d_backward_data(dev(dy_eff), dev(wt), x.shape, k, k, s, p, dx)
            nz.conv2d_backward_weight(dev(x), dev(dy_eff), wt.shape, k, k, s, p, dw)
            nz.conv2d_backward_bias(dev(dy_eff), x.shape, wt.shape, k, k, s, p, db)
        torch.cuda.synchronize()
        assert nz.device_status() == 0, tag
        if s == 1:
            assert emax(dx.cpu().numpy(), dx_ref) <= 5e-5, ("dx", tag)
        assert emax(dw.cpu().numpy(), dw_ref) <= 5e-5, ("dw", tag)
        assert emax(db.cpu().numpy(), db_ref) <= 5e-5, ("db", tag)
        done += 1
    assert done >= 30
