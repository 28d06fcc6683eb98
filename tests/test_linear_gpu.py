"""Linear forward/backward (Model::Linear composition) through the C ABI against the oracle:
Y = relu(X W^T + b); dX = dY' W; dW = dY'^T X; db = sum_b dY'; dY' = dY * (Y > 0).
Tolerances as for the GEMM: e_max <= 2e-5 on fp16-rounded operands (5e-5 where the result is
accumulated onto a non-zero gradient buffer)."""
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


@pytest.mark.parametrize("B,fin,fout,relu", [(8, 30, 16, True), (200, 130, 70, True), (64, 4100, 16, False),
                                             (300, 256, 512, True), (1, 50, 3, False),
                                             # few outputs, long rows: the weight gradient's direct kernel
                                             # (two output tiles, the 256-row variant, the ReLU mask, one output)
                                             (100, 8192, 24, True), (7, 4096, 1, False)])
def test_linear_forward_backward(B, fin, fout, relu):
    import neuzephyr_b200 as nz
    rng = np.random.default_rng(B + fin + fout)
    x = rng.normal(0, 1, (B, fin)).astype(np.float32)
    bound = np.sqrt(6.0 / fin)
    w = rng.uniform(-bound, bound, (fout, fin)).astype(np.float32)
    b = rng.normal(0, 0.1, fout).astype(np.float32)
    y = nz.linear_forward(dev(x), dev(w), dev(b), relu=relu)
    pre = O.gemm_f64(x, np.ascontiguousarray(w.T), True) + b[None, :]
    ref = np.maximum(pre, 0) if relu else pre
    yh = y.cpu().numpy()
    assert emax(yh, ref) <= 2e-5
    dy = rng.normal(0, 1, (B, fout)).astype(np.float32)
    dyp = dy * (yh > 0) if relu else dy
    dx0 = rng.normal(0, 1, x.shape).astype(np.float32)
    dw0 = rng.normal(0, 1, w.shape).astype(np.float32)
    db0 = rng.normal(0, 1, fout).astype(np.float32)
    dx, dw, db = dev(dx0), dev(dw0), dev(db0)
    nz.linear_backward(dev(x), dev(w), y, dev(dy), dx, dw, db, relu=relu)
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    assert emax(dx.cpu().numpy() - dx0, O.gemm_f64(dyp, w, True)) <= 5e-5
    assert emax(dw.cpu().numpy() - dw0, O.gemm_f64(np.ascontiguousarray(dyp.T), x, True)) <= 5e-5
    assert emax(db.cpu().numpy() - db0, dyp.astype(np.float64).sum(axis=0)) <= 5e-5
    # overwrite_dx: dx is written, not added to (whatever it held)
    dx2 = dev(dx0 * 1e6)
    nz.linear_backward(dev(x), dev(w), y, dev(dy), dx2, None, None, relu=relu, overwrite_dx=True)
    assert emax(dx2.cpu().numpy(), O.gemm_f64(dyp, w, True)) <= 5e-5
