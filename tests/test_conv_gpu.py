"""Fused implicit-GEMM convolution (forward, backward-data, bias gradient) through the C ABI
against the host oracle's restatement of NeuZephyr's Img2Col -> MatMul -> Bias -> Col2Img
composition. e_max = max|x - ref| / max|ref| <= 2e-5 against the fp64 result on fp16-rounded
operands (fp32 accumulation order is the only difference), <= 1e-2 against unrounded operands."""
import os

import numpy as np
import pytest
import torch

from oracle import nz_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-5


@pytest.fixture(scope="module")
def nz():
    import neuzephyr_b200 as nz
    return nz


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def emax(x, ref):
    ref = np.asarray(ref, np.float64)
    den = np.max(np.abs(ref))
    return float(np.max(np.abs(np.asarray(x, np.float64) - ref)) / (den if den > 0 else 1.0))


CASES = [
    # n, c, h, w, cout, k, stride, pad, per-sample weights
    (2, 3, 6, 5, 4, 3, 1, 1, False),
    (1, 3, 16, 16, 16, 3, 1, 1, False),
    (2, 16, 20, 24, 16, 3, 1, 1, False),
    (3, 5, 13, 11, 7, 3, 1, 1, True),
    (2, 64, 14, 14, 128, 3, 1, 1, False),
    (1, 8, 33, 29, 40, 5, 1, 2, False),
    (2, 4, 17, 19, 24, 3, 2, 0, False),
    (1, 70, 9, 9, 130, 1, 1, 0, False),
    (2, 2, 40, 40, 300, 3, 1, 0, True),
    # output rows of 32 pixels or more take the row-mode kernel (shared-memory window per k block)
    (2, 16, 20, 48, 16, 3, 1, 1, False),
    (1, 3, 10, 130, 16, 3, 1, 1, False),
    (2, 8, 9, 64, 24, 3, 2, 1, False),
    (1, 64, 6, 224, 128, 3, 1, 1, False),
    (1, 5, 12, 100, 7, 5, 1, 2, False),
    (1, 70, 5, 40, 130, 1, 1, 0, False),
    (3, 16, 7, 256, 16, 3, 1, 1, True),
    # stride 1 with taps up to 4x4 and rows of 32+ pixels: the TMA im2col kernel (shifted fp16 copies);
    # odd widths, channel counts that are not multiples of 16, several tiles per row, every pad
    (2, 40, 9, 35, 20, 3, 1, 0, False),
    (1, 6, 8, 70, 33, 2, 1, 1, False),
    (1, 20, 9, 60, 65, 4, 1, 2, False),
    (1, 3, 5, 300, 16, 3, 1, 2, False),
    # 3x3, pad 1, at most 64 output channels, rows of 32+ pixels: the three tap columns are stacked along N and
    # recombined in the epilogue (tiles of 112 output pixels: remainders of 1 and 26, several 16-channel blocks,
    # channel tiles of 16 / 32 / 64)
    (2, 40, 9, 250, 20, 3, 1, 1, False),
    (1, 24, 6, 113, 64, 3, 1, 1, False),
    (2, 16, 5, 112, 48, 3, 1, 1, True),
    # stride 1, shared weights, 64 input channels, 65..128 output channels, rows of 64+ pixels: the forward pass
    # runs from one channels-last fp16 copy (tap shifts are operand-row offsets); segments of 128 + a remainder,
    # pads 0 .. K - 1, 1x1
    (2, 64, 9, 200, 100, 3, 1, 0, False),
    (3, 64, 5, 64, 128, 1, 1, 0, False),
    (2, 64, 12, 130, 96, 3, 1, 2, False),
]


@pytest.mark.parametrize("n,c,h,w,co,k,s,p,per_sample", CASES)
def test_conv_forward(nz, n, c, h, w, co, k, s, p, per_sample):
    rng = np.random.default_rng(n * 100 + c * 10 + co)
    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
    wn = n if per_sample else 1
    wt = (rng.normal(0, 1, (wn, 1, c * k * k, co)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
    ho, wo = O.conv_out_hw(h, w, k, k, s, p)
    bias = rng.normal(0, 1, (1, 1, ho * wo, co)).astype(np.float32)
    y = nz.conv2d_forward(dev(x), dev(wt), dev(bias), k, k, s, p).cpu().numpy()
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    assert emax(y, O.conv2d_forward(x, wt, bias, k, k, s, p, True)) <= TOL
    assert emax(y, O.conv2d_forward(x, wt, bias, k, k, s, p, False)) <= 1e-2
    # no bias + ReLU, and a per-channel bias
    y2 = nz.conv2d_forward(dev(x), dev(wt), None, k, k, s, p, relu=True).cpu().numpy()
    assert emax(y2, O.conv2d_forward(x, wt, None, k, k, s, p, True, relu=True)) <= TOL
    bvec = rng.normal(0, 1, co).astype(np.float32)
    y3 = nz.conv2d_forward(dev(x), dev(wt), dev(bvec), k, k, s, p).cpu().numpy()
    ref3 = O.conv2d_forward(x, wt, None, k, k, s, p, True).astype(np.float64) + bvec[None, :, None, None]
    assert emax(y3, ref3) <= TOL


# The channels-last kernel handles every swizzle width (16 / 32 / 64-channel operand rows), several channel
# blocks and narrow channel tiles; by default it is chosen only where it is the faster one. NZB_CONV_NHWC=2
# (read once per process) selects it wherever it can run.
NHWC_CASES = [
    (2, 16, 12, 130, 16, 3, 1, 1, False),
    (2, 32, 9, 150, 40, 3, 1, 0, False),
    (1, 128, 7, 129, 70, 5, 1, 2, False),
    (3, 64, 5, 64, 130, 1, 1, 0, False),
    (1, 16, 11, 200, 16, 3, 1, 2, False),
    (2, 64, 10, 96, 64, 3, 1, 1, False),
    (1, 64, 6, 224, 128, 3, 1, 1, False),
]


def test_conv_forward_channels_last_everywhere():
    import subprocess
    import sys
    if os.environ.get("NZB_CONV_NHWC") == "2":
        pytest.skip("already running with the channels-last kernel everywhere")
    code = (
        "import sys, numpy as np, torch\n"
        "sys.path.insert(0, %r)\n"
        "import neuzephyr_b200 as nz\n"
        "from oracle import nz_oracle as O\n"
        "from tests.test_conv_gpu import NHWC_CASES, dev, emax, TOL\n"
        "for (n, c, h, w, co, k, s, p, _) in NHWC_CASES:\n"
        "    rng = np.random.default_rng(n * 100 + c * 10 + co)\n"
        "    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)\n"
        "    wt = (rng.normal(0, 1, (1, 1, c * k * k, co)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)\n"
        "    ho, wo = O.conv_out_hw(h, w, k, k, s, p)\n"
        "    bias = rng.normal(0, 1, (1, 1, ho * wo, co)).astype(np.float32)\n"
        "    y = nz.conv2d_forward(dev(x), dev(wt), dev(bias), k, k, s, p, relu=True).cpu().numpy()\n"
        "    torch.cuda.synchronize()\n"
        "    assert nz.device_status() == 0\n"
        "    e = emax(y, O.conv2d_forward(x, wt, bias, k, k, s, p, True, relu=True))\n"
        "    assert e <= TOL, (n, c, h, w, co, k, p, e)\n"
        "    y0 = rng.normal(0, 1, y.shape).astype(np.float32)\n"
        "    ya = dev(y0)\n"
        "    nz.conv2d_forward(dev(x), dev(wt), None, k, k, s, p, out=ya, accumulate=True)\n"
        "    e = emax(ya.cpu().numpy() - y0, O.conv2d_forward(x, wt, None, k, k, s, p, True))\n"
        "    assert e <= 5e-5, ('accumulate', n, c, h, w, co, k, p, e)\n"
        "print('ok')\n"
    ) % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NZB_CONV_NHWC="2")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("n,c,h,w,co,k,s,p,per_sample", [cs for cs in CASES if cs[6] == 1])
def test_conv_backward_data_and_bias(nz, n, c, h, w, co, k, s, p, per_sample):
    rng = np.random.default_rng(n * 7 + c * 3 + co)
    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
    wn = n if per_sample else 1
    wt = (rng.normal(0, 1, (wn, 1, c * k * k, co)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
    ho, wo = O.conv_out_hw(h, w, k, k, s, p)
    dy = rng.normal(0, 1, (n, co, ho, wo)).astype(np.float32)
    dx_ref, _, db_ref = O.conv2d_backward(dy, x, wt, k, k, s, p, want_dw=False)
    dx0 = rng.normal(0, 1, x.shape).astype(np.float32)
    dx = dev(dx0)
    nz.conv2d_backward_data(dev(dy), dev(wt), x.shape, k, k, s, p, dx)
    db0 = rng.normal(0, 1, (1, 1, ho * wo, co)).astype(np.float32)
    db = dev(db0)
    nz.conv2d_backward_bias(dev(dy), x.shape, wt.shape, k, k, s, p, db)
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    assert emax(dx.cpu().numpy() - dx0, dx_ref) <= 5e-5  # accumulated onto dx0: one extra fp32 rounding
    assert emax(db.cpu().numpy() - db0, db_ref) <= 5e-6


@pytest.mark.parametrize("n,c,h,w,co,k,s,p,per_sample", CASES)
def test_conv_backward_weight(nz, n, c, h, w, co, k, s, p, per_sample):
    rng = np.random.default_rng(n * 11 + c * 5 + co)
    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
    wn = n if per_sample else 1
    wshape = (wn, 1, c * k * k, co)
    wt = rng.normal(0, 1, wshape).astype(np.float32)
    ho, wo = O.conv_out_hw(h, w, k, k, s, p)
    dy = rng.normal(0, 1, (n, co, ho, wo)).astype(np.float32)
    _, dw_ref, _ = O.conv2d_backward(dy, x, wt, k, k, s, p, want_dx=False, want_db=False)
    dw0 = rng.normal(0, 1, wshape).astype(np.float32)
    dw = dev(dw0)
    nz.conv2d_backward_weight(dev(x), dev(dy), wshape, k, k, s, p, dw)
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    assert emax(dw.cpu().numpy() - dw0, dw_ref) <= 5e-5


@pytest.mark.parametrize("n,c,h,w,co,k,p,per_sample,relu", [
    (2, 16, 20, 48, 16, 3, 1, False, True), (3, 16, 7, 256, 16, 3, 1, True, False), (1, 64, 6, 224, 128, 3, 1, False, True),
    (2, 40, 9, 35, 20, 3, 0, False, False), (1, 6, 8, 70, 33, 2, 1, False, True), (1, 20, 9, 60, 65, 4, 2, True, True),
    (2, 3, 5, 300, 16, 3, 2, False, False),
    # 3-wide kernels with up to 64 output channels: the weight gradient stacks the tap columns along N
    # (channel tiles of 64 and 32, several 16-channel blocks of x, per-sample weights, every pad)
    (2, 24, 11, 130, 40, 3, 1, False, True), (2, 16, 9, 200, 24, 3, 0, True, False), (1, 70, 6, 64, 64, 3, 2, False, True)])
def test_conv_backward_one_pass(nz, n, c, h, w, co, k, p, per_sample, relu):
    """nzb_conv2d_backward (dY read once: mask, fp16 copies, bias gradient; then both tensor-core kernels on
    the shared copies) against the oracle's backward of Conv2d (+ReLU)."""
    rng = np.random.default_rng(n * 13 + c + co)
    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
    wn = n if per_sample else 1
    wt = (rng.normal(0, 1, (wn, 1, c * k * k, co)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
    ho, wo = O.conv_out_hw(h, w, k, k, 1, p)
    dy = rng.normal(0, 1, (n, co, ho, wo)).astype(np.float32)
    y = rng.normal(0, 1, dy.shape).astype(np.float32) if relu else None
    dy_eff = dy * (y > 0) if relu else dy
    dx_ref, dw_ref, db_ref = O.conv2d_backward(dy_eff, x, wt, k, k, 1, p)
    dx0 = rng.normal(0, 1, x.shape).astype(np.float32)
    dw0 = rng.normal(0, 1, wt.shape).astype(np.float32)
    db0 = rng.normal(0, 1, (1, 1, ho * wo, co)).astype(np.float32)
    dx, dw, db = dev(dx0), dev(dw0), dev(db0)
    nz.conv2d_backward(dev(x), dev(wt), dev(dy), k, k, 1, p, dx=dx, dw=dw, dbias=db, y=dev(y) if relu else None)
    torch.cuda.synchronize()
    assert nz.device_status() == 0
    assert emax(dx.cpu().numpy() - dx0, dx_ref) <= 5e-5
    assert emax(dw.cpu().numpy() - dw0, dw_ref) <= 5e-5
    assert emax(db.cpu().numpy() - db0, db_ref) <= 5e-6
    # overwrite_dx: dx is written, not added to (whatever it held)
    dx3 = dev(dx0 * 1e6)
    nz.conv2d_backward(dev(x), dev(wt), dev(dy), k, k, 1, p, dx=dx3, y=dev(y) if relu else None, overwrite_dx=True)
    assert emax(dx3.cpu().numpy(), dx_ref) <= 5e-5
    # any subset of the outputs
    dw2 = dev(dw0)
    nz.conv2d_backward(dev(x), dev(wt), dev(dy), k, k, 1, p, dw=dw2, y=dev(y) if relu else None)
    assert emax(dw2.cpu().numpy() - dw0, dw_ref) <= 5e-5


def test_conv_chunked_staging_subprocess():
    """With a tiny staging budget the three directions process the batch in chunks of one or two images
    (the path large batches take); results must not change. Runs in a child process because the budget
    is read once per process."""
    import subprocess
    import sys
    code = r"""
import numpy as np, torch, sys
sys.path.insert(0, %r)
import neuzephyr_b200 as nz
from oracle import nz_oracle as O
def emax(x, ref):
    ref = np.asarray(ref, np.float64); den = np.max(np.abs(ref)) or 1.0
    return float(np.max(np.abs(np.asarray(x, np.float64) - ref)) / den)
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
for (n, c, h, w, co, k, p, per_sample) in [(5, 16, 9, 40, 16, 3, 1, False), (5, 3, 8, 64, 20, 3, 1, True)]:
    rng = np.random.default_rng(n + c + co)
    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
    wn = n if per_sample else 1
    wt = (rng.normal(0, 1, (wn, 1, c * k * k, co)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
    ho, wo = O.conv_out_hw(h, w, k, k, 1, p)
    bias = rng.normal(0, 1, (1, 1, ho * wo, co)).astype(np.float32)
    y = nz.conv2d_forward(dev(x), dev(wt), dev(bias), k, k, 1, p).cpu().numpy()
    assert emax(y, O.conv2d_forward(x, wt, bias, k, k, 1, p, True)) <= 3e-5
    dy = rng.normal(0, 1, y.shape).astype(np.float32)
    dx0 = rng.normal(0, 1, x.shape).astype(np.float32)
    dw0 = rng.normal(0, 1, wt.shape).astype(np.float32)
    rdx, rdw, _ = O.conv2d_backward(dy, x, wt, k, k, 1, p, want_db=False)
    dx = dev(dx0); nz.conv2d_backward_data(dev(dy), dev(wt), x.shape, k, k, 1, p, dx)
    assert emax(dx.cpu().numpy() - dx0, rdx) <= 5e-5
    dw = dev(dw0); nz.conv2d_backward_weight(dev(x), dev(dy), wt.shape, k, k, 1, p, dw)
    assert emax(dw.cpu().numpy() - dw0, rdw) <= 5e-5
    db0 = rng.normal(0, 1, bias.shape).astype(np.float32)
    _, _, rdb = O.conv2d_backward(dy, x, wt, k, k, 1, p)
    dx, dw, db = dev(dx0), dev(dw0), dev(db0)
    nz.conv2d_backward(dev(x), dev(wt), dev(dy), k, k, 1, p, dx=dx, dw=dw, dbias=db)
    assert emax(dx.cpu().numpy() - dx0, rdx) <= 5e-5
    assert emax(dw.cpu().numpy() - dw0, rdw) <= 5e-5
    assert emax(db.cpu().numpy() - db0, rdb) <= 5e-6
    torch.cuda.synchronize(); assert nz.device_status() == 0
print("chunked ok")
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NZB_CONV_STAGE_BYTES="40000")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "chunked ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
