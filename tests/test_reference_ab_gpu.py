"""A/B against NeuZephyr itself: the reference library rebuilt for sm_100 (oracle/_ref, built by
oracle/build_ref.sh from the reference's own sources) runs GEMMTensorCore / iGEMMBackward on the same
seeded inputs, and both results are measured against the fp64 oracle on the unrounded inputs.
Acceptance (the baseline contract): e_max(ours) <= 1e-2 and e_max(ours) <= 2 * e_max(reference).
Skipped when oracle/_ref has not been built (it needs the reference source tree at build time)."""
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import nz_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
needs_ref = pytest.mark.skipif(not os.path.exists(HARNESS), reason="oracle/_ref/ref_harness not built")


def emax(x, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(x, np.float64) - ref)) / np.max(np.abs(ref)))


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


@needs_ref
@pytest.mark.parametrize("sa,sb,dist", [((1, 1, 1024, 1024), (1, 1, 1024, 1024), "uniform"),
                                        ((1, 1, 127, 131), (1, 1, 131, 129), "uniform"),
                                        ((2, 1, 300, 200), (1, 3, 200, 150), "normal"),
                                        ((1, 1, 1, 4096), (1, 1, 4096, 512), "uniform")])
def test_forward_against_reference(tmp_path, sa, sb, dist):
    import neuzephyr_b200 as nz
    rng = np.random.default_rng(0 if sa[2] == 1024 else sum(sa))
    gen = (lambda s: rng.uniform(-1, 1, s)) if dist == "uniform" else (lambda s: rng.normal(0, 1, s))
    A, B = gen(sa).astype(np.float32), gen(sb).astype(np.float32)
    fa, fb, fc = [str(tmp_path / n) for n in ("A.bin", "B.bin", "C.bin")]
    A.tofile(fa)
    B.tofile(fb)
    r = subprocess.run([HARNESS, "gemm_file", fa, fb, fc] + [str(v) for v in sa] + [str(sb[0]), str(sb[1]), str(sb[3])],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1000:]
    sc = (max(sa[0], sb[0]), max(sa[1], sb[1]), sa[2], sb[3])
    c_ref = np.fromfile(fc, dtype=np.float32).reshape(sc)
    c_ours = nz.tensorcore_gemm(dev(A), dev(B)).cpu().numpy()
    truth = O.gemm_forward(A, B, round_operands=False, f64=True)
    e_ref, e_ours = emax(c_ref, truth), emax(c_ours, truth)
    assert e_ours <= 1e-2
    assert e_ours <= 2 * e_ref + 1e-7, (e_ours, e_ref)
    # the two implementations round the same operands the same way: they agree far below the fp16 error
    assert emax(c_ours, c_ref) <= 5e-5


@needs_ref
def test_backward_against_reference(tmp_path):
    import neuzephyr_b200 as nz
    rng = np.random.default_rng(5)
    sa, sb, sc = (3, 2, 64, 90), (3, 2, 90, 40), (1, 2, 64, 40)  # summed over N
    A, B = rng.normal(0, 1, sa).astype(np.float32), rng.normal(0, 1, sb).astype(np.float32)
    C0 = rng.normal(0, 1, sc).astype(np.float32)
    fa, fb, fc = [str(tmp_path / n) for n in ("A.bin", "B.bin", "C.bin")]
    A.tofile(fa)
    B.tofile(fb)
    C0.tofile(fc)
    r = subprocess.run([HARNESS, "gemm_bwd", fa, fb, fc] + [str(v) for v in sa] + [str(sb[0]), str(sb[1]), str(sb[3]),
                                                                                   str(sc[0]), str(sc[1])],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1000:]
    c_ref = np.fromfile(fc, dtype=np.float32).reshape(sc)
    out = dev(C0)
    nz.gemm_backward(dev(A), dev(B), out)
    truth = C0.astype(np.float64)
    O.gemm_backward(A, B, truth, round_operands=False)
    e_ref, e_ours = emax(c_ref, truth), emax(out.cpu().numpy(), truth)
    assert e_ours <= 1e-2 and e_ours <= 2 * e_ref + 1e-7, (e_ours, e_ref)
