"""One (and two) full training steps of the segmentation model -- conv -> ReLU -> conv -> avg-pool ->
linear -> softmax -> BCE -> Adam -- on the sm_100a host layer (neuzephyr_b200/bin/seg_model step_file),
compared on the same injected inputs and parameters with

  * oracle/model_step.py in its rounded mode (what the reference computes up to summation order) and in
    exact float64 (the error budget), and
  * NeuZephyr itself rebuilt for sm_100 (oracle/_ref/ref_harness model_file), which builds the same
    node sequence Model's builders create and runs ComputeGraph::forward/backward/update + zeroGrad.

(The reference's backward is only partly defined for this model, see test_step_against_reference.)
Acceptance per gradient tensor: e_max = max|g - g64| / max|g64| <= max(1e-2, 2 * e_max(the rounded oracle))
and <= 2 * e_max(reference) -- gradients reaching the first layers are 1e-5 and smaller, inside fp16's
subnormal range, so the reference's own arithmetic (fp16 GEMM operands, no loss scaling) already loses
more than 1e-2 there;
parameters after Adam (per-call time steps, default configuration) within 1e-4 of the rounded oracle
wherever the gradient is not within rounding noise of zero. The reference's bias gradient is a racy
`+=` over batch slices (src/Nodes.cu:106-121): with more than one sample every element of its db
must be the sum over SOME subset of the samples, and is reported separately.
"""
import json
import os
import subprocess

import numpy as np
import pytest

from oracle import model_step as MS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
needs_ref = pytest.mark.skipif(not os.path.exists(HARNESS), reason="oracle/_ref/ref_harness not built")
NAMES = ["conv1.w", "conv1.b", "conv2.w", "conv2.b", "linear.w", "linear.b"]


def _tool():
    from neuzephyr_b200 import build as B
    B.build()
    return [t for t in B.build_tools() if t.endswith("seg_model")][0]


def _case(tmp, N, S, per_sample, seed):
    rng = np.random.default_rng(seed)
    hp = (S - 5) // 2 + 1
    x = rng.normal(0, 1, (N, 3, S, S)).astype(np.float32)
    t = (rng.uniform(0, 1, (N, 1, 16, 1)) < 0.5).astype(np.float32)
    wn = N if per_sample else 1
    bound = lambda fan: (6.0 / fan) ** 0.5  # Kaiming-uniform
    params = [rng.uniform(-bound(27), bound(27), (wn, 1, 27, 16)), rng.uniform(-0.1, 0.1, (1, 1, S * S, 16)),
              rng.uniform(-bound(144), bound(144), (wn, 1, 144, 16)), rng.uniform(-0.1, 0.1, (1, 1, S * S, 16)),
              rng.uniform(-bound(16 * hp * hp), bound(16 * hp * hp), (1, 1, 16, 16 * hp * hp)),
              rng.uniform(-0.1, 0.1, (1, 1, 16, 1))]
    params = [p.astype(np.float32) for p in params]
    x.tofile(str(tmp / "x.bin"))
    t.tofile(str(tmp / "t.bin"))
    for i, p in enumerate(params):
        p.tofile(str(tmp / ("p%d.bin" % i)))
    return x, t, params


def _load(tmp, prefix, params, steps):
    g = [np.fromfile(str(tmp / ("%sg%d.bin" % (prefix, i))), dtype=np.float32).reshape(p.shape)
         for i, p in enumerate(params)]
    q = [[np.fromfile(str(tmp / ("%sq%d_%d.bin" % (prefix, s, i))), dtype=np.float32).reshape(p.shape)
          for i, p in enumerate(params)] for s in range(steps)]
    losses = [float(v) for v in open(str(tmp / ("%sloss.txt" % prefix))).read().split()]
    return g, q, losses


def emax(a, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(a, np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-30))


def _param_diff(q, q_ref, g_ref):
    """Largest parameter difference where the gradient is clear of rounding noise around zero (there
    Adam's g / (|g| + eps) turns noise into a step of up to lr)."""
    gmax = np.max(np.abs(g_ref))
    mask = np.abs(g_ref) > 1e-2 * gmax
    return float(np.max(np.abs(q - q_ref)[mask])) if mask.any() else 0.0


@pytest.mark.parametrize("N,S,per_sample", [(2, 32, False), (3, 20, True)])
def test_two_steps_against_oracle(tmp_path, N, S, per_sample):
    x, t, params = _case(tmp_path, N, S, per_sample, 100 + N)
    # a learning rate that keeps the second step's softmax away from saturation (at 0.01 one update moves
    # a logit by several units through the linear layer's thousands of inputs)
    lr = 1e-3
    r = subprocess.run([_tool(), "step_file", str(tmp_path), str(N), str(S), "2", "0" if per_sample else "1", str(lr)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    g, q, losses = _load(tmp_path, "", params, 2)
    o_losses, o_g, o_q = MS.seg_model_steps(x, t, params, 2, lr=lr)
    x_loss, x_g = MS.seg_model_gradients(x, t, params, exact=True)
    assert abs(losses[0] - o_losses[0]) <= 2e-5 * abs(o_losses[0])
    assert abs(losses[0] - x_loss) <= 1e-3 * abs(x_loss)
    # the loss node accumulates over steps (src/Nodes.cu:822-840)
    assert abs(losses[1] - (o_losses[0] + o_losses[1])) <= 1e-4 * abs(o_losses[0] + o_losses[1])
    report = {}
    for i, name in enumerate(NAMES):
        e_r, e_x, e_alg = emax(g[i], o_g[i]), emax(g[i], x_g[i]), emax(o_g[i], x_g[i])
        report[name] = (e_r, e_x, e_alg)
        # same rounding points; fp32 summation order differs and flips fp16 roundings downstream
        assert e_r <= max(2e-3, e_alg), (name, e_r, e_alg)
        # against the unrounded fp64 step: the contract's bound, or what the algorithm itself loses
        assert e_x <= max(1e-2, 2 * e_alg), (name, e_x, e_alg)
        for s in range(2):
            d = _param_diff(q[s][i], o_q[s][i], o_g[i])
            assert d <= 1e-2 * lr, (name, s, d)  # a hundredth of one Adam step
    print(json.dumps(report))


@needs_ref
@pytest.mark.parametrize("N,S,shared", [(1, 32, False), (2, 24, False), (2, 24, True)])
def test_step_against_reference(tmp_path, N, S, shared):
    """A/B with NeuZephyr: same inputs, same injected parameters, one training step each.

    What can be compared is bounded by a defect of the reference: its transpose launches a grid that
    covers the whole matrix only when both extents span equally many 32-wide tiles
    (src/TensorOperations.cu:122-126 against src/OperationKernels.cu:125-146), and MatMulNode::backward
    transposes both operands (src/Nodes.cu:169-182). In this model only the loss, the linear layer's bias
    gradient and the first 32 input columns of the linear layer's weight gradient are therefore defined in
    the reference (x^T of an {in, 1} vector is transposed for its first 32 rows only; everything upstream
    goes through W^T, of which only 32 columns exist). Those are compared, together with the
    parameters they update: the linear bias is the LAST parameter the reference's optimizer steps, so its
    update checks the per-call Adam time step (t = 17, after every earlier node's tick) end to end."""
    x, t, params = _case(tmp_path, N, S, not shared, 200 + 7 * N + int(shared))
    r = subprocess.run([_tool(), "step_file", str(tmp_path), str(N), str(S), "1", "1" if shared else "0"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    r = subprocess.run([HARNESS, "model_file", str(tmp_path), str(N), str(S), "1", "1" if shared else "0"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    g, q, losses = _load(tmp_path, "", params, 1)
    rg, rq, rlosses = _load(tmp_path, "ref_", params, 1)
    x_loss, x_g = MS.seg_model_gradients(x, t, params, exact=True)
    assert abs(losses[0] - rlosses[0]) <= 1e-4 * abs(rlosses[0])
    assert abs(losses[0] - x_loss) <= 1e-3 * abs(x_loss)
    report = {}
    for i, cols in ((4, 32), (5, None)):  # linear.w (first 32 input columns), linear.b
        sl = (Ellipsis, slice(0, cols)) if cols else Ellipsis
        ours, ref, truth = g[i][sl], rg[i][sl], x_g[i][sl]
        den = np.max(np.abs(x_g[i]))
        e_ours = float(np.max(np.abs(ours - truth)) / den)
        e_ref = float(np.max(np.abs(ref - truth)) / den)
        report[NAMES[i]] = {"e_ours": e_ours, "e_ref": e_ref}
        if i == 5 and N > 1:
            # the racy bias gradient (see the module docstring): report how often every term survived
            report[NAMES[i]]["ref_full_sum_fraction"] = float(np.mean(np.abs(ref - ours) <= 1e-3 * den))
            continue
        assert e_ours <= max(1e-2, 2 * e_ref) and e_ours <= 2 * e_ref + 1e-6, (NAMES[i], e_ours, e_ref)
        assert float(np.max(np.abs(ours - ref)) / den) <= max(2e-3, e_ref), NAMES[i]
        # parameters after the update: both sides use the per-call Adam time steps (t = 15 and t = 17)
        gmax = np.max(np.abs(truth))
        mask = np.abs(truth) > 1e-2 * gmax
        d = float(np.max(np.abs(q[0][i][sl] - rq[0][i][sl])[mask]))
        assert d <= 1e-4, (NAMES[i], d)
        # and a wrong time step would show: t = 1 instead of 17 moves a weight 1.8 times as far
        moved = float(np.max(np.abs(q[0][i][sl] - params[i][sl])[mask]))
        assert moved > 3e-3, moved
    print(json.dumps(report))
