"""Host restatement of one training step of the benchmark's segmentation model as NeuZephyr's
Model builders compose it (TEST INFRASTRUCTURE ONLY -- imported by tests/, never by the product):

    x {N,3,S,S} -> Conv2d(3->16,3x3,s1,p1) -> ReLU -> Conv2d(16->16,3x3,s1,p1) -> AvgPool2d(5,2)
      -> Linear(->16) -> Softmax -> BCE(target {N,1,16,1});  Adam(lr, b1, b2, eps 1e-6)

Reference sources followed, op by op:
  Model::Conv2d  = Img2Col -> MatMul(col, W) -> Add(bias {1,1,Ho*Wo,Cout}) -> Col2Img   src/Model.cu:244-263
                   (img2colKernel src/OperationKernels.cu:1308-1328, col2imgKernel :1364-1376)
  ReLU           src/OperationKernels.cu:230-253 (backward masks on the node's INPUT > 0)
  AvgPool2d      src/OperationKernels.cu:1404-1482 (no padding: backward divides by pool*pool)
  Model::Linear  = Reshape -> MatMul(W {1,1,out,in}, x {N,1,in,1}) -> Add(bias {1,1,out,1})   src/Model.cu:87-103
  Softmax        src/OperationKernels.cu:477-523; backward = J(y) * dY through the tensor-core GEMM,
                 src/Nodes.cu:538-548 (so J and dY are rounded to fp16)
  BCE            src/OperationKernels.cu:648-704 (mean over all N*16 elements)
  MatMul forward / backward: fp16-rounded operands, wide accumulation (src/OperationKernels.cu:821-883,
                 src/Nodes.cu:165-182); a shared weight's gradient is summed over the batch (:1121-1137)
  Adam           src/OperationKernels.cu:753-766, one time step PER step() CALL (src/Optimizer.cu:86-102):
                 ComputeGraph::update (src/ComputeGraph.cu:541-547) steps every gradient-requiring node in
                 insertion order, activations included, so the parameters of this model see
                 t = 1, 3, 7, 10, 15, 17 in the first update and 20 more in each later one (REF_T).

Two modes: `exact=False` keeps fp32 storage between operations and rounds GEMM operands to fp16
(what the reference and the sm_100a path compute, up to accumulation order); `exact=True` is the
same algebra in float64 with no rounding anywhere (ground truth for error budgets).
"""
import numpy as np

from . import nz_oracle as O

# Adam time step each parameter (w1, b1, w2, b2, wl, bl) sees in the first Model::update, and the
# number of step() calls per update, from the node insertion order of the builders (see above).
REF_T = (1, 3, 7, 10, 15, 17)
REF_T_PER_UPDATE = 20


def _img2col_index(C, H, W, k, pad):
    """Index arrays of the im2col gather: col[p, c*k*k + kh*k + kw] = xpad[c, oh+kh, ow+kw]."""
    Ho, Wo = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    oh, ow = np.meshgrid(np.arange(Ho), np.arange(Wo), indexing="ij")
    c, kh, kw = np.meshgrid(np.arange(C), np.arange(k), np.arange(k), indexing="ij")
    ci = np.broadcast_to(c.reshape(1, -1), (Ho * Wo, C * k * k))
    hi = oh.reshape(-1, 1) + kh.reshape(1, -1)
    wi = ow.reshape(-1, 1) + kw.reshape(1, -1)
    return ci, hi, wi, Ho, Wo


class _Conv:
    """Img2Col -> MatMul -> Add -> Col2Img of one layer, forward and backward."""

    def __init__(self, shape, k, pad, cout, rnd, dt):
        self.N, self.C, self.H, self.W = shape
        self.k, self.pad, self.cout, self.rnd, self.dt = k, pad, cout, rnd, dt
        self.ci, self.hi, self.wi, self.Ho, self.Wo = _img2col_index(self.C, self.H, self.W, k, pad)

    def forward(self, x, w, b):
        p = self.pad
        xp = np.pad(x, ((0, 0), (0, 0), (p, p), (p, p)))
        self.col = xp[:, self.ci, self.hi, self.wi]  # {N, P, K}
        wn = w.reshape(-1, self.C * self.k * self.k, self.cout)
        mm = np.einsum("npk,nkc->npc", self.rnd(self.col).astype(np.float64),
                       np.broadcast_to(self.rnd(wn).astype(np.float64), (self.N,) + wn.shape[1:]))
        mm = mm.astype(self.dt)
        a = (mm + b.reshape(1, self.Ho * self.Wo, self.cout)).astype(self.dt)
        return np.ascontiguousarray(a.transpose(0, 2, 1)).reshape(self.N, self.cout, self.Ho, self.Wo)

    def backward(self, dy, w, want_dx):
        da = dy.reshape(self.N, self.cout, self.Ho * self.Wo).transpose(0, 2, 1)  # {N, P, Cout}
        db = da.astype(np.float64).sum(axis=0).astype(self.dt).reshape(1, 1, self.Ho * self.Wo, self.cout)
        wn = w.reshape(-1, self.C * self.k * self.k, self.cout)
        per_sample = wn.shape[0] > 1
        dwn = np.einsum("npk,npc->nkc", self.rnd(self.col).astype(np.float64), self.rnd(da).astype(np.float64))
        dw = (dwn if per_sample else dwn.sum(axis=0, keepdims=True)).astype(self.dt).reshape(w.shape)
        dx = None
        if want_dx:
            dcol = np.einsum("npc,nkc->npk", self.rnd(da).astype(np.float64),
                             np.broadcast_to(self.rnd(wn).astype(np.float64), (self.N,) + wn.shape[1:]))
            dcol = dcol.astype(self.dt)
            p = self.pad
            dxp = np.zeros((self.N, self.C, self.H + 2 * p, self.W + 2 * p), dtype=np.float64)
            for n in range(self.N):
                np.add.at(dxp[n], (self.ci, self.hi, self.wi), dcol[n])
            dx = dxp[:, :, p:p + self.H, p:p + self.W].astype(self.dt)
        return dx, dw, db


def _avgpool(x, pool, stride):
    N, C, H, W = x.shape
    Ho, Wo = (H - pool) // stride + 1, (W - pool) // stride + 1
    acc = np.zeros((N, C, Ho, Wo), dtype=np.float64)
    for i in range(pool):
        for j in range(pool):
            acc += x[:, :, i:i + stride * Ho:stride, j:j + stride * Wo:stride]
    return (acc / (pool * pool)).astype(x.dtype)


def _avgpool_backward(g, xshape, pool, stride):
    N, C, H, W = xshape
    Ho, Wo = g.shape[2], g.shape[3]
    out = np.zeros(xshape, dtype=np.float64)
    gg = (g / g.dtype.type(pool * pool)).astype(np.float64)
    for i in range(pool):
        for j in range(pool):
            out[:, :, i:i + stride * Ho:stride, j:j + stride * Wo:stride] += gg
    return out.astype(g.dtype)


def adam_step(p, m, v, g, lr, b1, b2, eps, t):
    """In-place Adam update of float arrays (AdamKernel); returns nothing."""
    dt = p.dtype
    m[...] = (m * dt.type(b1) + g * dt.type(1 - b1)).astype(dt)
    v[...] = (v * dt.type(b2) + g * g * dt.type(1 - b2)).astype(dt)
    c1, c2 = 1.0 - float(b1) ** t, 1.0 - float(b2) ** t
    p[...] = (p - lr * (m.astype(np.float64) / c1) / (np.sqrt(v.astype(np.float64) / c2) + eps)).astype(dt)


def seg_model_gradients(x, target, params, exact=False):
    """One forward + backward. params = [w1, b1, w2, b2, wl, bl] with the reference's shapes
    (w {1|N,1,C*9,16}, b {1,1,S*S,16}, wl {1,1,16,in}, bl {1,1,16,1}). Returns (loss, [grads]) ."""
    dt = np.float64 if exact else np.float32
    rnd = (lambda a: a) if exact else (lambda a: O.round_f16(np.ascontiguousarray(a, dtype=np.float32)))
    x = np.asarray(x, dtype=dt)
    w1, b1, w2, b2, wl, bl = [np.asarray(p, dtype=dt) for p in params]
    N, _, S, _ = x.shape
    c1 = _Conv(x.shape, 3, 1, 16, rnd, dt)
    y1 = c1.forward(x, w1, b1)
    r1 = np.maximum(y1, 0)
    c2 = _Conv(r1.shape, 3, 1, 16, rnd, dt)
    y2 = c2.forward(r1, w2, b2)
    pl = _avgpool(y2, 5, 2)
    v = pl.reshape(N, -1)  # {N, in}
    W = wl.reshape(16, -1)
    z = (rnd(v).astype(np.float64) @ rnd(W).astype(np.float64).T).astype(dt) + bl.reshape(1, 16)
    z = z.astype(dt)
    e = np.exp(z.astype(np.float64))
    s = (e / e.sum(axis=1, keepdims=True)).astype(dt)
    tg = np.asarray(target, dtype=np.float64).reshape(N, 16)
    s64 = s.astype(np.float64)
    n_el = N * 16
    loss = float(np.sum(-tg * np.log(s64) - (1 - tg) * np.log(1 - s64)) / n_el)
    ds = (((s64 - tg) / (s64 * (1 - s64))) / n_el).astype(dt)
    # softmax backward: J(y) * dY, operands rounded like the reference's tensor-core product
    J = -s[:, :, None] * s[:, None, :]
    idx = np.arange(16)
    J[:, idx, idx] = s * (dt(1) - s)
    dz = np.einsum("nij,nj->ni", rnd(J).astype(np.float64), rnd(ds).astype(np.float64)).astype(dt)
    dbl = dz.astype(np.float64).sum(axis=0).astype(dt).reshape(bl.shape)
    dwl = (rnd(dz).astype(np.float64).T @ rnd(v).astype(np.float64)).astype(dt).reshape(wl.shape)
    dv = (rnd(dz).astype(np.float64) @ rnd(W).astype(np.float64)).astype(dt)
    dy2 = _avgpool_backward(dv.reshape(pl.shape), y2.shape, 5, 2)
    dr1, dw2, db2 = c2.backward(dy2, w2, True)
    dy1 = np.where(y1 > 0, dr1, dt(0)).astype(dt)
    _, dw1, db1 = c1.backward(dy1, w1, False)
    return loss, [dw1, db1, dw2, db2, dwl, dbl]


def seg_model_steps(x, target, params, steps, lr=0.01, b1=0.9, b2=0.999, eps=1e-6, exact=False, ts=REF_T,
                    t_per_update=REF_T_PER_UPDATE):
    """`steps` x (forward, backward, Adam update). Returns (losses, first-step gradients, parameters
    after each update). Parameter i uses time step ts[i] + step * t_per_update."""
    dt = np.float64 if exact else np.float32
    ps = [np.array(p, dtype=dt) for p in params]
    ms = [np.zeros_like(p) for p in ps]
    vs = [np.zeros_like(p) for p in ps]
    losses, first, after = [], None, []
    for s in range(steps):
        loss, gs = seg_model_gradients(x, target, ps, exact)
        losses.append(loss)
        if first is None:
            first = gs
        for i, (p, m, v, g) in enumerate(zip(ps, ms, vs, gs)):
            adam_step(p, m, v, g.astype(dt), lr, b1, b2, eps, ts[i] + s * t_per_update)
        after.append([p.copy() for p in ps])
    return losses, first, after
