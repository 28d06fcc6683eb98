"""ctypes/numpy binding of the host oracle (libnz_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's cpu_baseline / reference legs. The product package never imports it.
Each wrapper names the reference source its C function restates; see
nz_oracle.cpp for line-level citations.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnz_oracle.so")

_i64 = ctypes.c_int64
_f = ctypes.c_float
_int = ctypes.c_int
_vp = ctypes.c_void_p


def build(force=False):
    """Compile the C++ restatement with the host compiler."""
    src = os.path.join(_HERE, "nz_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libnz_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.nzo_bce.restype = ctypes.c_double
        _lib.nzo_num_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else _vp(a.ctypes.data)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _shape4(s):
    return (ctypes.c_int64 * 4)(*[int(v) for v in s])


def num_threads():
    return int(lib().nzo_num_threads())


def round_f16(x):
    """fp32 -> fp16 (round to nearest even) -> fp32, as Padding's __float2half (OperationKernels.cu:846-860)."""
    x = _f32(x)
    out = np.empty_like(x)
    lib().nzo_round_f16(_p(x), _p(out), _i64(x.size))
    return out


def f16_bits(x):
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().nzo_f32_to_f16_bits(_p(x), _p(out), _i64(x.size))
    return out


def gemm_f64(A, B, round_operands=True):
    """Ground truth C = A @ B in double, operands optionally rounded to fp16 first."""
    A, B = _f32(A), _f32(B)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    C = np.empty((M, N), dtype=np.float64)
    lib().nzo_gemm_f64(_p(A), _p(B), _p(C), _i64(M), _i64(N), _i64(K), _int(int(round_operands)))
    return C


def gemm_f64_rows(A, B, rows, round_operands=True):
    A, B = _f32(A), _f32(B)
    M, K = A.shape
    N = B.shape[1]
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    C = np.empty((rows.size, N), dtype=np.float64)
    lib().nzo_gemm_f64_rows(_p(A), _p(B), _p(C), _p(rows), _i64(rows.size), _i64(M), _i64(N), _i64(K),
                            _int(int(round_operands)))
    return C


def gemm_f32(A, B, round_operands=True):
    """Timed CPU baseline: fp32 accumulation, all host threads."""
    A, B = _f32(A), _f32(B)
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N), dtype=np.float32)
    lib().nzo_gemm_f32(_p(A), _p(B), _p(C), _i64(M), _i64(N), _i64(K), _int(int(round_operands)))
    return C


def _out_shape(sa, sb):
    return (max(sa[0], sb[0]), max(sa[1], sb[1]), sa[2], sb[3])


def gemm_forward(A, B, round_operands=True, f64=False):
    """Batched 4-D GEMM with N/C broadcast, overwrite (TensorCoreGEMMParallel, OperationKernels.cu:914-1026)."""
    A, B = _f32(A), _f32(B)
    sc = _out_shape(A.shape, B.shape)
    C = np.zeros(sc, dtype=np.float64 if f64 else np.float32)
    fn = lib().nzo_gemm_forward_f64 if f64 else lib().nzo_gemm_forward
    fn(_p(A), _p(B), _p(C), _shape4(A.shape), _shape4(B.shape), _shape4(sc), _int(int(round_operands)))
    return C


def gemm_backward(A, B, C, round_operands=True):
    """C += A @ B with batch reduction into broadcast dims of C (GEMMBackwardParallel, OperationKernels.cu:1028-1144).

    C is updated in place (float32 or float64 array of the target shape)."""
    A, B = _f32(A), _f32(B)
    assert C.flags["C_CONTIGUOUS"]
    fn = lib().nzo_gemm_backward_f64 if C.dtype == np.float64 else lib().nzo_gemm_backward
    assert C.dtype in (np.float32, np.float64)
    fn(_p(A), _p(B), _p(C), _shape4(A.shape), _shape4(B.shape), _shape4(C.shape), _int(int(round_operands)))
    return C


def transpose(x):
    x = _f32(x)
    n, c, h, w = x.shape
    out = np.empty((n, c, w, h), dtype=np.float32)
    lib().nzo_transpose(_p(x), _p(out), _i64(n * c), _i64(h), _i64(w))
    return out


def matmul_node_backward(A, B, dC, dA=None, dB=None, round_operands=True):
    """MatMulNode::backward (Nodes.cu:169-182): dA += dC @ B^T, dB += A^T @ dC, each reduced over broadcast dims."""
    if dA is not None:
        gemm_backward(dC, transpose(B), dA, round_operands)
    if dB is not None:
        gemm_backward(transpose(A), dC, dB, round_operands)
    return dA, dB


def conv_out_hw(H, W, Kh, Kw, stride, pad):
    return (H + 2 * pad - Kh) // stride + 1, (W + 2 * pad - Kw) // stride + 1


def img2col(x, Kh, Kw, stride, pad):
    """{N,C,H,W} -> {N,1,Ho*Wo,C*Kh*Kw} (img2colKernel, OperationKernels.cu:1308-1328)."""
    x = _f32(x)
    n, c, h, w = x.shape
    ho, wo = conv_out_hw(h, w, Kh, Kw, stride, pad)
    out = np.empty((n, 1, ho * wo, c * Kh * Kw), dtype=np.float32)
    lib().nzo_img2col(_p(out), _p(x), _i64(ho), _i64(wo), _i64(c), _i64(Kh), _i64(Kw), _i64(stride), _i64(pad),
                      _i64(h), _i64(w), _i64(n))
    return out


def img2col_backward(dcol, xshape, Kh, Kw, stride, pad, dx=None):
    dcol = _f32(dcol)
    n, c, h, w = xshape
    ho, wo = conv_out_hw(h, w, Kh, Kw, stride, pad)
    if dx is None:
        dx = np.zeros(xshape, dtype=np.float32)
    lib().nzo_img2col_backward(_p(dx), _p(dcol), _i64(ho), _i64(wo), _i64(c), _i64(Kh), _i64(Kw), _i64(stride),
                               _i64(pad), _i64(h), _i64(w), _i64(n))
    return dx


def col2img(x, Ho, Wo, Cout):
    """{N,1,Ho*Wo,Cout} -> {N,Cout,Ho,Wo} (col2imgKernel, OperationKernels.cu:1364-1376)."""
    x = _f32(x)
    n = x.shape[0]
    out = np.empty((n, Cout, Ho, Wo), dtype=np.float32)
    lib().nzo_col2img(_p(out), _p(x), _i64(Ho), _i64(Wo), _i64(Cout), _i64(n))
    return out


def col2img_backward(g):
    g = _f32(g)
    n, co, ho, wo = g.shape
    out = np.empty((n, 1, ho * wo, co), dtype=np.float32)
    lib().nzo_col2img_backward(_p(out), _p(g), _i64(ho), _i64(wo), _i64(co), _i64(n))
    return out


def add_broadcast(a, b):
    a, b = _f32(a), _f32(b)
    so = (max(a.shape[0], b.shape[0]), max(a.shape[1], b.shape[1]), a.shape[2], a.shape[3])
    out = np.empty(so, dtype=np.float32)
    lib().nzo_add_broadcast(_p(out), _p(a), _p(b), _shape4(a.shape), _shape4(b.shape))
    return out


def add_backward(gout, in_shape, gin=None):
    gout = _f32(gout)
    if gin is None:
        gin = np.zeros(in_shape, dtype=np.float32)
    lib().nzo_add_backward(_p(gin), _p(gout), _shape4(in_shape), _shape4(gout.shape))
    return gin


def relu(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().nzo_relu(_p(out), _p(x), _i64(x.size))
    return out


def relu_backward(x, gout):
    x, gout = _f32(x), _f32(gout)
    gin = np.empty_like(x)
    lib().nzo_relu_backward(_p(gin), _p(x), _p(gout), _i64(x.size))
    return gin


def avgpool(x, pool, stride, pad):
    x = _f32(x)
    n, c, h, w = x.shape
    ho, wo = (h + 2 * pad - pool) // stride + 1, (w + 2 * pad - pool) // stride + 1
    out = np.empty((n, c, ho, wo), dtype=np.float32)
    lib().nzo_avgpool(_p(out), _p(x), _i64(pool), _i64(stride), _i64(pad), _i64(n), _i64(c), _i64(h), _i64(w),
                      _i64(ho), _i64(wo))
    return out


def avgpool_backward(gout, xshape, pool, stride, pad, gin=None):
    gout = _f32(gout)
    n, c, h, w = xshape
    ho, wo = gout.shape[2], gout.shape[3]
    if gin is None:
        gin = np.zeros(xshape, dtype=np.float32)
    lib().nzo_avgpool_backward(_p(gin), _p(gout), _i64(pool), _i64(stride), _i64(pad), _i64(n), _i64(c), _i64(h),
                               _i64(w), _i64(ho), _i64(wo))
    return gin


def maxpool(x, pool, stride, pad):
    """(out, position) of MaxPoolingKernel (OperationKernels.cu:1507-1540)."""
    x = _f32(x)
    n, c, h, w = x.shape
    ho, wo = (h + 2 * pad - pool) // stride + 1, (w + 2 * pad - pool) // stride + 1
    out = np.empty((n, c, ho, wo), dtype=np.float32)
    pos = np.empty((n, c, ho, wo), dtype=np.float32)
    lib().nzo_maxpool(_p(out), _p(pos), _p(x), _i64(pool), _i64(stride), _i64(pad), _i64(n), _i64(c), _i64(h), _i64(w),
                      _i64(ho), _i64(wo))
    return out, pos


def maxpool_backward(gout, position, xshape, pool, stride, pad, gin=None):
    gout, position = _f32(gout), _f32(position)
    n, c, h, w = xshape
    if gin is None:
        gin = np.zeros(xshape, dtype=np.float32)
    lib().nzo_maxpool_backward(_p(gin), _p(position), _p(gout), _i64(pool), _i64(stride), _i64(pad), _i64(n), _i64(c),
                               _i64(h), _i64(w), _i64(gout.shape[2]), _i64(gout.shape[3]))
    return gin


def softmax(x):
    """Softmax over each {H,W} matrix of an {N,C,H,W} tensor."""
    x = _f32(x)
    n = x.shape[2] * x.shape[3]
    out = np.empty_like(x)
    lib().nzo_softmax(_p(out), _p(x), _i64(x.size // n), _i64(n))
    return out


def softmax_jacobian(y):
    y = _f32(y).reshape(-1)
    n = y.size
    out = np.empty((n, n), dtype=np.float32)
    lib().nzo_softmax_jacobian(_p(out), _p(y), _i64(1), _i64(n))
    return out


def softmax_backward(y, gout, round_operands=True):
    y, gout = _f32(y), _f32(gout)
    n = y.shape[2] * y.shape[3]
    gin = np.empty_like(y)
    lib().nzo_softmax_backward(_p(gin), _p(y), _p(gout), _i64(y.size // n), _i64(n), _int(int(round_operands)))
    return gin


def bce(p, t):
    p, t = _f32(p), _f32(t)
    return float(lib().nzo_bce(_p(p), _p(t), _i64(p.size)))


def bce_backward(p, t):
    p, t = _f32(p), _f32(t)
    out = np.empty_like(p)
    lib().nzo_bce_backward(_p(out), _p(p), _p(t), _i64(p.size))
    return out


def adam(data, m, v, grad, lr, beta1, beta2, eps, t):
    """In-place Adam step on float32 arrays (AdamKernel, OperationKernels.cu:753-766)."""
    for a in (data, m, v):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    grad = _f32(grad)
    lib().nzo_adam(_p(data), _p(m), _p(v), _p(grad), _f(lr), _f(beta1), _f(beta2), _f(eps), _int(t),
                   _i64(data.size))


def conv2d_forward(x, w, bias, Kh, Kw, stride, pad, round_operands=True, relu=False):
    """Model::Conv2d composition (Model.cu:244-263). w: {wN,1,C*Kh*Kw,Cout}; bias {1,1,Ho*Wo,Cout} or None."""
    x, w = _f32(x), _f32(w)
    n, c, h, ww = x.shape
    wn, cout = w.shape[0], w.shape[3]
    ho, wo = conv_out_hw(h, ww, Kh, Kw, stride, pad)
    y = np.empty((n, cout, ho, wo), dtype=np.float32)
    b = None if bias is None else _f32(bias)
    lib().nzo_conv2d_forward(_p(y), _p(x), _p(w), _p(b), _i64(n), _i64(c), _i64(h), _i64(ww), _i64(cout), _i64(Kh),
                             _i64(Kw), _i64(stride), _i64(pad), _i64(wn), _int(int(round_operands)),
                             _int(int(relu)))
    return y


def conv2d_backward(dy, x, w, Kh, Kw, stride, pad, want_dx=True, want_dw=True, want_db=True, round_operands=True):
    dy, x, w = _f32(dy), _f32(x), _f32(w)
    n, c, h, ww = x.shape
    wn, cout = w.shape[0], w.shape[3]
    ho, wo = dy.shape[2], dy.shape[3]
    dx = np.zeros_like(x) if want_dx else None
    dw = np.zeros_like(w) if want_dw else None
    db = np.zeros((1, 1, ho * wo, cout), dtype=np.float32) if want_db else None
    lib().nzo_conv2d_backward(_p(dx), _p(dw), _p(db), _p(dy), _p(x), _p(w), _i64(n), _i64(c), _i64(h), _i64(ww),
                              _i64(cout), _i64(Kh), _i64(Kw), _i64(stride), _i64(pad), _i64(wn),
                              _int(int(round_operands)))
    return dx, dw, db
