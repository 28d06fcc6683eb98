"""Torch-tensor conveniences over the C ABI (device memory and the current stream come
from torch; every computation is a libnzb kernel). Used by the tests and the benchmark."""
import ctypes

import torch

from . import _capi as C

_ws_cache = {}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _workspace(nbytes, device):
    """Grow-only scratch buffer per device (stream-ordered reuse on torch's current stream)."""
    buf = _ws_cache.get(device)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _ws_cache[device] = buf
    return buf


def _check_f32_cuda(*ts):
    for t in ts:
        if t is None:
            continue
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
            raise ValueError("expected contiguous float32 CUDA tensors")


def gemm_workspace_bytes(desc):
    n = ctypes.c_size_t(0)
    C.check(C.lib().nzb_gemm_workspace_bytes(ctypes.byref(desc), ctypes.byref(n)))
    return n.value


def gemm(A, B, out=None, transA=False, transB=False, bias=None, bias_mode=C.BIAS_NONE, relu=False,
         accumulate=False):
    """C = op(A) @ op(B) for 2-D row-major float32 tensors through nzb_gemm."""
    _check_f32_cuda(A, B, bias, out)
    M, K = (A.shape[1], A.shape[0]) if transA else A.shape
    K2, N = (B.shape[1], B.shape[0]) if transB else B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=A.device)
    d = C.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.lda, d.ldb, d.ldc = A.shape[1], B.shape[1], N
    d.transA, d.transB = int(transA), int(transB)
    d.batch[0] = d.batch[1] = 1
    d.accumulate, d.relu = int(accumulate), int(relu)
    d.bias_mode = bias_mode if bias is not None else C.BIAS_NONE
    d.bias_ld = N
    ws = _workspace(gemm_workspace_bytes(d), A.device)
    C.check(C.lib().nzb_gemm(ctypes.byref(d), _ptr(A), _ptr(B), _ptr(out), _ptr(bias), _ptr(ws), ws.numel(),
                             _stream()))
    return out


def gemm_host(hA, hB, hC=None, transB=False, bias=None, bias_mode=C.BIAS_NONE, relu=False, device=None):
    """C = A @ op(B) with A, B, C (and bias) in host memory (pinned for overlap) through nzb_gemm_host:
    copies in, staging + GEMM per row block, and copies out are pipelined on three streams. The call
    is asynchronous on torch's current stream; synchronise it before reading hC."""
    for t in (hA, hB, hC, bias):
        if t is not None and (t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous()):
            raise ValueError("expected contiguous float32 host tensors")
    device = device or torch.device("cuda", torch.cuda.current_device())
    M, K = hA.shape
    K2, N = (hB.shape[1], hB.shape[0]) if transB else hB.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if hC is None:
        hC = torch.empty((M, N), dtype=torch.float32).pin_memory()
    d = C.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.lda, d.ldb, d.ldc = hA.shape[1], hB.shape[1], N
    d.transA, d.transB = 0, int(transB)
    d.batch[0] = d.batch[1] = 1
    d.relu = int(relu)
    d.bias_mode = bias_mode if bias is not None else C.BIAS_NONE
    d.bias_ld = N
    n = ctypes.c_size_t(0)
    C.check(C.lib().nzb_gemm_host_workspace_bytes(ctypes.byref(d), ctypes.byref(n)))
    ws = _workspace(n.value, device)
    C.check(C.lib().nzb_gemm_host(ctypes.byref(d), _ptr(hA), _ptr(hB), _ptr(hC), _ptr(bias), _ptr(ws), ws.numel(),
                                  _stream()))
    return hC


def gemm_f16(A16, B16, M, N, K, out=None, bias=None, bias_mode=C.BIAS_NONE, relu=False, accumulate=False):
    """GEMM on pre-staged K-major fp16 operands A16 [M][ldk], B16 [N][ldk] (nzb_gemm_f16)."""
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=A16.device)
    d = C.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.ldc = N
    d.batch[0] = d.batch[1] = 1
    d.accumulate, d.relu = int(accumulate), int(relu)
    d.bias_mode = bias_mode if bias is not None else C.BIAS_NONE
    d.bias_ld = N
    C.check(C.lib().nzb_gemm_f16(ctypes.byref(d), _ptr(A16), _ptr(B16), A16.shape[1], _ptr(out), _ptr(bias),
                                 _stream()))
    return out


def _ws4(A, B, Cs):
    n = ctypes.c_size_t(0)
    C.check(C.lib().nzb_tensorcore_gemm_workspace_bytes(C.shape4(A.shape), C.shape4(B.shape), C.shape4(Cs),
                                                        ctypes.byref(n)))
    return n.value


def tensorcore_gemm(A, B, out=None):
    """4-D batched forward GEMM with N/C broadcast (the iTensorCoreGEMM seam)."""
    _check_f32_cuda(A, B, out)
    sc = (max(A.shape[0], B.shape[0]), max(A.shape[1], B.shape[1]), A.shape[2], B.shape[3])
    if out is None:
        out = torch.empty(sc, dtype=torch.float32, device=A.device)
    ws = _workspace(_ws4(A, B, out.shape), A.device)
    C.check(C.lib().nzb_tensorcore_gemm(_ptr(A), _ptr(B), _ptr(out), C.shape4(A.shape), C.shape4(B.shape),
                                        C.shape4(out.shape), _ptr(ws), ws.numel(), _stream()))
    return out


def matmul_f32(A, B, out=None):
    """4-D batched product with N/C broadcast at fp32 accuracy (the Tensor::operator* seam, nzb_matmul_f32)."""
    _check_f32_cuda(A, B, out)
    sc = (max(A.shape[0], B.shape[0]), max(A.shape[1], B.shape[1]), A.shape[2], B.shape[3])
    if out is None:
        out = torch.empty(sc, dtype=torch.float32, device=A.device)
    n = ctypes.c_size_t(0)
    C.check(C.lib().nzb_matmul_f32_workspace_bytes(C.shape4(A.shape), C.shape4(B.shape), C.shape4(out.shape),
                                                   ctypes.byref(n)))
    ws = _workspace(n.value, A.device)
    C.check(C.lib().nzb_matmul_f32(_ptr(A), _ptr(B), _ptr(out), C.shape4(A.shape), C.shape4(B.shape),
                                   C.shape4(out.shape), _ptr(ws), ws.numel(), _stream()))
    return out


def gemm_backward(A, B, out):
    """out += A @ B reduced over broadcast batch dims of out (the iGEMMBackward seam)."""
    _check_f32_cuda(A, B, out)
    ws = _workspace(_ws4(A, B, out.shape), A.device)
    C.check(C.lib().nzb_gemm_backward(_ptr(A), _ptr(B), _ptr(out), C.shape4(A.shape), C.shape4(B.shape),
                                      C.shape4(out.shape), _ptr(ws), ws.numel(), _stream()))
    return out


def cast_f32_f16(x, transpose=False):
    """Returns the [rows][ld_out] fp16 operand copy of a 2-D float32 tensor."""
    _check_f32_cuda(x)
    rows, cols = (x.shape[1], x.shape[0]) if transpose else x.shape
    ld_out = (cols + 63) // 64 * 64
    out = torch.empty((rows, ld_out), dtype=torch.float16, device=x.device)
    C.check(C.lib().nzb_cast_f32_f16(_ptr(x), _ptr(out), rows, cols, x.shape[1], ld_out, int(transpose), _stream()))
    return out


def device_status():
    return C.device_status()


def _conv_desc(x_shape, w_shape, Kh, Kw, stride, pad, bias_mode=C.BIAS_NONE, relu=False, accumulate=False):
    d = C.ConvDesc()
    d.N, d.C, d.H, d.W = [int(v) for v in x_shape]
    d.Cout, d.Kh, d.Kw, d.stride, d.pad = int(w_shape[3]), Kh, Kw, stride, pad
    d.weights_per_sample = int(w_shape[0] > 1)
    d.bias_mode, d.relu, d.accumulate = bias_mode, int(relu), int(accumulate)
    return d


def _conv_ws(d, device):
    n = ctypes.c_size_t(0)
    C.check(C.lib().nzb_conv2d_workspace_bytes(ctypes.byref(d), ctypes.byref(n)))
    return _workspace(n.value, device)


def conv2d_forward(x, w, bias, Kh, Kw, stride, pad, relu=False, bias_mode=None, out=None, accumulate=False):
    """y = conv(x, w) (+ bias) (ReLU); x {N,C,H,W}, w {wN,1,C*Kh*Kw,Cout}, bias {1,1,Ho*Wo,Cout} or [Cout].
    accumulate=True adds the result (before ReLU) to the values already in `out`."""
    _check_f32_cuda(x, w, bias, out)
    if bias_mode is None:
        bias_mode = C.BIAS_NONE if bias is None else (C.BIAS_ROW if bias.dim() == 1 else C.BIAS_MATRIX)
    d = _conv_desc(x.shape, w.shape, Kh, Kw, stride, pad, bias_mode, relu, accumulate)
    Ho, Wo = (d.H + 2 * pad - Kh) // stride + 1, (d.W + 2 * pad - Kw) // stride + 1
    if out is None:
        out = torch.empty((d.N, d.Cout, Ho, Wo), dtype=torch.float32, device=x.device)
    ws = _conv_ws(d, x.device)
    C.check(C.lib().nzb_conv2d_forward(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _ptr(ws),
                                       ws.numel(), _stream()))
    return out


def conv2d_backward_data(dy, w, x_shape, Kh, Kw, stride, pad, dx):
    """dx += d(conv)/dx (stride 1)."""
    _check_f32_cuda(dy, w, dx)
    d = _conv_desc(x_shape, w.shape, Kh, Kw, stride, pad)
    ws = _conv_ws(d, dy.device)
    C.check(C.lib().nzb_conv2d_backward_data(ctypes.byref(d), _ptr(dy), _ptr(w), _ptr(dx), _ptr(ws), ws.numel(),
                                             _stream()))
    return dx


def conv2d_backward_weight(x, dy, w_shape, Kh, Kw, stride, pad, dw):
    """dw += d(conv)/dw, summed over the batch for shared weights."""
    _check_f32_cuda(x, dy, dw)
    d = _conv_desc(x.shape, w_shape, Kh, Kw, stride, pad)
    ws = _conv_ws(d, x.device)
    C.check(C.lib().nzb_conv2d_backward_weight(ctypes.byref(d), _ptr(x), _ptr(dy), _ptr(dw), _ptr(ws), ws.numel(),
                                               _stream()))
    return dw


def conv2d_backward_bias(dy, x_shape, w_shape, Kh, Kw, stride, pad, dbias):
    _check_f32_cuda(dy, dbias)
    d = _conv_desc(x_shape, w_shape, Kh, Kw, stride, pad)
    C.check(C.lib().nzb_conv2d_backward_bias(ctypes.byref(d), _ptr(dy), _ptr(dbias), _stream()))
    return dbias


def conv2d_backward(x, w, dy, Kh, Kw, stride, pad, dx=None, dw=None, dbias=None, y=None, overwrite_dx=False):
    """The whole backward of one layer through nzb_conv2d_backward (dY read once): accumulates into the
    given dx / dw / dbias ({1,1,Ho*Wo,Cout}); y, when given, is the forward output whose sign masks dY
    (a layer with a fused ReLU). Raises for shapes the one-pass form does not take."""
    _check_f32_cuda(x, w, dy, dx, dw, dbias, y)
    d = _conv_desc(x.shape, w.shape, Kh, Kw, stride, pad)
    d.bias_mode = C.BIAS_MATRIX if dbias is not None else C.BIAS_NONE
    d.relu = int(y is not None)
    d.overwrite_dx = int(overwrite_dx)
    n = ctypes.c_size_t(0)
    C.check(C.lib().nzb_conv2d_backward_workspace_bytes(ctypes.byref(d), ctypes.byref(n)))
    ws = _workspace(n.value, x.device)
    C.check(C.lib().nzb_conv2d_backward(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(y), _ptr(dy), _ptr(dx), _ptr(dw),
                                        _ptr(dbias), _ptr(ws), ws.numel(), _stream()))


def _linear_desc(batch, fin, fout, relu):
    d = C.LinearDesc()
    d.batch, d.in_features, d.out_features, d.relu = batch, fin, fout, int(relu)
    return d


def _linear_ws(d, device):
    n = ctypes.c_size_t(0)
    C.check(C.lib().nzb_linear_workspace_bytes(ctypes.byref(d), ctypes.byref(n)))
    return _workspace(n.value, device)


def linear_forward(x, w, bias=None, relu=False, out=None):
    """y[b][o] = relu(sum_i w[o][i] x[b][i] + bias[o]); x {B,in}, w {out,in}."""
    _check_f32_cuda(x, w, bias, out)
    d = _linear_desc(x.shape[0], x.shape[1], w.shape[0], relu)
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
    ws = _linear_ws(d, x.device)
    C.check(C.lib().nzb_linear_forward(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _ptr(ws),
                                       ws.numel(), _stream()))
    return out


def linear_backward(x, w, y, dy, dx=None, dw=None, dbias=None, relu=False, overwrite_dx=False):
    """dx += dy' w (dx = ... with overwrite_dx), dw += dy'^T x, dbias += colsum(dy'), dy' = dy * (y > 0) if relu."""
    _check_f32_cuda(x, w, y, dy, dx, dw, dbias)
    d = _linear_desc(x.shape[0], x.shape[1], w.shape[0], relu)
    d.overwrite_dx = int(overwrite_dx)
    ws = _linear_ws(d, x.device)
    C.check(C.lib().nzb_linear_backward(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(y), _ptr(dy), _ptr(dx), _ptr(dw),
                                        _ptr(dbias), _ptr(ws), ws.numel(), _stream()))
