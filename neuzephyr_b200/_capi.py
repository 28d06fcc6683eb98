"""ctypes binding of libnzb.so (include/nzb.h). No torch types cross this boundary:
callers pass raw device addresses, sizes and a stream handle."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnzb.so")

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_NO_DEVICE = range(7)
BIAS_NONE, BIAS_ROW, BIAS_COL, BIAS_MATRIX = range(4)
STATIC_SCRATCH_BYTES = 32 << 20

EXPORTS = [
    "nzb_version", "nzb_last_error_string", "nzb_device_status", "nzb_device_status_reset", "nzb_selftest_wait_timeout",
    "nzb_gemm_workspace_bytes", "nzb_gemm", "nzb_gemm_kernel_launches", "nzb_gemm_f16", "nzb_gemm_static", "nzb_gemm_static_status", "nzb_gemm_static_status_reset", "nzb_gemm_host_workspace_bytes", "nzb_gemm_host", "nzb_tensorcore_gemm_workspace_bytes", "nzb_tensorcore_gemm",
    "nzb_gemm_backward", "nzb_matmul_f32_workspace_bytes", "nzb_matmul_f32", "nzb_cast_f32_f16",
    "nzb_linear_workspace_bytes", "nzb_linear_forward", "nzb_linear_backward",
    "nzb_conv2d_workspace_bytes", "nzb_conv2d_forward", "nzb_conv2d_backward_data", "nzb_conv2d_backward_weight",
    "nzb_conv2d_backward_bias", "nzb_conv2d_backward_workspace_bytes", "nzb_conv2d_backward",
    "nzb_img2col", "nzb_img2col_backward", "nzb_col2img", "nzb_col2img_backward", "nzb_add_broadcast",
    "nzb_add_backward", "nzb_relu", "nzb_relu_backward", "nzb_avgpool", "nzb_avgpool_backward", "nzb_avgpool_backward_ex", "nzb_softmax",
    "nzb_softmax_backward", "nzb_bce", "nzb_bce_backward", "nzb_adam", "nzb_adam_multi", "nzb_softmax_bce_forward",
    "nzb_softmax_bce_backward", "nzb_maxpool", "nzb_maxpool_backward", "nzb_fill", "nzb_expand", "nzb_scale",
]


class GemmDesc(ctypes.Structure):
    """struct nzb_gemm_desc"""
    _fields_ = [
        ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
        ("transA", ctypes.c_int32), ("transB", ctypes.c_int32),
        ("batch", ctypes.c_int32 * 2),
        ("strideA", ctypes.c_int64 * 2), ("strideB", ctypes.c_int64 * 2), ("strideC", ctypes.c_int64 * 2),
        ("accumulate", ctypes.c_int32), ("bias_mode", ctypes.c_int32),
        ("bias_ld", ctypes.c_int64),
        ("relu", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class ConvDesc(ctypes.Structure):
    """struct nzb_conv_desc"""
    _fields_ = [(n, ctypes.c_int64) for n in ("N", "C", "H", "W", "Cout", "Kh", "Kw", "stride", "pad")] + \
               [(n, ctypes.c_int32) for n in ("weights_per_sample", "bias_mode", "relu", "accumulate", "overwrite_dx",
                                              "reserved")]


class LinearDesc(ctypes.Structure):
    """struct nzb_linear_desc"""
    _fields_ = [("batch", ctypes.c_int64), ("in_features", ctypes.c_int64), ("out_features", ctypes.c_int64),
                ("relu", ctypes.c_int32), ("overwrite_dx", ctypes.c_int32)]


class AdamTensor(ctypes.Structure):
    """struct nzb_adam_tensor"""
    _fields_ = [("data", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p), ("grad", ctypes.c_void_p),
                ("shadow_f16", ctypes.c_void_p), ("n", ctypes.c_int64), ("t", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class NzbError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("nzb error %d: %s" % (code, msg))
        self.code = code


_lib = None


def lib():
    """Loads libnzb.so; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libnzb.so is missing: run `python -m neuzephyr_b200.build` (needs nvcc)")
        L = ctypes.CDLL(LIB_PATH)
        L.nzb_last_error_string.restype = ctypes.c_char_p
        i64p = ctypes.POINTER(ctypes.c_int64)
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        L.nzb_gemm_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc), ctypes.POINTER(sz)]
        L.nzb_gemm.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp, sz, vp]
        L.nzb_gemm_kernel_launches.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, ctypes.POINTER(ctypes.c_int)]
        L.nzb_gemm_static.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp]
        L.nzb_gemm_static_status.argtypes = [ctypes.POINTER(ctypes.c_int), vp]
        L.nzb_gemm_static_status_reset.argtypes = [vp]
        L.nzb_gemm_host_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc), ctypes.POINTER(sz)]
        L.nzb_gemm_host.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp, sz, vp]
        L.nzb_gemm_f16.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, ctypes.c_int64, vp, vp, vp]
        L.nzb_tensorcore_gemm_workspace_bytes.argtypes = [i64p, i64p, i64p, ctypes.POINTER(sz)]
        L.nzb_tensorcore_gemm.argtypes = [vp, vp, vp, i64p, i64p, i64p, vp, sz, vp]
        L.nzb_gemm_backward.argtypes = [vp, vp, vp, i64p, i64p, i64p, vp, sz, vp]
        L.nzb_matmul_f32_workspace_bytes.argtypes = [i64p, i64p, i64p, ctypes.POINTER(sz)]
        L.nzb_matmul_f32.argtypes = [vp, vp, vp, i64p, i64p, i64p, vp, sz, vp]
        L.nzb_cast_f32_f16.argtypes = [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                       ctypes.c_int, vp]
        L.nzb_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
        L.nzb_selftest_wait_timeout.argtypes = [ctypes.c_longlong, vp, vp]
        i64, f32, ci = ctypes.c_int64, ctypes.c_float, ctypes.c_int
        ld = ctypes.POINTER(LinearDesc)
        L.nzb_linear_workspace_bytes.argtypes = [ld, ctypes.POINTER(sz)]
        L.nzb_linear_forward.argtypes = [ld, vp, vp, vp, vp, vp, sz, vp]
        L.nzb_linear_backward.argtypes = [ld, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
        cd = ctypes.POINTER(ConvDesc)
        L.nzb_conv2d_workspace_bytes.argtypes = [cd, ctypes.POINTER(sz)]
        L.nzb_conv2d_forward.argtypes = [cd, vp, vp, vp, vp, vp, sz, vp]
        L.nzb_conv2d_backward_data.argtypes = [cd, vp, vp, vp, vp, sz, vp]
        L.nzb_conv2d_backward_weight.argtypes = [cd, vp, vp, vp, vp, sz, vp]
        L.nzb_conv2d_backward_bias.argtypes = [cd, vp, vp, vp]
        L.nzb_conv2d_backward_workspace_bytes.argtypes = [cd, ctypes.POINTER(sz)]
        L.nzb_conv2d_backward.argtypes = [cd, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
        L.nzb_img2col.argtypes = [vp, vp] + [i64] * 10 + [vp]
        L.nzb_img2col_backward.argtypes = [vp, vp] + [i64] * 10 + [vp]
        L.nzb_col2img.argtypes = [vp, vp] + [i64] * 4 + [vp]
        L.nzb_col2img_backward.argtypes = [vp, vp] + [i64] * 4 + [vp]
        L.nzb_add_broadcast.argtypes = [vp, vp, vp, i64p, i64p, vp]
        L.nzb_add_backward.argtypes = [vp, vp, i64p, i64p, vp]
        L.nzb_relu.argtypes = [vp, vp, i64, vp]
        L.nzb_relu_backward.argtypes = [vp, vp, vp, i64, vp]
        L.nzb_avgpool.argtypes = [vp, vp] + [i64] * 9 + [vp]
        L.nzb_avgpool_backward.argtypes = [vp, vp] + [i64] * 9 + [vp]
        L.nzb_avgpool_backward_ex.argtypes = [vp, vp] + [i64] * 9 + [ci, vp]
        L.nzb_softmax.argtypes = [vp, vp, i64, i64, vp]
        L.nzb_softmax_backward.argtypes = [vp, vp, vp, i64, i64, ci, vp]
        L.nzb_bce.argtypes = [vp, vp, vp, i64, vp]
        L.nzb_bce_backward.argtypes = [vp, vp, vp, i64, vp]
        L.nzb_adam.argtypes = [vp, vp, vp, vp, f32, f32, f32, f32, ci, i64, vp]
        L.nzb_adam_multi.argtypes = [ctypes.POINTER(AdamTensor), ci, f32, f32, f32, f32, vp]
        L.nzb_softmax_bce_forward.argtypes = [vp, vp, vp, vp, i64, i64, vp]
        L.nzb_softmax_bce_backward.argtypes = [vp, vp, vp, i64, i64, ci, vp]
        L.nzb_maxpool.argtypes = [vp, vp, vp] + [i64] * 9 + [vp]
        L.nzb_maxpool_backward.argtypes = [vp, vp, vp] + [i64] * 9 + [vp]
        L.nzb_fill.argtypes = [vp, f32, i64, vp]
        L.nzb_expand.argtypes = [vp, vp, i64, i64, vp]
        L.nzb_scale.argtypes = [vp, f32, i64, vp]
        _lib = L
    return _lib


def check(rc):
    if rc != OK:
        raise NzbError(rc, lib().nzb_last_error_string().decode())


def shape4(s):
    return (ctypes.c_int64 * 4)(*[int(v) for v in s])


def device_status():
    s = ctypes.c_int(0)
    check(lib().nzb_device_status(ctypes.byref(s)))
    return s.value
