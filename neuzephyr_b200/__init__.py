"""neuzephyr_b200: B200 (sm_100a) kernels behind NeuZephyr's dense-contraction path.

The product is the C-ABI library libnzb.so (include/nzb.h) and the C++ host layer that
mirrors NeuZephyr's API on top of it. This Python package only builds and binds them for
tests and benchmarks; it uses torch for device memory and streams, never for compute.
"""
from . import _capi  # noqa: F401
from .ops import (gemm, gemm_host, gemm_f16, gemm_workspace_bytes, tensorcore_gemm, gemm_backward, matmul_f32, cast_f32_f16,  # noqa: F401
                  device_status, conv2d_forward, conv2d_backward_data, conv2d_backward_weight,
                  conv2d_backward_bias, conv2d_backward, linear_forward, linear_backward)
