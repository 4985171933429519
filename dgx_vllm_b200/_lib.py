"""ctypes binding of libb200nvfp4.so (the C ABI declared in include/b200_nvfp4.h).

There is no CPU or PyTorch fallback: if the library is missing or an entry point returns a
non-zero status the call raises."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200nvfp4.so")

F16, BF16, F32 = 0, 1, 2
MOE_ROUTER_WEIGHT_ON_INPUT, SPARSE_META_ORDERED, MOE_SEPARATE_LAUNCHES, MOE_HOST_DIRECT_OUT = 1, 2, 4, 8     # flags of the sparse entry points

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int
_sz = ctypes.c_size_t

# name -> (restype, argtypes); must list every symbol include/b200_nvfp4.h declares
SIGNATURES = {
    "b200fp4_get_error_string": (ctypes.c_char_p, [_i32]),
    "b200fp4_version": (_i32, []),
    "b200fp4_version_string": (ctypes.c_char_p, []),
    "b200fp4_has_hardware_acceleration": (_i32, []),
    "b200fp4_launch_count": (ctypes.c_uint64, []),
    "b200fp4_sf_swizzled_bytes": (_sz, [_i64, _i64]),
    "b200fp4_sf_swizzle": (_i32, [_vp, _i64, _i64, _vp, _vp]),
    "b200fp4_quantize": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _vp]),
    "b200fp4_experts_quantize": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp, _vp, _i32, _i64, _i32, _vp, _vp, _vp]),
    "b200fp4_experts_quantize_gather": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp, _vp, _i32, _i64, _vp, _i32, _vp, _vp, _vp]),
    "b200fp4_experts_quantize_scatter": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _vp, _i64,
                                              _vp, _vp, _vp]),
    "b200fp4_gemm_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "b200fp4_gemm_nvfp4": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_moe_permute": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "b200fp4_shuffle_rows": (_i32, [_vp, _i64, _vp, _i64, _i64, _vp, _vp]),
    "b200fp4_grouped_gemm_workspace_bytes": (_sz, [_i64, _i64]),
    "b200fp4_grouped_gemm_nvfp4": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_grouped_gemm_nvfp4_silu_quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i64, _i64, _i64,
                                                     _i64, _vp, _sz, _vp]),
    "b200fp4_moe_unpermute_reduce": (_i32, [_vp, _i32, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "b200fp4_sparse_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "b200fp4_sparse_gemv": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_sparse_gemv_static": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _vp]),
    "b200fp4_dense_gemv": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _vp, _sz, _vp]),
    "b200fp4_sparse_packed_gemv": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _vp, _sz, _vp]),
    "b200fp4_convert_to_sparse_2of4": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "b200fp4_fused_moe_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64]),
    "b200fp4_moe_router_workspace_bytes": (_sz, [_i64, _i64]),
    "b200fp4_moe_router": (_i32, [_vp, _i64, _i32, _vp, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _sz, _vp]),
    "b200fp4_ep_record_bytes": (_sz, [_i64, _i64]),
    "b200fp4_ep_pack": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "b200fp4_fused_sparse_moe_records": (_i32, [_vp, _i64, _i32, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp,
                                                _i64, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_ep_combine": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp]),
    "b200fp4_ep_dispatch_p2p": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _i32, _vp, _vp]),
    "b200fp4_fused_sparse_moe_records_scatter": (_i32, [_vp, _i64, _i32, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp,
                                                        _i64, _vp, _i64, _i64, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_ep_combine_p2p": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _i32, _vp, _vp, _i32, _vp]),
    "b200fp4_fused_moe_profile_events": (None, [_vp, _vp, _vp]),
    "b200fp4_fused_sparse_moe": (_i32, [_vp, _i32, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp,
                                        _i64, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_fused_moe_set_wait_limit": (None, [_i64, _i32]),
    "b200fp4_fused_moe_last_status": (_i32, [_vp, _vp, _vp]),
    # the reference's declared C API (cutlass_nvfp4/cuda_fp4_gemm.h) under its own names
    "cudaFP4Create": (_i32, [_vp]),
    "cudaFP4Destroy": (_i32, [_vp]),
    "cudaFP4SetStream": (_i32, [_vp, _vp]),
    "cudaFP4GemmEx": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp, ctypes.c_float, _vp, _vp, ctypes.c_float, _vp, _i32]),
    "cudaFP4Gemm": (_i32, [_vp, _i32, _i32, _i32, ctypes.c_float, _vp, _vp, _vp]),
    "cudaFP4GetVersionString": (ctypes.c_char_p, []),
    "cudaFP4GetVersion": (_i32, []),
    "cudaFP4HasHardwareAcceleration": (_i32, []),
    "cudaFP4GetErrorString": (ctypes.c_char_p, [_i32]),
    "cudaFP4ConvertFromFP32": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "cudaFP4ConvertToFP32": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "cudaFP4Quantize": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "b200fp4_fused_moe_host_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64]),
    "b200fp4_fused_sparse_moe_host": (_i32, [_vp, _i32, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp,
                                             _i64, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_linear_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "b200fp4_linear_nvfp4": (_i32, [_vp, _i32, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b200fp4_fused_sparse_moe_host_async": (_i32, [_vp, _i32, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp,
                                                   _vp, _i64, _vp, _i32, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _sz,
                                                   _vp, _vp]),
}

_lib = None


class B200Fp4Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().b200fp4_get_error_string(status).decode()
        super().__init__(f"{where}: status {status} ({msg})")


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dgx_vllm_b200.build` (needs nvcc). "
                "This package has no fallback path.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise B200Fp4Error(status, where)
