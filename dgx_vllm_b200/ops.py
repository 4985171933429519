"""Mirrors of the dense NVFP4 ops the reference enables in vLLM (`torch.ops._C.*` wrappers in
vllm/_custom_ops.py), backed by libb200nvfp4.so."""
from __future__ import annotations

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, require, require_cuda, stream_ptr


def scaled_fp4_quant(input: torch.Tensor, input_global_scale: torch.Tensor, is_sf_swizzled_layout: bool = True):
    """bf16/f16 [M,K] -> (packed E2M1 codes u8 [M,K/2], E4M3 block scales).

    Mirrors scaled_fp4_quant (vllm/_custom_ops.py:1600-1671).  Scales come back as float8_e4m3fn:
    [round_up(M,128), round_up(K/16,4)] in the 128x4 swizzled tile layout (default) or [M, K/16]
    linear when is_sf_swizzled_layout is False.  input_global_scale is a one-element f32 CUDA tensor."""
    dev = require_cuda(input, input_global_scale)
    require(input.dim() == 2, "input must be 2-D")
    require(input.dtype in (torch.float16, torch.bfloat16), "input must be float16 or bfloat16")
    require(input.stride(1) == 1, "input rows must be contiguous")
    require(input_global_scale.dtype == torch.float32 and input_global_scale.numel() == 1, "global scale must be one f32")
    M, K = input.shape
    require(K % 16 == 0, "K must be a multiple of 16")
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    KB = K // 16
    if is_sf_swizzled_layout:
        sf = torch.empty(((M + 127) // 128 * 128, (KB + 3) // 4 * 4), dtype=torch.uint8, device=dev)
    else:
        sf = torch.empty((M, KB), dtype=torch.uint8, device=dev)
    L = _lib.lib()
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_quantize(ptr(input), dtype_code(input.dtype), M, K, input.stride(0) if M > 1 else K,
                                      ptr(input_global_scale), ptr(codes), ptr(sf), 1 if is_sf_swizzled_layout else 0,
                                      stream_ptr(dev)), "scaled_fp4_quant")
    return codes, sf.view(torch.float8_e4m3fn)
