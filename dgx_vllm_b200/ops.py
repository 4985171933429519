"""Mirrors of the dense NVFP4 ops the reference enables in vLLM (`torch.ops._C.*` wrappers in
vllm/_custom_ops.py), backed by libb200nvfp4.so."""
from __future__ import annotations

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, require, require_cuda, stream_ptr, workspace


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


def cutlass_scaled_fp4_mm(a: torch.Tensor, b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                          alpha: torch.Tensor, out_dtype: torch.dtype, *, out: torch.Tensor | None = None,
                          tile_n: int = 0) -> torch.Tensor:
    """out[M,N] = alpha * (a . block_scale_a)(b . block_scale_b)^T on the tcgen05 tensor cores.

    Mirrors cutlass_scaled_fp4_mm (vllm/_custom_ops.py:741-753): a [M,K/2] and b [N,K/2] packed E2M1
    bytes, block scales in the swizzled 128x4 layout as produced by scaled_fp4_quant, alpha a
    one-element f32 CUDA tensor, out_dtype bf16 or f16.  Pass `out` to write in place like the raw
    torch.ops._C op does."""
    dev = require_cuda(a, b, block_scale_a, block_scale_b, alpha)
    require(a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1], "a [M,K/2] and b [N,K/2] must share K")
    require(a.dtype == torch.uint8 and b.dtype == torch.uint8, "a and b must be uint8 (packed E2M1)")
    require(a.is_contiguous() and b.is_contiguous(), "a and b must be contiguous")
    M, K2 = a.shape
    N = b.shape[0]
    K = K2 * 2
    require(K % 64 == 0, "K must be a multiple of 64")
    L = _lib.lib()
    need_a, need_b = L.b200fp4_sf_swizzled_bytes(M, K // 16), L.b200fp4_sf_swizzled_bytes(N, K // 16)
    for t, need, name in ((block_scale_a, need_a, "block_scale_a"), (block_scale_b, need_b, "block_scale_b")):
        require(t.is_contiguous() and t.element_size() * t.numel() >= need,
                f"{name} must be the swizzled scale tensor of at least {need} bytes")
    require(alpha.dtype == torch.float32 and alpha.numel() == 1, "alpha must be one f32")
    require(out_dtype in (torch.bfloat16, torch.float16), "out_dtype must be bfloat16 or float16")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    else:
        require(out.is_cuda and out.dtype == out_dtype and tuple(out.shape) == (M, N) and out.is_contiguous(),
                "out must be a contiguous [M,N] CUDA tensor of out_dtype")
    ws = workspace(dev, L.b200fp4_gemm_workspace_bytes(M, N, K))
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_gemm_nvfp4(ptr(a), ptr(b), ptr(block_scale_a), ptr(block_scale_b), ptr(alpha), ptr(out),
                                        dtype_code(out_dtype), M, N, K, tile_n, ptr(ws), ws.numel(), stream_ptr(dev)),
                   "cutlass_scaled_fp4_mm")
    return out


_linear_ws = {}


def nvfp4_linear(x: torch.Tensor, x_global_scale: torch.Tensor, w_codes: torch.Tensor, w_block_scale: torch.Tensor,
                 alpha: torch.Tensor, *, out: torch.Tensor | None = None, tile_n: int = 0) -> torch.Tensor:
    """y[M,N] = alpha * NVFP4(x) @ W^T: scaled_fp4_quant followed by cutlass_scaled_fp4_mm in ONE library call
    (b200fp4_linear_nvfp4), which is what a quantized linear layer does on every forward (the pair of ops in vLLM's
    NVFP4 linear apply, nvfp4_utils.py; emulated by the reference at fix_nvfp4_emulation_backend.py:60-102).  Same bytes
    as calling the two ops; the launches are a few microseconds apart instead of a Python call apart.
    x [M,K] bf16/f16 (rows may be strided), w_codes [N,K/2] u8, w_block_scale swizzled, alpha / x_global_scale one f32."""
    dev = require_cuda(x, x_global_scale, w_codes, w_block_scale, alpha)
    require(x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and x.stride(1) == 1, "x must be [M,K] bf16/f16, unit inner stride")
    require(w_codes.dim() == 2 and w_codes.dtype == torch.uint8 and w_codes.is_contiguous() and w_codes.shape[1] * 2 == x.shape[1],
            "w_codes must be contiguous [N,K/2] uint8")
    M, K = x.shape
    N = w_codes.shape[0]
    require(K % 64 == 0, "K must be a multiple of 64")
    L = _lib.lib()
    require(w_block_scale.is_contiguous() and
            w_block_scale.element_size() * w_block_scale.numel() >= L.b200fp4_sf_swizzled_bytes(N, K // 16),
            "w_block_scale must be the swizzled scale tensor of the weight")
    require(alpha.dtype == torch.float32 and alpha.numel() == 1 and x_global_scale.dtype == torch.float32 and
            x_global_scale.numel() == 1, "alpha and x_global_scale must be one f32 each")
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=dev)
    else:
        require(out.is_cuda and out.dtype in (torch.bfloat16, torch.float16) and tuple(out.shape) == (M, N) and
                out.is_contiguous(), "out must be a contiguous [M,N] 16-bit CUDA tensor")
    if M == 0:
        return out
    need = L.b200fp4_linear_workspace_bytes(M, N, K)
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _linear_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = _linear_ws[key] = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_linear_nvfp4(ptr(x), dtype_code(x.dtype), x.stride(0) if M > 1 else K, ptr(x_global_scale),
                                          ptr(w_codes), ptr(w_block_scale), ptr(alpha), ptr(out), dtype_code(out.dtype), M, N, K,
                                          tile_n, ptr(ws), ws.numel(), stream_ptr(dev)), "nvfp4_linear")
    return out


def last_gemm_status(device=None) -> int:
    """Status word of the most recent GEMM on the current stream of `device` (0 = ok).  Synchronises."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    torch.cuda.synchronize(dev)
    return int(workspace(dev, 256)[:4].view(torch.int32).item())
