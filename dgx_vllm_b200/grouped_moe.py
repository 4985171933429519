"""Grouped NVFP4 MoE path for prefill: routing metadata, row shuffle, per-expert quantization,
grouped GEMM, un-permute.  Function names and argument order mirror the ops vLLM's NVFP4 MoE flow
calls (vllm/_custom_ops.py: get_cutlass_moe_mm_data :854-896, shuffle_rows :921-933,
scaled_fp4_experts_quant :1674-1733, silu_and_mul_scaled_fp4_experts_quant, cutlass_fp4_moe_mm
:1017-1054; flow: vllm/model_executor/layers/fused_moe/experts/cutlass_moe.py:567-663), which is
the path the reference's grouped-MM files (grouped_mm_gb10_native.cu) stand in front of."""
from __future__ import annotations

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, require, require_cuda, stream_ptr, workspace


def get_cutlass_moe_mm_data(topk_ids, expert_offsets, problem_sizes1, problem_sizes2, input_permutation,
                            output_permutation, num_experts, n, k, blockscale_offsets=None, is_gated=True,
                            expert_map=None, pair_indices: bool = False):
    """Fills, in place: expert_offsets [E+1], blockscale_offsets [E+1], problem_sizes1/2 [E,3],
    input_permutation [M*topk] (permuted row -> source token row, -1 past the end) and
    output_permutation [M*topk] (pair -> permuted row, -1 if not local).  pair_indices=True leaves
    input_permutation holding pair indices (token*topk + slot) as the C routine writes them."""
    dev = require_cuda(topk_ids, expert_offsets, input_permutation, output_permutation)
    M, topk = topk_ids.shape
    ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
    ids = ids.contiguous()
    for t in (expert_offsets, input_permutation, output_permutation):
        require(t.dtype == torch.int32 and t.is_contiguous(), "metadata tensors must be contiguous int32")
    require(expert_offsets.numel() >= num_experts + 1, "expert_offsets must hold E+1 entries")
    bso = blockscale_offsets if blockscale_offsets is not None else torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    emap = None
    if expert_map is not None and expert_map.numel() > 0:
        emap = expert_map.to(torch.int32).contiguous()
    L = _lib.lib()
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_moe_permute(ptr(ids), ptr(emap), 0 if emap is None else emap.numel(), M, topk, num_experts,
                                         ptr(expert_offsets), ptr(bso), ptr(input_permutation), ptr(output_permutation),
                                         stream_ptr(dev)), "get_cutlass_moe_mm_data")
    if problem_sizes1 is not None or problem_sizes2 is not None:
        counts = expert_offsets[1:num_experts + 1] - expert_offsets[:num_experts]
    if problem_sizes1 is not None:
        problem_sizes1[:, 0] = counts
        problem_sizes1[:, 1] = 2 * n if is_gated else n
        problem_sizes1[:, 2] = k
    if problem_sizes2 is not None:
        problem_sizes2[:, 0] = counts
        problem_sizes2[:, 1] = k
        problem_sizes2[:, 2] = n
    # the C routine records pair indices; vLLM's a_map holds source token rows
    if not pair_indices:
        torch.div(input_permutation, topk, rounding_mode="floor", out=input_permutation)
    return bso


def shuffle_rows(input_tensor: torch.Tensor, dst2src_map: torch.Tensor) -> torch.Tensor:
    """out[i] = input[dst2src_map[i]] (zero rows where the map is negative)."""
    dev = require_cuda(input_tensor, dst2src_map)
    require(input_tensor.dim() == 2 and input_tensor.is_contiguous(), "input must be a contiguous 2-D tensor")
    require(dst2src_map.dtype == torch.int32 and dst2src_map.is_contiguous(), "map must be contiguous int32")
    row_bytes = input_tensor.shape[1] * input_tensor.element_size()
    require(row_bytes % 16 == 0, "rows must be a multiple of 16 bytes")
    out = torch.empty((dst2src_map.numel(), input_tensor.shape[1]), dtype=input_tensor.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_shuffle_rows(ptr(input_tensor), row_bytes, ptr(dst2src_map), dst2src_map.numel(), 1,
                                                   ptr(out), stream_ptr(dev)), "shuffle_rows")
    return out


def _experts_quant(input_tensor, input_global_scale, expert_offsets, blockscale_offsets, silu: bool):
    dev = require_cuda(input_tensor, input_global_scale, expert_offsets, blockscale_offsets)
    require(input_tensor.dim() == 2 and input_tensor.is_contiguous(), "input must be a contiguous 2-D tensor")
    require(input_tensor.dtype in (torch.float16, torch.bfloat16), "input must be float16 or bfloat16")
    rows, width = input_tensor.shape
    K = width // 2 if silu else width
    require(K % 16 == 0, "K must be a multiple of 16")
    E = expert_offsets.numel() - 1
    require(input_global_scale.dtype == torch.float32 and input_global_scale.numel() >= E, "one f32 global scale per expert")
    sf_rows = (rows + 127) // 128 * 128 + 128 * E
    codes = torch.empty((rows, K // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty((sf_rows, (K // 16 + 3) // 4 * 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_experts_quantize(ptr(input_tensor), dtype_code(input_tensor.dtype), rows, K,
                                                       ptr(input_global_scale), ptr(expert_offsets), ptr(blockscale_offsets),
                                                       E, sf_rows, 1 if silu else 0, ptr(codes), ptr(sf), stream_ptr(dev)),
                   "scaled_fp4_experts_quant")
    return codes, sf.view(torch.float8_e4m3fn)


def scaled_fp4_experts_quant(input_tensor, input_global_scale, expert_offsets, blockscale_offsets, topk=None):
    """Per-expert NVFP4 quantization of permuted rows -> (codes [rows,K/2], swizzled scales)."""
    return _experts_quant(input_tensor, input_global_scale, expert_offsets, blockscale_offsets, False)


def shuffle_rows_scaled_fp4_experts_quant(input_tensor, dst2src_map, input_global_scale, expert_offsets, blockscale_offsets):
    """shuffle_rows(input, dst2src_map) followed by scaled_fp4_experts_quant in one kernel: permuted row i
    quantizes input row dst2src_map[i] (zeros for a negative entry); the [rows, K] copy is never written."""
    dev = require_cuda(input_tensor, dst2src_map, input_global_scale, expert_offsets, blockscale_offsets)
    require(input_tensor.dim() == 2 and input_tensor.is_contiguous(), "input must be a contiguous 2-D tensor")
    require(input_tensor.dtype in (torch.float16, torch.bfloat16), "input must be float16 or bfloat16")
    require(dst2src_map.dtype == torch.int32 and dst2src_map.is_contiguous(), "map must be contiguous int32")
    rows, K = dst2src_map.numel(), input_tensor.shape[1]
    require(K % 16 == 0, "K must be a multiple of 16")
    E = expert_offsets.numel() - 1
    require(input_global_scale.dtype == torch.float32 and input_global_scale.numel() >= E, "one f32 global scale per expert")
    sf_rows = (rows + 127) // 128 * 128 + 128 * E
    codes = torch.empty((rows, K // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty((sf_rows, (K // 16 + 3) // 4 * 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_experts_quantize_gather(
            ptr(input_tensor), dtype_code(input_tensor.dtype), rows, K, ptr(input_global_scale), ptr(expert_offsets),
            ptr(blockscale_offsets), E, sf_rows, ptr(dst2src_map), 1, ptr(codes), ptr(sf), stream_ptr(dev)),
            "shuffle_rows_scaled_fp4_experts_quant")
    return codes, sf.view(torch.float8_e4m3fn)


def scatter_scaled_fp4_experts_quant(input_tensor, output_permutation, topk, input_global_scale, expert_offsets,
                                     blockscale_offsets, topk_ids=None, expert_map=None):
    """The result of shuffle_rows_scaled_fp4_experts_quant computed token-major: row t of input_tensor [M, K] is
    read once and quantized for each destination output_permutation[t*topk + s] (negative = none) with the global
    scale of the expert that owns that row.  Rows no pair maps to are left unwritten.  topk <= 32.
    topk_ids (int32 [M, topk], with expert_map if one was used) lets the kernel read the owning expert from the
    routing instead of searching expert_offsets for it."""
    dev = require_cuda(input_tensor, output_permutation, input_global_scale, expert_offsets, blockscale_offsets)
    require(input_tensor.dim() == 2 and input_tensor.is_contiguous(), "input must be a contiguous 2-D tensor")
    require(input_tensor.dtype in (torch.float16, torch.bfloat16), "input must be float16 or bfloat16")
    require(output_permutation.dtype == torch.int32 and output_permutation.is_contiguous(), "map must be contiguous int32")
    M, K = input_tensor.shape
    rows = output_permutation.numel()
    require(rows == M * topk and 0 < topk <= 32, "output_permutation must hold M*topk entries, topk <= 32")
    require(K % 16 == 0, "K must be a multiple of 16")
    E = expert_offsets.numel() - 1
    require(input_global_scale.dtype == torch.float32 and input_global_scale.numel() >= E, "one f32 global scale per expert")
    sf_rows = (rows + 127) // 128 * 128 + 128 * E
    codes = torch.empty((rows, K // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty((sf_rows, (K // 16 + 3) // 4 * 4), dtype=torch.uint8, device=dev)
    ids = emap = None
    if topk_ids is not None:
        ids = (topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)).contiguous()
        require(ids.is_cuda and ids.numel() == rows, "topk_ids must be a CUDA tensor [M, topk]")
        if expert_map is not None and expert_map.numel() > 0:
            emap = expert_map.to(torch.int32).contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_experts_quantize_scatter(
            ptr(input_tensor), dtype_code(input_tensor.dtype), M, K, topk, ptr(output_permutation), ptr(input_global_scale),
            ptr(expert_offsets), ptr(blockscale_offsets), E, sf_rows, ptr(ids), ptr(emap),
            0 if emap is None else emap.numel(), ptr(codes), ptr(sf), stream_ptr(dev)),
            "scatter_scaled_fp4_experts_quant")
    return codes, sf.view(torch.float8_e4m3fn)


def silu_and_mul_scaled_fp4_experts_quant(input_tensor, input_global_scale, expert_offsets, blockscale_offsets, topk=None):
    """SiLU(x[:, :K]) * x[:, K:] then per-expert NVFP4 quantization."""
    return _experts_quant(input_tensor, input_global_scale, expert_offsets, blockscale_offsets, True)


def cutlass_fp4_moe_mm(out_tensors, a_tensors, b_tensors, a_scales, b_scales, alphas, problem_sizes, expert_offsets,
                       sf_offsets, *, tile_n: int = 0):
    """Grouped NVFP4 GEMM, in place into out_tensors [rows, N] (bf16/f16).  problem_sizes is accepted for
    signature compatibility; the row ranges come from expert_offsets."""
    dev = require_cuda(out_tensors, a_tensors, b_tensors, a_scales, b_scales, alphas, expert_offsets, sf_offsets)
    require(a_tensors.dim() == 2 and b_tensors.dim() == 3, "a [rows,K/2], b [E,N,K/2]")
    rows, K2 = a_tensors.shape
    E, N, K2b = b_tensors.shape
    require(K2 == K2b and a_tensors.is_contiguous() and b_tensors.is_contiguous(), "a and b must share K and be contiguous")
    require(tuple(out_tensors.shape) == (rows, N) and out_tensors.is_contiguous(), "out must be contiguous [rows, N]")
    require(alphas.dtype == torch.float32 and alphas.numel() >= E, "one f32 alpha per expert")
    require(expert_offsets.dtype == torch.int32 and sf_offsets.dtype == torch.int32, "offsets must be int32")
    L = _lib.lib()
    K = K2 * 2
    require(b_scales.numel() * b_scales.element_size() >= E * L.b200fp4_sf_swizzled_bytes(N, K // 16),
            "b_scales must hold one swizzled scale tensor per expert")
    ws = workspace(dev, L.b200fp4_grouped_gemm_workspace_bytes(rows, E))
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_grouped_gemm_nvfp4(ptr(a_tensors), ptr(b_tensors), ptr(a_scales), ptr(b_scales), ptr(alphas),
                                                ptr(expert_offsets), ptr(sf_offsets), ptr(out_tensors),
                                                dtype_code(out_tensors.dtype), rows, N, K, E, tile_n, ptr(ws), ws.numel(),
                                                stream_ptr(dev)), "cutlass_fp4_moe_mm")
    return out_tensors


def cutlass_fp4_moe_mm_silu_and_mul_quant(a_tensors, b_tensors, a_scales, b_scales, alphas, expert_offsets, sf_offsets,
                                          out_global_scale, mid_dtype=torch.bfloat16):
    """cutlass_fp4_moe_mm into a [rows, 2I] tensor of mid_dtype followed by
    silu_and_mul_scaled_fp4_experts_quant, in one kernel: the gate_up projection's epilogue applies
    SiLU(gate)*up to the 16-bit rounded products and quantizes them, so the [rows, 2I] tensor is never
    written.  b_tensors [E, 2I, K/2] with the gate rows first (I a multiple of 128).  Returns
    (codes [rows, I/2], swizzled scales) with the bytes the two separate ops give for every valid row."""
    dev = require_cuda(a_tensors, b_tensors, a_scales, b_scales, alphas, expert_offsets, sf_offsets, out_global_scale)
    require(a_tensors.dim() == 2 and b_tensors.dim() == 3, "a [rows,K/2], b [E,2I,K/2]")
    rows, K2 = a_tensors.shape
    E, N, K2b = b_tensors.shape
    require(K2 == K2b and a_tensors.is_contiguous() and b_tensors.is_contiguous(), "a and b must share K and be contiguous")
    require(N % 256 == 0, "the intermediate size must be a multiple of 128")
    require(alphas.dtype == torch.float32 and alphas.numel() >= E, "one f32 alpha per expert")
    require(out_global_scale.dtype == torch.float32 and out_global_scale.numel() >= E, "one f32 global scale per expert")
    require(expert_offsets.dtype == torch.int32 and sf_offsets.dtype == torch.int32, "offsets must be int32")
    require(mid_dtype in (torch.float16, torch.bfloat16), "mid_dtype must be float16 or bfloat16")
    L = _lib.lib()
    K, I = K2 * 2, N // 2
    require(b_scales.numel() * b_scales.element_size() >= E * L.b200fp4_sf_swizzled_bytes(N, K // 16),
            "b_scales must hold one swizzled scale tensor per expert")
    sf_rows = (rows + 127) // 128 * 128 + 128 * E
    codes = torch.empty((rows, I // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty((sf_rows, (I // 16 + 3) // 4 * 4), dtype=torch.uint8, device=dev)
    ws = workspace(dev, L.b200fp4_grouped_gemm_workspace_bytes(rows, E))
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_grouped_gemm_nvfp4_silu_quant(
            ptr(a_tensors), ptr(b_tensors), ptr(a_scales), ptr(b_scales), ptr(alphas), ptr(expert_offsets), ptr(sf_offsets),
            ptr(out_global_scale), dtype_code(mid_dtype), ptr(codes), ptr(sf), rows, N, K, E, ptr(ws), ws.numel(),
            stream_ptr(dev)), "cutlass_fp4_moe_mm_silu_and_mul_quant")
    return codes, sf.view(torch.float8_e4m3fn)


def moe_unpermute_reduce(expert_out, output_permutation, topk_weights):
    """out[m] = sum_t topk_weights[m,t] * expert_out[output_permutation[m*topk+t]] over local pairs."""
    dev = require_cuda(expert_out, output_permutation, topk_weights)
    M, topk = topk_weights.shape
    H = expert_out.shape[1]
    tw = topk_weights.to(torch.float32).contiguous()
    out = torch.empty((M, H), dtype=expert_out.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200fp4_moe_unpermute_reduce(ptr(expert_out), dtype_code(expert_out.dtype),
                                                           ptr(output_permutation), ptr(tw), M, topk, H, ptr(out),
                                                           stream_ptr(dev)), "moe_unpermute_reduce")
    return out


def nvfp4_moe_alphas(w13_gs, w2_gs, a1_gs, a2_gs):
    """The per-expert output scales of the two grouped GEMMs, 1 / (activation scale * weight scale): constants
    of a layer, computed once and passed to nvfp4_moe_prefill as alphas=."""
    return (1.0 / (a1_gs * w13_gs)).float().contiguous(), (1.0 / (a2_gs * w2_gs)).float().contiguous()


def nvfp4_moe_prefill(hidden, topk_weights, topk_ids, w13_codes, w13_sf, w13_gs, w2_codes, w2_sf, w2_gs,
                      a1_gs, a2_gs, expert_map=None, alphas=None):
    """One MoE layer over dense NVFP4 expert weights (the flow of cutlass_moe.py:567-663):
    permute metadata -> quantize each token for its experts -> grouped GEMM (gate_up) with SiLU*up + quantize in its epilogue ->
    grouped GEMM (down) -> combine.

    w13_codes [E,2I,H/2], w13_sf [E, swizzled(2I,H/16)], w13_gs [E] weight global scales (448*6/amax);
    w2_* likewise for [E,H,I/2]; a1_gs / a2_gs [E] activation global scales of the two GEMM inputs."""
    dev = hidden.device
    M, H = hidden.shape
    topk = topk_ids.shape[1]
    E, N1, _ = w13_codes.shape
    P = M * topk
    eo = torch.empty(E + 1, dtype=torch.int32, device=dev)
    a_map = torch.empty(P, dtype=torch.int32, device=dev)
    c_map = torch.empty(P, dtype=torch.int32, device=dev)
    alpha1, alpha2 = alphas if alphas is not None else nvfp4_moe_alphas(w13_gs, w2_gs, a1_gs, a2_gs)
    bso = get_cutlass_moe_mm_data(topk_ids, eo, None, None, a_map, c_map, E, N1 // 2, H, expert_map=expert_map,
                                  pair_indices=topk <= 32)
    if topk <= 32:
        xq, xsf = scatter_scaled_fp4_experts_quant(hidden, c_map, topk, a1_gs, eo, bso, topk_ids, expert_map)
    else:
        xq, xsf = shuffle_rows_scaled_fp4_experts_quant(hidden, a_map, a1_gs, eo, bso)
    if N1 % 256 == 0:
        hq, hsf = cutlass_fp4_moe_mm_silu_and_mul_quant(xq, w13_codes, xsf, w13_sf, alpha1, eo, bso, a2_gs, hidden.dtype)
    else:
        c1 = torch.empty((P, N1), dtype=hidden.dtype, device=dev)
        cutlass_fp4_moe_mm(c1, xq, w13_codes, xsf, w13_sf, alpha1, None, eo, bso)
        hq, hsf = silu_and_mul_scaled_fp4_experts_quant(c1, a2_gs, eo, bso)
    c2 = torch.empty((P, H), dtype=hidden.dtype, device=dev)
    cutlass_fp4_moe_mm(c2, hq, w2_codes, hsf, w2_sf, alpha2, None, eo, bso)
    return moe_unpermute_reduce(c2, c_map, topk_weights)
