"""torch custom-op registration: `torch.ops.b200_nvfp4.*` with the schemas of the ops the reference
wires into vLLM, so the library is a drop-in at the dispatcher level (torch.compile sees opaque ops
with shape-only fake implementations).

    scaled_fp4_quant(input, input_scale, is_sf_swizzled_layout) -> (codes, scales)     vllm _C::scaled_fp4_quant
    cutlass_scaled_fp4_mm(out!, a, b, block_scale_a, block_scale_b, alpha) -> ()        vllm _C::cutlass_scaled_fp4_mm
    cutlass_fp4_group_mm(out!, a, b, a_scales, b_scales, alphas, problem_sizes, expert_offsets, sf_offsets) -> ()
    batched_sparse_v7 / fused_sparse_moe_v7                                             sparse_fp4_v7.cu:744-749

`install_into_vllm()` points vllm._custom_ops at them (the B200 counterpart of the reference's
CMake/patch step cmake_patch_gb10_nvfp4_v6_full_kernels.sh:50-64 and of sparse_v7_moe_patch.patch_vllm)."""
from __future__ import annotations

import torch

from . import grouped_moe, ops, sparse_fp4_v7

_lib = torch.library.Library("b200_nvfp4", "DEF")
_lib.define("scaled_fp4_quant(Tensor input, Tensor input_scale, bool is_sf_swizzled_layout) -> (Tensor, Tensor)")
_lib.define("cutlass_scaled_fp4_mm(Tensor(a!) out, Tensor a, Tensor b, Tensor block_scale_a, Tensor block_scale_b, "
            "Tensor alpha) -> ()")
_lib.define("cutlass_fp4_group_mm(Tensor(a!) out, Tensor a, Tensor b, Tensor a_scales, Tensor b_scales, Tensor alphas, "
            "Tensor problem_sizes, Tensor expert_offsets, Tensor sf_offsets) -> ()")
_lib.define("batched_sparse_v7(Tensor A, Tensor B_comp_T, Tensor Meta_T_pk, Tensor scales_T, Tensor g_scales, "
            "Tensor expert_ids) -> Tensor")
_lib.define("fused_sparse_moe_v7(Tensor hidden_states, Tensor topk_weights, Tensor topk_ids, Tensor expert_map, "
            "Tensor w13_comp, Tensor w13_meta, Tensor w13_scale, Tensor w13_g_scales, Tensor w2_comp, Tensor w2_meta, "
            "Tensor w2_scale, Tensor w2_g_scales, int inter_size, bool apply_router_weight_on_input) -> Tensor")


def _quant_cuda(input, input_scale, is_sf_swizzled_layout):
    return ops.scaled_fp4_quant(input, input_scale, is_sf_swizzled_layout)


def _quant_fake(input, input_scale, is_sf_swizzled_layout):
    m, k = input.shape
    kb = k // 16
    codes = input.new_empty((m, k // 2), dtype=torch.uint8)
    shape = ((m + 127) // 128 * 128, (kb + 3) // 4 * 4) if is_sf_swizzled_layout else (m, kb)
    return codes, input.new_empty(shape, dtype=torch.float8_e4m3fn)


def _mm_cuda(out, a, b, block_scale_a, block_scale_b, alpha):
    ops.cutlass_scaled_fp4_mm(a, b, block_scale_a, block_scale_b, alpha, out.dtype, out=out)


def _group_mm_cuda(out, a, b, a_scales, b_scales, alphas, problem_sizes, expert_offsets, sf_offsets):
    grouped_moe.cutlass_fp4_moe_mm(out, a, b, a_scales, b_scales, alphas, problem_sizes, expert_offsets, sf_offsets)


def _sparse_cuda(A, B_comp_T, Meta_T_pk, scales_T, g_scales, expert_ids):
    return sparse_fp4_v7.batched_sparse_v7(A, B_comp_T, Meta_T_pk, scales_T, g_scales, expert_ids)


def _fused_cuda(hidden_states, topk_weights, topk_ids, expert_map, w13_comp, w13_meta, w13_scale, w13_g_scales, w2_comp,
                w2_meta, w2_scale, w2_g_scales, inter_size, apply_router_weight_on_input):
    return sparse_fp4_v7.fused_sparse_moe_v7(hidden_states, topk_weights, topk_ids, expert_map, w13_comp, w13_meta, w13_scale,
                                             w13_g_scales, w2_comp, w2_meta, w2_scale, w2_g_scales, inter_size,
                                             apply_router_weight_on_input)


_lib.impl("scaled_fp4_quant", _quant_cuda, "CUDA")
_lib.impl("cutlass_scaled_fp4_mm", _mm_cuda, "CUDA")
_lib.impl("cutlass_fp4_group_mm", _group_mm_cuda, "CUDA")
_lib.impl("batched_sparse_v7", _sparse_cuda, "CUDA")
_lib.impl("fused_sparse_moe_v7", _fused_cuda, "CUDA")
torch.library.register_fake("b200_nvfp4::scaled_fp4_quant", _quant_fake, lib=_lib)
torch.library.register_fake("b200_nvfp4::cutlass_scaled_fp4_mm", lambda *a: None, lib=_lib)
torch.library.register_fake("b200_nvfp4::cutlass_fp4_group_mm", lambda *a: None, lib=_lib)
torch.library.register_fake("b200_nvfp4::batched_sparse_v7",
                            lambda A, B, M, S, g, ids: A.new_empty((A.shape[0], B.shape[2])), lib=_lib)
torch.library.register_fake("b200_nvfp4::fused_sparse_moe_v7", lambda h, *a: torch.empty_like(h), lib=_lib)


def install_into_vllm() -> None:
    """Route vLLM's NVFP4 entry points to this library (call once, before the model is built)."""
    import vllm._custom_ops as vops

    def scaled_fp4_quant(input, input_global_scale, is_sf_swizzled_layout=True, backend=None):
        return torch.ops.b200_nvfp4.scaled_fp4_quant(input, input_global_scale, is_sf_swizzled_layout)

    def cutlass_scaled_fp4_mm(a, b, block_scale_a, block_scale_b, alpha, out_dtype):
        out = torch.empty((a.shape[0], b.shape[0]), dtype=out_dtype, device=a.device)
        torch.ops.b200_nvfp4.cutlass_scaled_fp4_mm(out, a, b, block_scale_a, block_scale_b, alpha)
        return out

    vops.scaled_fp4_quant = scaled_fp4_quant
    vops.cutlass_scaled_fp4_mm = cutlass_scaled_fp4_mm
    vops.cutlass_fp4_moe_mm = grouped_moe.cutlass_fp4_moe_mm
    vops.shuffle_rows = grouped_moe.shuffle_rows
    vops.scaled_fp4_experts_quant = grouped_moe.scaled_fp4_experts_quant
    vops.silu_and_mul_scaled_fp4_experts_quant = grouped_moe.silu_and_mul_scaled_fp4_experts_quant
