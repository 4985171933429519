"""Torch-on-CPU restatement of the reference's dequantize-to-bf16 emulation path -- TEST
INFRASTRUCTURE and the timed CPU baseline; never imported by the shipped package.

  * nvfp4_linear_emulation: run_nvfp4_emulations as rewritten by the reference,
    fix_nvfp4_emulation_backend.py:60-102 (quantize-dequantize x with ref_nvfp4_quant's operation
    order, dequantize W from packed codes x linear e4m3 scales / global scale to bf16, bf16 matmul).
  * moe_layer_emulation: per active expert dequantize -> matmul -> SiLU*up -> matmul ->
    router-weighted sum, after sparse_fp4_kernel/test_patch_standalone.py:219-247 and
    bench_v7_scaled.py compute_dense_ref, vectorised per expert.

Parity: the leaf arithmetic here is the same torch code as vLLM's nvfp4_emulation_utils
(ref_nvfp4_quant :439-453, cast_to_fp4 :425-436, break_fp4_bytes :328-345) restated, and is
checked against the C oracle and the golden vectors in tests/test_oracle_golden.py.
"""
from __future__ import annotations

import torch

_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def _reciprocal(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (x + (x == 0) * 1e8)


def cast_to_fp4(x: torch.Tensor) -> torch.Tensor:
    sign = torch.sign(x)
    x = torch.abs(x)
    x[(x >= 0.0) & (x <= 0.25)] = 0.0
    x[(x > 0.25) & (x < 0.75)] = 0.5
    x[(x >= 0.75) & (x <= 1.25)] = 1.0
    x[(x > 1.25) & (x < 1.75)] = 1.5
    x[(x >= 1.75) & (x <= 2.5)] = 2.0
    x[(x > 2.5) & (x < 3.5)] = 3.0
    x[(x >= 3.5) & (x <= 5.0)] = 4.0
    x[x > 5.0] = 6.0
    return x * sign


def ref_nvfp4_quant(x: torch.Tensor, global_scale: torch.Tensor, block_size: int = 16):
    m, n = x.shape
    x = torch.reshape(x, (m, n // block_size, block_size))
    vec_max = torch.max(torch.abs(x), dim=-1, keepdim=True)[0].to(torch.float32)
    scale = global_scale * (vec_max * (1 / 6.0))
    scale = torch.clamp(scale, max=448, min=-448)
    scale = scale.to(torch.float8_e4m3fn).to(torch.float32)
    output_scale = _reciprocal(scale * _reciprocal(global_scale))
    scaled_x = x.to(torch.float32) * output_scale
    clipped_x = torch.clamp(scaled_x, -6.0, 6.0).reshape(m, n)
    return cast_to_fp4(clipped_x), scale.squeeze(-1)


def break_fp4_bytes(a: torch.Tensor) -> torch.Tensor:
    """[R, K/2] u8 -> [R, K] f32 (element 2i in the low nibble)."""
    lo = (a & 0x0F).long()
    hi = (a >> 4).long()
    return torch.stack((_E2M1[lo], _E2M1[hi]), dim=-1).reshape(a.shape[0], a.shape[1] * 2)


def dequantize_weight(codes: torch.Tensor, sf_linear_u8: torch.Tensor, gs: torch.Tensor, dtype) -> torch.Tensor:
    m, k2 = codes.shape
    k = k2 * 2
    w = break_fp4_bytes(codes).reshape(m, k // 16, 16)
    sf = sf_linear_u8.view(torch.float8_e4m3fn)[:m, :k // 16].to(torch.float32) / gs
    return (w * sf.unsqueeze(-1)).reshape(m, k).to(dtype)


def nvfp4_linear_emulation(x: torch.Tensor, gs_x: torch.Tensor, w_codes: torch.Tensor, w_sf: torch.Tensor,
                           gs_w: torch.Tensor) -> torch.Tensor:
    """x [M,K] bf16/f16; returns [M,N] in x.dtype (fix_nvfp4_emulation_backend.py:60-102)."""
    m, k = x.shape
    x_fp4, x_bs = ref_nvfp4_quant(x, gs_x, 16)
    x_dq = (x_fp4.reshape(m, k // 16, 16) * (x_bs.unsqueeze(-1) / gs_x)).reshape(m, k).to(x.dtype)
    w_dq = dequantize_weight(w_codes, w_sf, gs_w, x.dtype)
    return torch.matmul(x_dq, w_dq.t())


def expand_sparse_expert(comp_T: torch.Tensor, meta_T: torch.Tensor, scale_T: torch.Tensor, g: float, dtype):
    """2:4 compressed tensors of one expert -> dense W [N,K] (sparse_fp4_kernel/test_real_weights.py:239-257)."""
    K4, N = comp_T.shape
    K = K4 * 4
    G = scale_T.shape[0]
    comp = comp_T.t().long()                                   # [N, K/4]
    meta = meta_T.t().long()                                   # [N, K/8]
    v0 = _E2M1[comp & 15]
    v1 = _E2M1[comp >> 4]
    sh = (torch.arange(K4) % 2) * 4
    mg = meta.repeat_interleave(2, dim=1) >> sh
    i0, i1 = mg & 3, (mg >> 2) & 3
    W = torch.zeros(N, K4, 4)
    W.scatter_add_(2, i0.unsqueeze(-1), v0.unsqueeze(-1))
    W.scatter_add_(2, i1.unsqueeze(-1), v1.unsqueeze(-1))
    s = scale_T.view(torch.float8_e4m3fn).to(torch.float32).t() * g          # [N, G]
    W = W.reshape(N, G, K // G) * s.unsqueeze(-1)
    return W.reshape(N, K).to(dtype)


def moe_layer_emulation(hidden: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor, w13: dict, w2: dict,
                        inter: int, table_rows: int | None = None) -> torch.Tensor:
    """One MoE layer on the CPU: for every active expert dequantize both projections to the
    activation dtype, run its tokens through gate_up -> SiLU*up -> down, accumulate the
    router-weighted result in fp32.

    table_rows: the weight tables hold only this many experts and expert id x reads row x % table_rows
    (the timed baseline keeps a small table on the host; every routed expert is still dequantized and
    multiplied on its own, so the work per step is that of the full table)."""
    M, H = hidden.shape
    out = torch.zeros(M, H, dtype=torch.float32)
    ids = topk_ids.long()
    for x in ids.unique().tolist():
        tok, slot = (ids == x).nonzero(as_tuple=True)
        e = x if table_rows is None else x % table_rows
        W13 = expand_sparse_expert(w13["comp_T"][e], w13["meta_T"][e], w13["scale_T"][e], float(w13["g_scales"][e]), hidden.dtype)
        W2 = expand_sparse_expert(w2["comp_T"][e], w2["meta_T"][e], w2["scale_T"][e], float(w2["g_scales"][e]), hidden.dtype)
        gu = hidden[tok] @ W13.t()
        act = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
        down = act @ W2.t()
        out.index_add_(0, tok, down.float() * topk_w[tok, slot].unsqueeze(-1))
    return out.to(hidden.dtype)
