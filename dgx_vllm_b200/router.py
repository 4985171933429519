"""MoE router on the GPU: gate projection + softmax + top-k + renormalisation in two small kernels, producing the
(topk_weights f32, topk_ids i32) pair the fused MoE ops take.  The reference leaves this step to vLLM; its benches
restate it in torch (sparse_fp4_kernel/bench_moe_layer_e2e.py:230-236), which is what the parity test compares with."""
from __future__ import annotations

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, require, require_cuda, stream_ptr, workspace


def moe_router(hidden_states: torch.Tensor, gate_weight: torch.Tensor, topk: int, renormalize: bool = True):
    """hidden_states [M,H], gate_weight [E,H] (both bf16 or both f16) -> (topk_weights [M,topk] f32, topk_ids [M,topk] i32).
    Weights are softmax probabilities of the selected experts, divided by their sum when renormalize is set."""
    dev = require_cuda(hidden_states, gate_weight)
    require(hidden_states.dim() == 2 and gate_weight.dim() == 2 and hidden_states.shape[1] == gate_weight.shape[1],
            "hidden_states [M,H] and gate_weight [E,H] must share H")
    require(hidden_states.dtype == gate_weight.dtype and hidden_states.dtype in (torch.bfloat16, torch.float16),
            "hidden_states and gate_weight must both be bfloat16 or both float16")
    require(hidden_states.stride(1) == 1 and gate_weight.is_contiguous(), "rows must be contiguous")
    M, H = hidden_states.shape
    E = gate_weight.shape[0]
    tw = torch.empty((M, topk), dtype=torch.float32, device=dev)
    ids = torch.empty((M, topk), dtype=torch.int32, device=dev)
    L = _lib.lib()
    ws = workspace(dev, L.b200fp4_moe_router_workspace_bytes(M, E))
    with torch.cuda.device(dev):
        _lib.check(L.b200fp4_moe_router(ptr(hidden_states), hidden_states.stride(0) if M > 1 else H, dtype_code(hidden_states.dtype),
                                        ptr(gate_weight), M, H, E, topk, 1 if renormalize else 0, ptr(tw), ptr(ids), ptr(ws),
                                        ws.numel(), stream_ptr(dev)), "moe_router")
    return tw, ids
