"""Helpers shared by the tests: torch <-> numpy views and oracle-backed quantization."""
import numpy as np
import torch

import oracle


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bf16_bits(bits: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    if t.dtype == torch.float8_e4m3fn:
        t = t.view(torch.uint8)
    return t.numpy()


def oracle_quantize_fn(w_bf16: torch.Tensor, gs: torch.Tensor):
    """quantize_fn for synth.make_*_experts on CPU tensors, through the C oracle."""
    codes, sf = oracle.quantize_bf16(bf16_bits(w_bf16), float(gs.reshape(-1)[0]))
    return torch.from_numpy(codes), torch.from_numpy(sf)


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max|got-ref| / max|ref| -- the reference's own error metric
    (sparse_fp4_kernel/bench_v7_scaled.py:127-128, test_real_weights.py:219-221)."""
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64))) / (np.max(np.abs(ref)) + 1e-30))


def expert_fetch(w13: dict, w2: dict):
    """fetch(e) for oracle.fused_sparse_moe_by_expert over expert tables that may live on the GPU: copies one
    expert's 2:4 tensors (comp_T, meta_T, scale_T) and its global scale to the host on demand."""
    keys = ("comp_T", "meta_T", "scale_T")

    def one(w, e):
        return tuple(w[k][e].cpu().numpy() for k in keys) + (float(w["g_scales"][e]),)

    return lambda e: (one(w13, e), one(w2, e))


def gpu_quantize_fn(w_bf16: torch.Tensor, gs: torch.Tensor):
    """quantize_fn for synth.make_*_experts on CUDA tensors, through the CUDA quantizer (bit-exact with the oracle's,
    which the quantizer tests establish); used where the oracle would take minutes (512 experts)."""
    from dgx_vllm_b200 import scaled_fp4_quant
    c, s = scaled_fp4_quant(w_bf16, gs, is_sf_swizzled_layout=False)
    return c, s.view(torch.uint8)
