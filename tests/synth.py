"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

They stand in for the Qwen3-Next-80B-A3B NVFP4 checkpoint the reference's own scripts load
(sparse_fp4_kernel/test_patch_standalone.py:95-100), which cannot be downloaded.  Everything is
torch so the same code builds small CPU cases for the parity tests (quantizing through the
oracle) and full-size GPU cases for the benchmark (quantizing through the CUDA quantizer): the
caller supplies `quantize_fn(w_bf16 [R,K], gs f32[1]) -> (codes u8 [R,K/2], sf u8 [R,K/16])`.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

E2M1_MAX = 6.0
E4M3_MAX = 448.0


def global_scale_of(x: torch.Tensor) -> torch.Tensor:
    """vLLM's input_global_scale convention, 448*6/amax, as a one-element f32 tensor."""
    amax = x.abs().max().to(torch.float32)
    return (torch.tensor(E4M3_MAX * E2M1_MAX, dtype=torch.float32, device=x.device) / amax).reshape(1)


def unpack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K/2] u8 -> [..., K] nibbles (element 2i = low nibble of byte i)."""
    lo = codes & 0x0F
    hi = codes >> 4
    return torch.stack((lo, hi), dim=-1).reshape(*codes.shape[:-1], codes.shape[-1] * 2)


def random_2of4_positions(rows: int, K: int, gen: torch.Generator, device) -> torch.Tensor:
    """[rows, K/4, 2] sorted positions of the two kept elements of every group of four."""
    r = torch.rand(rows, K // 4, 4, generator=gen, device=device)
    pos = r.topk(2, dim=-1).indices
    return pos.sort(dim=-1).values


def mask_from_positions(pos: torch.Tensor) -> torch.Tensor:
    rows, G, _ = pos.shape
    m = torch.zeros(rows, G, 4, dtype=torch.bool, device=pos.device)
    m.scatter_(2, pos, True)
    return m.reshape(rows, G * 4)


def pack_2of4(codes: torch.Tensor, pos: torch.Tensor):
    """codes [R,K/2] + kept positions [R,K/4,2] -> comp [R,K/4], meta [R,K/8] (reference byte
    formats: sparse_fp4_kernel/sparse_v7_moe_patch.py:63-74)."""
    R = codes.shape[0]
    nib = unpack_nibbles(codes).reshape(R, -1, 4)
    v = nib.gather(2, pos)
    comp = (v[:, :, 0] | (v[:, :, 1] << 4)).to(torch.uint8)
    p = pos.to(torch.uint8).reshape(R, -1, 2, 2)          # [R, K/8, group-in-pair, which]
    meta = p[:, :, 0, 0] | (p[:, :, 0, 1] << 2) | (p[:, :, 1, 0] << 4) | (p[:, :, 1, 1] << 6)
    return comp, meta.to(torch.uint8)


def make_sparse_experts(E: int, N: int, K: int, seed: int, device, quantize_fn: Callable,
                        std: float = 0.02, chunk: int = 32):
    """E experts of 2:4-sparse NVFP4 weights [N,K] in the reference's transposed tensor format.

    Returns dict(comp_T [E,K/4,N], meta_T [E,K/8,N], scale_T [E,K/16,N], g_scales [E]); kept
    positions are drawn uniformly and the compressed tensors are built from those positions."""
    gen = torch.Generator(device=device).manual_seed(seed)
    comp_T = torch.empty(E, K // 4, N, dtype=torch.uint8, device=device)
    meta_T = torch.empty(E, K // 8, N, dtype=torch.uint8, device=device)
    scale_T = torch.empty(E, K // 16, N, dtype=torch.uint8, device=device)
    g = torch.empty(E, dtype=torch.float32, device=device)
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        w = std * torch.randn(n * N, K, generator=gen, device=device, dtype=torch.float32)
        pos = random_2of4_positions(n * N, K, gen, device)
        w = (w * mask_from_positions(pos)).to(torch.bfloat16)
        for i in range(n):
            we = w[i * N:(i + 1) * N]
            gs = global_scale_of(we)
            codes, sf = quantize_fn(we, gs)
            comp, meta = pack_2of4(codes, pos[i * N:(i + 1) * N])
            comp_T[e0 + i] = comp.t()
            meta_T[e0 + i] = meta.t()
            scale_T[e0 + i] = sf.view(torch.uint8).t()
            g[e0 + i] = 1.0 / gs[0]
    return {"comp_T": comp_T, "meta_T": meta_T, "scale_T": scale_T, "g_scales": g}


def make_dense_experts(E: int, N: int, K: int, seed: int, device, quantize_fn: Callable, std: float = 0.02,
                       chunk: int = 32):
    """E experts of dense NVFP4 weights: codes [E,N,K/2], linear scales [E,N,K/16], gs [E]."""
    gen = torch.Generator(device=device).manual_seed(seed)
    codes = torch.empty(E, N, K // 2, dtype=torch.uint8, device=device)
    sf = torch.empty(E, N, K // 16, dtype=torch.uint8, device=device)
    gs_all = torch.empty(E, dtype=torch.float32, device=device)
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        w = (std * torch.randn(n, N, K, generator=gen, device=device, dtype=torch.float32)).to(torch.bfloat16)
        for i in range(n):
            gs = global_scale_of(w[i])
            c, s = quantize_fn(w[i], gs)
            codes[e0 + i] = c
            sf[e0 + i] = s.view(torch.uint8)
            gs_all[e0 + i] = gs[0]
    return {"codes": codes, "sf": sf, "gs": gs_all}


def make_routing(B: int, E: int, topk: int, seed: int, device, zipf: Optional[float] = None):
    """top-k routing: softmax of N(0,1) logits, renormalised (bench_moe_layer_e2e.py:235), or --
    with zipf set -- experts drawn without replacement from a Zipf(zipf) popularity over a seeded
    permutation of the experts (Gumbel top-k) with softmax-of-normal weights."""
    gen = torch.Generator(device=device).manual_seed(seed)
    if zipf is None:
        logits = torch.randn(B, E, generator=gen, device=device)
        w, ids = torch.softmax(logits, dim=-1).topk(topk, dim=-1)
        w = w / w.sum(-1, keepdim=True)
    else:
        rank = torch.randperm(E, generator=gen, device=device).to(torch.float32) + 1.0
        logp = -zipf * torch.log(rank)
        u = torch.rand(B, E, generator=gen, device=device).clamp_min(1e-20)
        gumbel = -torch.log(-torch.log(u))
        ids = (logp.unsqueeze(0) + gumbel).topk(topk, dim=-1).indices
        w = torch.softmax(torch.randn(B, topk, generator=gen, device=device), dim=-1)
    return w.to(torch.float32).contiguous(), ids.to(torch.int32).contiguous()


def make_hidden(B: int, H: int, seed: int, device, dtype=torch.bfloat16) -> torch.Tensor:
    gen = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(B, H, generator=gen, device=device, dtype=torch.float32).to(dtype)
