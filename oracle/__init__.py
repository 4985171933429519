"""CPU oracle for the NVFP4 hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

numpy front end of ``nvfp4_oracle.c`` (a plain-C restatement of the reference's arithmetic; every
C function cites the reference file:line it follows).  Only ``tests/``, the smoke check and the
CPU-baseline leg of the benchmark import this package.  The shipped package never does and has
no CPU fallback.

Parity status (details in the header of ``nvfp4_oracle.c``): pinned for the quantizer, codecs,
scale swizzle, dense dequantize-then-matmul and the 2:4 sparse format (golden vectors generated
from the reference's own Python under ``tests/golden``); unpinned for the grouped MoE GEMM.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_f32p = ctypes.POINTER(ctypes.c_float)
_i64 = ctypes.c_int64


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (``make -C oracle``) and return the library path."""
    src = os.path.join(_HERE, "nvfp4_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-s"] + (["-B"] if force else []), check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.orc_e2m1_encode.argtypes = [ctypes.c_float]
        L.orc_e2m1_encode.restype = ctypes.c_uint8
        L.orc_e2m1_decode.argtypes = [ctypes.c_uint8]
        L.orc_e2m1_decode.restype = ctypes.c_float
        L.orc_e4m3_encode.argtypes = [ctypes.c_float]
        L.orc_e4m3_encode.restype = ctypes.c_uint8
        L.orc_e4m3_decode.argtypes = [ctypes.c_uint8]
        L.orc_e4m3_decode.restype = ctypes.c_float
        L.orc_quantize_bf16.argtypes = [_u16p, _i64, _i64, ctypes.c_float, _u8p, _u8p]
        L.orc_quantize_f32.argtypes = [_f32p, _i64, _i64, ctypes.c_float, _u8p, _u8p]
        L.orc_sf_swizzled_offset.argtypes = [_i64, _i64, _i64]
        L.orc_sf_swizzled_offset.restype = _i64
        L.orc_sf_swizzled_bytes.argtypes = [_i64, _i64]
        L.orc_sf_swizzled_bytes.restype = _i64
        L.orc_sf_linear_to_swizzled.argtypes = [_u8p, _i64, _i64, _u8p]
        L.orc_sf_swizzled_to_linear.argtypes = [_u8p, _i64, _i64, _u8p]
        L.orc_dequantize.argtypes = [_u8p, _u8p, ctypes.c_float, _i64, _i64, ctypes.c_int, _f32p]
        L.orc_matmul_nt.argtypes = [_f32p, _f32p, _i64, _i64, _i64, _f32p]
        L.orc_sparse_2of4_pack.argtypes = [_u8p, _i64, _i64, _u8p, _u8p]
        L.orc_sparse_expand.argtypes = [_u8p, _u8p, _u8p, ctypes.c_float, _i64, _i64, _i64, _f32p]
        L.orc_dense_T_expand.argtypes = [_u8p, _u8p, ctypes.c_float, _i64, _i64, _i64, _f32p]
        L.orc_silu_mul.argtypes = [_f32p, _i64, _i64, _f32p]
        _lib = L
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=dtype)


# ----------------------------------------------------------------------------- scalar codecs

def e2m1_encode(x: float) -> int:
    return int(lib().orc_e2m1_encode(float(np.float32(x))))


def e2m1_decode(code: int) -> float:
    return float(lib().orc_e2m1_decode(int(code) & 15))


def e4m3_encode(x: float) -> int:
    return int(lib().orc_e4m3_encode(float(np.float32(x))))


def e4m3_decode(b: int) -> float:
    return float(lib().orc_e4m3_decode(int(b) & 255))


E2M1_LUT = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def e4m3_lut() -> np.ndarray:
    return np.array([e4m3_decode(i) for i in range(256)], dtype=np.float32)


# ----------------------------------------------------------------------------- bf16 helpers

def f32_to_bf16_bits(x) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round-to-nearest-even."""
    u = _c(x, np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (_c(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f16_round(x) -> np.ndarray:
    return _c(x, np.float32).astype(np.float16).astype(np.float32)


# ----------------------------------------------------------------------------- quantizer

def global_scale(x) -> np.float32:
    """vLLM's ``input_global_scale`` convention: 448*6/amax (fp32)."""
    amax = np.float32(np.max(np.abs(_c(x, np.float32))))
    return np.float32(np.float32(448.0 * 6.0) / amax)


def quantize_bf16(x_bits, gs: float):
    """bf16 bit patterns [M,K] -> (codes u8 [M,K/2], linear e4m3 scales u8 [M,K/16])."""
    x_bits = _c(x_bits, np.uint16)
    M, K = x_bits.shape
    assert K % 16 == 0
    codes = np.empty((M, K // 2), np.uint8)
    sf = np.empty((M, K // 16), np.uint8)
    lib().orc_quantize_bf16(_p(x_bits, _u16p), M, K, float(np.float32(gs)), _p(codes, _u8p), _p(sf, _u8p))
    return codes, sf


def quantize_f32(x, gs: float):
    x = _c(x, np.float32)
    M, K = x.shape
    assert K % 16 == 0
    codes = np.empty((M, K // 2), np.uint8)
    sf = np.empty((M, K // 16), np.uint8)
    lib().orc_quantize_f32(_p(x, _f32p), M, K, float(np.float32(gs)), _p(codes, _u8p), _p(sf, _u8p))
    return codes, sf


def sf_swizzled_bytes(M: int, KB: int) -> int:
    return int(lib().orc_sf_swizzled_bytes(M, KB))


def sf_linear_to_swizzled(sf) -> np.ndarray:
    sf = _c(sf, np.uint8)
    M, KB = sf.shape
    out = np.empty(sf_swizzled_bytes(M, KB), np.uint8)
    lib().orc_sf_linear_to_swizzled(_p(sf, _u8p), M, KB, _p(out, _u8p))
    return out.reshape(((M + 127) // 128) * 128, ((KB + 3) // 4) * 4)


def sf_swizzled_to_linear(swz, M: int, KB: int) -> np.ndarray:
    swz = _c(swz, np.uint8).reshape(-1)
    assert swz.size >= sf_swizzled_bytes(M, KB)
    out = np.empty((M, KB), np.uint8)
    lib().orc_sf_swizzled_to_linear(_p(swz, _u8p), M, KB, _p(out, _u8p))
    return out


def dequantize(codes, sf, gs: float, round_bf16: bool = False) -> np.ndarray:
    """codes [M,K/2] + linear scales [M,K/16] -> fp32 [M,K] = lut[code]*sf/gs."""
    codes = _c(codes, np.uint8)
    sf = _c(sf, np.uint8)
    M, K2 = codes.shape
    out = np.empty((M, K2 * 2), np.float32)
    lib().orc_dequantize(_p(codes, _u8p), _p(sf, _u8p), float(np.float32(gs)), M, K2 * 2,
                         1 if round_bf16 else 0, _p(out, _f32p))
    return out


def matmul_nt(A, B, exact_c_loop: bool = False) -> np.ndarray:
    """C = A . B^T, accumulated in float64 and returned as fp32."""
    A = _c(A, np.float32)
    B = _c(B, np.float32)
    if exact_c_loop:
        C = np.empty((A.shape[0], B.shape[0]), np.float32)
        lib().orc_matmul_nt(_p(A, _f32p), _p(B, _f32p), A.shape[0], B.shape[0], A.shape[1], _p(C, _f32p))
        return C
    return (A.astype(np.float64) @ B.astype(np.float64).T).astype(np.float32)


def nvfp4_linear(x_bits, gs_x, w_codes, w_sf, gs_w, round_bf16: bool = False) -> np.ndarray:
    """The dense NVFP4 linear yardstick: quantize x, dequantize both operands, matmul in fp64.

    round_bf16=True rounds the dequantized operands to bf16 first, as the reference's emulation
    path does (fix_nvfp4_emulation_backend.py:77,97)."""
    xc, xs = quantize_bf16(x_bits, gs_x)
    xd = dequantize(xc, xs, gs_x, round_bf16)
    wd = dequantize(w_codes, w_sf, gs_w, round_bf16)
    return matmul_nt(xd, wd)


# ----------------------------------------------------------------------------- 2:4 sparse format

def sparse_2of4_pack(codes):
    """NVFP4 codes [N,K/2] -> (comp_T [K/4,N], meta_T [K/8,N]); ties: lower index kept."""
    codes = _c(codes, np.uint8)
    N, K2 = codes.shape
    K = K2 * 2
    assert K % 8 == 0
    comp = np.zeros((K // 4, N), np.uint8)
    meta = np.zeros((K // 8, N), np.uint8)
    lib().orc_sparse_2of4_pack(_p(codes, _u8p), N, K, _p(comp, _u8p), _p(meta, _u8p))
    return comp, meta


def sparse_expand(comp_T, meta_T, scale_T, g_scale: float) -> np.ndarray:
    """One expert's 2:4 tensors -> dense fp32 W [N,K]."""
    comp_T = _c(comp_T, np.uint8)
    meta_T = _c(meta_T, np.uint8)
    scale_T = _c(scale_T, np.uint8)
    K4, N = comp_T.shape
    K = K4 * 4
    G = scale_T.shape[0]
    W = np.empty((N, K), np.float32)
    lib().orc_sparse_expand(_p(comp_T, _u8p), _p(meta_T, _u8p), _p(scale_T, _u8p),
                            float(np.float32(g_scale)), N, K, G, _p(W, _f32p))
    return W


def dense_T_expand(dense_T, scale_T, g_scale: float) -> np.ndarray:
    dense_T = _c(dense_T, np.uint8)
    scale_T = _c(scale_T, np.uint8)
    K2, N = dense_T.shape
    K = K2 * 2
    W = np.empty((N, K), np.float32)
    lib().orc_dense_T_expand(_p(dense_T, _u8p), _p(scale_T, _u8p), float(np.float32(g_scale)), N, K,
                             scale_T.shape[0], _p(W, _f32p))
    return W


def batched_sparse_gemv(A, comp_T, meta_T, scale_T, g_scales, expert_ids) -> np.ndarray:
    """Oracle of batched_sparse_v7 (sparse_fp4_v7.cu:374-406): out[p] = A[p] . W[expert_ids[p]]^T.

    Returned in fp32 without the reference's fp16 partial-sum roundings."""
    A = _c(A, np.float32)
    out = np.zeros((A.shape[0], comp_T.shape[2]), np.float32)
    cache = {}
    for p, e in enumerate(np.asarray(expert_ids).reshape(-1)):
        e = int(e)
        if e < 0:
            continue
        if e not in cache:
            cache[e] = sparse_expand(comp_T[e], meta_T[e], scale_T[e], g_scales[e]).astype(np.float64)
        out[p] = (cache[e] @ A[p].astype(np.float64)).astype(np.float32)
    return out


def batched_dense_gemv(A, dense_T, scale_T, g_scales, expert_ids) -> np.ndarray:
    """Oracle of batched_dense_v7 (sparse_fp4_v7.cu:341-372)."""
    A = _c(A, np.float32)
    out = np.zeros((A.shape[0], dense_T.shape[2]), np.float32)
    for p, e in enumerate(np.asarray(expert_ids).reshape(-1)):
        e = int(e)
        if e < 0:
            continue
        W = dense_T_expand(dense_T[e], scale_T[e], g_scales[e]).astype(np.float64)
        out[p] = (W @ A[p].astype(np.float64)).astype(np.float32)
    return out


def silu_mul(x, inter: int) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty((x.shape[0], inter), np.float32)
    lib().orc_silu_mul(_p(x, _f32p), x.shape[0], inter, _p(out, _f32p))
    return out


def fused_sparse_moe(hidden, topk_w, topk_ids, expert_map, w13, w2, inter: int,
                     apply_router_weight_on_input: bool = False, round_fp16: bool = True) -> np.ndarray:
    """Oracle of fused_sparse_moe_v7 (sparse_fp4_v7.cu:607-742): per (token, expert) pair
    gate_up GEMV -> SiLU(gate)*up -> down GEMV -> router-weighted sum per token.

    w13 / w2 are (comp_T, meta_T, scale_T, g_scales) tuples.  hidden is fp32 holding the values
    the kernel sees (bf16- or fp16-representable).  round_fp16 applies the reference's fp16
    roundings of the two intermediate activations (gate_up and SiLU output are fp16 tensors there).
    Pairs whose mapped expert id is negative (expert not local) contribute nothing."""
    hidden = _c(hidden, np.float32)
    topk_ids = np.asarray(topk_ids)
    M, topk = topk_ids.shape
    ids = topk_ids.reshape(-1).astype(np.int64)
    if expert_map is not None and len(expert_map) > 0:
        ids = np.asarray(expert_map).astype(np.int64)[ids]
    A = np.repeat(hidden, topk, axis=0)
    gu = batched_sparse_gemv(A, *w13, ids)
    if round_fp16:
        gu = f16_round(gu)
    act = silu_mul(gu, inter)
    if round_fp16:
        act = f16_round(act)
    down = batched_sparse_gemv(act, *w2, ids)
    down[ids < 0] = 0.0
    down = down.reshape(M, topk, -1)
    if apply_router_weight_on_input:
        return down.sum(1).astype(np.float32)
    w = _c(topk_w, np.float32).reshape(M, topk, 1)
    return (down.astype(np.float64) * w).sum(1).astype(np.float32)


def fused_sparse_moe_by_expert(hidden, topk_w, mapped_ids, fetch, inter: int,
                               apply_router_weight_on_input: bool = False) -> np.ndarray:
    """fused_sparse_moe(round_fp16=False) evaluated expert by expert, for layers whose expert table is too
    large to expand on the host at once (512 experts): only the experts that `mapped_ids` names are
    touched.  mapped_ids [M, topk] holds local expert ids, negative = the pair contributes nothing (what
    expert_map does in fused_sparse_moe_v7, sparse_fp4_v7.cu:640-645).  fetch(e) returns
    ((comp_T, meta_T, scale_T, g_scale), (comp_T, meta_T, scale_T, g_scale)) of expert e for the gate_up and
    the down projection: 2-D arrays and one float each.  Same arithmetic as fused_sparse_moe: per pair
    gate_up GEMV -> SiLU(gate)*up -> down GEMV in fp64 on the fp32 expansion, router-weighted sum per token."""
    hidden = _c(hidden, np.float32)
    ids = np.asarray(mapped_ids).astype(np.int64)
    M, topk = ids.shape
    w = _c(topk_w, np.float32).reshape(M, topk)
    out = np.zeros((M, hidden.shape[1]), np.float64)
    for e in np.unique(ids[ids >= 0]):
        (c13, m13, s13, g13), (c2, m2, s2, g2) = fetch(int(e))
        tok, slot = np.nonzero(ids == e)
        W13 = sparse_expand(c13, m13, s13, g13).astype(np.float64)
        gu = (hidden[tok].astype(np.float64) @ W13.T).astype(np.float32)
        act = silu_mul(gu, inter)
        W2 = sparse_expand(c2, m2, s2, g2).astype(np.float64)
        down = (act.astype(np.float64) @ W2.T).astype(np.float32).astype(np.float64)
        scale = np.ones(len(tok)) if apply_router_weight_on_input else w[tok, slot].astype(np.float64)
        np.add.at(out, tok, down * scale[:, None])
    return out.astype(np.float32)


# ----------------------------------------------------------------------------- grouped GEMM

def grouped_nvfp4_gemm(a_codes, a_sf, b_codes, b_sf, alphas, expert_offsets, problem_m) -> np.ndarray:
    """Oracle of the grouped NVFP4 GEMM (cutlass_fp4_group_mm contract, vllm/_custom_ops.py:854-933):
    rows [off_e, off_e + m_e) of a are multiplied with expert e's weight; out = alpha_e * (a.sfa)(b.sfb)^T.

    a_sf here is linear [rows, K/16] and b_sf linear [E, N, K/16] (the swizzled forms are converted
    by the caller).  Parity unpinned: no reference test covers this boundary."""
    rows = a_codes.shape[0]
    E, N, _ = b_codes.shape
    out = np.zeros((rows, N), np.float32)
    for e in range(E):
        m = int(problem_m[e])
        if m == 0:
            continue
        o = int(expert_offsets[e])
        ad = dequantize(a_codes[o:o + m], a_sf[o:o + m], 1.0)
        bd = dequantize(b_codes[e], b_sf[e], 1.0)
        out[o:o + m] = matmul_nt(ad, bd) * np.float32(alphas[e])
    return out
