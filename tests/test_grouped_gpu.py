"""GPU parity of the grouped (per-expert) NVFP4 path: routing metadata, row shuffle, per-expert
quantization (bit-exact), grouped GEMM and un-permute, each against the oracle.
The grouped-GEMM oracle is a per-expert loop over the pinned dense oracle (no reference test covers
this boundary, so its parity is 'unpinned')."""
import numpy as np
import pytest
import torch

import oracle
from util import bf16_bits, rel_err, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _routing(M, E, topk, seed, zipf=1.1):
    import synth
    return synth.make_routing(M, E, topk, seed, "cpu", zipf=zipf)


def _metadata(ids, E, emap=None):
    from dgx_vllm_b200 import grouped_moe as gm
    M, topk = ids.shape
    eo = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    a_map = torch.empty(M * topk, dtype=torch.int32, device="cuda")
    c_map = torch.empty(M * topk, dtype=torch.int32, device="cuda")
    bso = gm.get_cutlass_moe_mm_data(ids.cuda(), eo, None, None, a_map, c_map, E, 0, 0,
                                     expert_map=None if emap is None else torch.from_numpy(emap).cuda())
    return eo, bso, a_map, c_map


@pytest.mark.parametrize("M,E,topk", [(40, 8, 2), (300, 64, 10), (5, 16, 4)])
def test_permute_metadata(M, E, topk):
    _, ids = _routing(M, E, topk, M)
    eo, bso, a_map, c_map = [to_np(t) for t in _metadata(ids, E)]
    idn = ids.numpy().reshape(-1)
    counts = np.bincount(idn, minlength=E)
    np.testing.assert_array_equal(np.diff(eo), counts)
    np.testing.assert_array_equal(np.diff(bso), (counts + 127) // 128 * 128)
    assert eo[0] == 0 and bso[0] == 0
    for p in range(M * topk):                      # pair -> permuted row lies in its expert's range, maps are inverse
        r = c_map[p]
        assert eo[idn[p]] <= r < eo[idn[p] + 1]
        assert a_map[r] == p // topk
    assert len(set(c_map.tolist())) == M * topk


def test_permute_with_expert_map_drops_foreign_pairs():
    M, E_local, E_global, topk = 50, 4, 8, 3
    _, ids = _routing(M, E_global, topk, 3)
    emap = np.array([-1, 0, 1, -1, -1, 2, -1, 3], np.int32)
    eo, bso, a_map, c_map = [to_np(t) for t in _metadata(ids, E_local, emap)]
    local = emap[ids.numpy().reshape(-1)]
    np.testing.assert_array_equal(np.diff(eo), np.bincount(local[local >= 0], minlength=E_local))
    assert np.all((c_map >= 0) == (local >= 0))
    assert np.all(a_map[eo[-1]:] == -1)


@pytest.mark.parametrize("with_map", [False, True])
def test_permute_metadata_large_batch(with_map):
    """Batches of 8192 pairs and more take the grid-wide routing pass; same contract as the one-block pass."""
    M, E_global, topk = 2048, 96, 10
    _, ids = _routing(M, E_global, topk, 11)
    if with_map:
        emap = np.full(E_global, -1, np.int32)
        emap[np.arange(0, E_global, 2)] = np.arange(E_global // 2)
        E = E_global // 2
    else:
        emap, E = None, E_global
    eo, bso, a_map, c_map = [to_np(t) for t in _metadata(ids, E, emap)]
    idn = ids.numpy().reshape(-1)
    local = idn if emap is None else emap[idn]
    counts = np.bincount(local[local >= 0], minlength=E)
    np.testing.assert_array_equal(eo, np.concatenate([[0], np.cumsum(counts)]))
    np.testing.assert_array_equal(bso, np.concatenate([[0], np.cumsum((counts + 127) // 128 * 128)]))
    kept = local >= 0
    assert np.all((c_map >= 0) == kept)
    rows = c_map[kept]
    assert np.all((eo[local[kept]] <= rows) & (rows < eo[local[kept] + 1]))
    assert len(np.unique(rows)) == kept.sum()
    np.testing.assert_array_equal(a_map[rows], np.nonzero(kept)[0] // topk)
    assert np.all(a_map[eo[-1]:] == -1)


def _expert_weights(E, N, K, seed):
    """dense NVFP4 expert weights quantized by the oracle: codes [E,N,K/2], linear sf [E,N,K/16], gs [E]."""
    g = torch.Generator().manual_seed(seed)
    codes, sfs, gss = [], [], []
    for _ in range(E):
        w = (0.02 * torch.randn(N, K, generator=g)).bfloat16()
        gs = float(oracle.global_scale(w.float().numpy()))
        c, s = oracle.quantize_bf16(bf16_bits(w), gs)
        codes.append(c), sfs.append(s), gss.append(gs)
    return np.stack(codes), np.stack(sfs), np.array(gss, np.float32)


def _swizzle_experts(sf):
    return np.stack([oracle.sf_linear_to_swizzled(s) for s in sf])


@pytest.mark.parametrize("M,E,topk,N,K,tile_n", [
    (40, 8, 2, 256, 256, 0), (300, 16, 4, 384, 512, 128), (64, 4, 2, 512, 2048, 256), (3, 8, 1, 128, 64, 0)])
def test_experts_quant_and_grouped_gemm(M, E, topk, N, K, tile_n):
    from dgx_vllm_b200 import grouped_moe as gm
    from dgx_vllm_b200.ops import last_gemm_status
    _, ids = _routing(M, E, topk, M + N)
    eo, bso, a_map, c_map = _metadata(ids, E)
    hidden = torch.randn(M, K, generator=torch.Generator().manual_seed(1)).bfloat16()
    x = gm.shuffle_rows(hidden.cuda(), a_map)
    xn, amapn, eon, bson = to_np(x), to_np(a_map), to_np(eo), to_np(bso)
    np.testing.assert_array_equal(xn, hidden.float().numpy()[amapn])
    a_gs = (np.linspace(50.0, 400.0, E)).astype(np.float32)
    xq, xsf = gm.scaled_fp4_experts_quant(x, torch.from_numpy(a_gs).cuda(), eo, bso)
    xqn, xsfn = to_np(xq), to_np(xsf)
    # per-expert quantization: bit-exact codes and scales, scales at the expert's padded offset
    KB = K // 16
    lin = np.zeros((M * topk, KB), np.uint8)
    for e in range(E):
        r0, r1 = eon[e], eon[e + 1]
        if r1 == r0:
            continue
        oc, osf = oracle.quantize_bf16(bf16_bits(x[r0:r1]), float(a_gs[e]))
        np.testing.assert_array_equal(xqn[r0:r1], oc)
        got = oracle.sf_swizzled_to_linear(xsfn[bson[e]:bson[e] + (r1 - r0 + 127) // 128 * 128].reshape(-1), r1 - r0, KB)
        np.testing.assert_array_equal(got, osf)
        lin[r0:r1] = osf
    wc, wsf, wgs = _expert_weights(E, N, K, 7)
    alphas = (1.0 / (a_gs * wgs)).astype(np.float32)
    out = torch.zeros((M * topk, N), dtype=torch.bfloat16, device="cuda")
    gm.cutlass_fp4_moe_mm(out, xq, torch.from_numpy(wc).cuda(), xsf, torch.from_numpy(_swizzle_experts(wsf)).cuda(),
                          torch.from_numpy(alphas).cuda(), None, eo, bso, tile_n=tile_n)
    assert last_gemm_status() == 0
    ref = oracle.grouped_nvfp4_gemm(xqn, lin, wc, wsf, alphas, eon, np.diff(eon))
    assert rel_err(to_np(out), ref) < TOL


@pytest.mark.parametrize("M,E,topk,I,K,dtype", [
    (300, 8, 4, 128, 256, torch.bfloat16),      # experts with more than one 128-row tile, one output tile per row tile
    (64, 4, 2, 256, 2048, torch.bfloat16),      # several k stages, two output tiles per row tile
    (50, 16, 3, 512, 512, torch.float16),       # some experts without rows; f16 intermediate
])
def test_grouped_gemm_with_silu_quant_epilogue_matches_separate_ops(M, E, topk, I, K, dtype):
    """gate_up GEMM with SiLU*up + quantization in its epilogue == GEMM into a 16-bit tensor, then the
    SiLU-mul quantizer: identical codes and block scales for every valid row."""
    from dgx_vllm_b200 import grouped_moe as gm
    from dgx_vllm_b200.ops import last_gemm_status
    _, ids = _routing(M, E, topk, M + I)
    eo, bso, a_map, c_map = _metadata(ids, E)
    hidden = torch.randn(M, K, generator=torch.Generator().manual_seed(5)).to(dtype)
    a_gs = torch.linspace(50.0, 400.0, E).cuda()
    a2_gs = torch.linspace(300.0, 30.0, E).cuda()
    xq, xsf = gm.shuffle_rows_scaled_fp4_experts_quant(hidden.cuda(), a_map, a_gs, eo, bso)
    wc, wsf, wgs = _expert_weights(E, 2 * I, K, 9)
    wc_d, wsf_d = torch.from_numpy(wc).cuda(), torch.from_numpy(_swizzle_experts(wsf)).cuda()
    alphas = (1.0 / (a_gs * torch.from_numpy(wgs).cuda())).float()
    c1 = torch.zeros((M * topk, 2 * I), dtype=dtype, device="cuda")
    gm.cutlass_fp4_moe_mm(c1, xq, wc_d, xsf, wsf_d, alphas, None, eo, bso)
    ref_q, ref_sf = gm.silu_and_mul_scaled_fp4_experts_quant(c1, a2_gs, eo, bso)
    got_q, got_sf = gm.cutlass_fp4_moe_mm_silu_and_mul_quant(xq, wc_d, xsf, wsf_d, alphas, eo, bso, a2_gs, dtype)
    assert last_gemm_status() == 0
    eon, bson = to_np(eo), to_np(bso)
    rows = eon[-1]
    np.testing.assert_array_equal(to_np(got_q)[:rows], to_np(ref_q)[:rows])
    g, r = to_np(got_sf).reshape(-1), to_np(ref_sf).reshape(-1)
    KB = I // 16
    row_bytes = (KB + 3) // 4 * 4
    for e in range(E):
        n = eon[e + 1] - eon[e]
        if n == 0:
            continue
        pad = (n + 127) // 128 * 128
        sl = slice(bson[e] * row_bytes, (bson[e] + pad) * row_bytes)
        np.testing.assert_array_equal(oracle.sf_swizzled_to_linear(g[sl], n, KB), oracle.sf_swizzled_to_linear(r[sl], n, KB))


def test_silu_quant_and_unpermute():
    from dgx_vllm_b200 import grouped_moe as gm
    M, E, topk, I = 30, 4, 2, 128
    tw, ids = _routing(M, E, topk, 9)
    eo, bso, a_map, c_map = _metadata(ids, E)
    gu = torch.randn(M * topk, 2 * I, generator=torch.Generator().manual_seed(2)).bfloat16()
    gs = np.array([30.0, 60.0, 90.0, 120.0], np.float32)
    hq, hsf = gm.silu_and_mul_scaled_fp4_experts_quant(gu.cuda(), torch.from_numpy(gs).cuda(), eo, bso)
    g32 = gu.float()
    act = (torch.nn.functional.silu(g32[:, :I]) * g32[:, I:]).bfloat16()
    eon = to_np(eo)
    mism = 0
    for e in range(E):
        r0, r1 = eon[e], eon[e + 1]
        if r1 > r0:
            oc, _ = oracle.quantize_bf16(bf16_bits(act[r0:r1]), float(gs[e]))
            mism += np.count_nonzero(oc != to_np(hq)[r0:r1])
    assert mism <= 2e-3 * hq.numel()          # expf differs by an ulp between host and device at a few elements
    eout = torch.randn(M * topk, 64, generator=torch.Generator().manual_seed(3)).bfloat16()
    out = gm.moe_unpermute_reduce(eout.cuda(), c_map, tw.cuda())
    ref = (eout.float().numpy()[to_np(c_map)].reshape(M, topk, 64) * tw.numpy()[:, :, None]).sum(1)
    assert rel_err(to_np(out), ref) < TOL


def test_moe_prefill_layer_small():
    # whole flow against a per-expert reference that quantizes both GEMM inputs the way the flow does
    from dgx_vllm_b200 import grouped_moe as gm
    M, E, topk, H, I = 64, 8, 2, 256, 128
    tw, ids = _routing(M, E, topk, 21)
    hidden = torch.randn(M, H, generator=torch.Generator().manual_seed(5)).bfloat16()
    w13c, w13s, w13g = _expert_weights(E, 2 * I, H, 11)
    w2c, w2s, w2g = _expert_weights(E, H, I, 12)
    a1 = np.full(E, 448.0 * 6.0 / float(hidden.float().abs().max()), np.float32)
    a2 = np.full(E, 448.0 * 6.0 / 1.0, np.float32)
    c = lambda a: torch.from_numpy(a).cuda()
    out = gm.nvfp4_moe_prefill(hidden.cuda(), tw.cuda(), ids.cuda(), c(w13c), c(_swizzle_experts(w13s)), c(w13g),
                               c(w2c), c(_swizzle_experts(w2s)), c(w2g), c(a1), c(a2))
    ref = np.zeros((M, H))
    f32_to_bf16 = lambda v: oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(v))
    for m in range(M):
        for t in range(topk):
            e = int(ids[m, t])
            W13 = oracle.dequantize(w13c[e], w13s[e], float(w13g[e])).astype(np.float64)
            W2 = oracle.dequantize(w2c[e], w2s[e], float(w2g[e])).astype(np.float64)
            xc, xs = oracle.quantize_bf16(bf16_bits(hidden[m:m + 1]), float(a1[e]))
            xq = oracle.dequantize(xc, xs, float(a1[e]))[0].astype(np.float64)
            gu = f32_to_bf16((W13 @ xq).astype(np.float32))                       # bf16 output of the first GEMM
            act = f32_to_bf16((gu[:I] / (1 + np.exp(-gu[:I])) * gu[I:]).astype(np.float32))
            ac, asf = oracle.quantize_bf16(oracle.f32_to_bf16_bits(act)[None, :], float(a2[e]))
            aq = oracle.dequantize(ac, asf, float(a2[e]))[0].astype(np.float64)
            ref[m] += float(tw[m, t]) * (W2 @ aq)
    assert rel_err(to_np(out), ref.astype(np.float32)) < 3e-2      # a few re-quantized codes flip on bf16 rounding
    cos = float((to_np(out).ravel() @ ref.ravel()) / (np.linalg.norm(to_np(out)) * np.linalg.norm(ref)))
    assert cos > 0.999


def test_ep_prefill_local_step_replays_from_a_graph():
    """The expert-parallel prefill layer captures its local layer (routing metadata, quantizer, grouped GEMMs, un-permute)
    into a CUDA graph per shape; replays over new contents of the gathered buffers equal the eager calls."""
    from dgx_vllm_b200 import grouped_moe as gm
    from dgx_vllm_b200.moe_ep import ExpertParallelMoEPrefill, expert_map_for_rank
    M, E, topk, H, I = 96, 8, 2, 256, 128
    w13c, w13s, w13g = _expert_weights(E, 2 * I, H, 31)
    w2c, w2s, w2g = _expert_weights(E, H, I, 32)
    c = lambda a: torch.from_numpy(a).cuda()
    a1 = np.full(E, 448.0 * 6.0 / 4.0, np.float32)
    a2 = np.full(E, 448.0 * 6.0 / 1.0, np.float32)
    weights = (c(w13c), c(_swizzle_experts(w13s)), c(w13g), c(w2c), c(_swizzle_experts(w2s)), c(w2g), c(a1), c(a2))
    layer = ExpertParallelMoEPrefill(E, weights)
    layer._emap = expert_map_for_rank(E, 1, 0, torch.device("cuda"))
    bufs = {"h": torch.empty(M, H, dtype=torch.bfloat16, device="cuda"), "i": torch.empty(M, topk, dtype=torch.int32, device="cuda"),
            "w": torch.empty(M, topk, dtype=torch.float32, device="cuda")}
    for seed in (41, 42, 43):
        tw, ids = _routing(M, E, topk, seed)
        hidden = torch.randn(M, H, generator=torch.Generator().manual_seed(seed)).bfloat16()
        bufs["h"].copy_(hidden)
        bufs["i"].copy_(ids)
        bufs["w"].copy_(tw)
        out = layer._local_step(bufs, "k").clone()
        ref = gm.nvfp4_moe_prefill(hidden.cuda(), tw.cuda(), ids.cuda(), *weights, expert_map=layer._emap)
        assert torch.equal(out, ref)
    assert "k" in layer._graphs


def test_gather_quant_matches_shuffle_then_quant():
    from dgx_vllm_b200 import grouped_moe as gm
    T, H, E, topk = 37, 256, 6, 3
    g = torch.Generator().manual_seed(5)
    hidden = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).to(torch.int32).cuda()
    emap = torch.arange(E, dtype=torch.int32)
    emap[2] = -1                                           # one expert is not local: its rows drop out of the map
    P = T * topk
    eo = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    a_map = torch.empty(P, dtype=torch.int32, device="cuda")
    c_map = torch.empty(P, dtype=torch.int32, device="cuda")
    bso = gm.get_cutlass_moe_mm_data(ids, eo, None, None, a_map, c_map, E, 64, H, expert_map=emap.cuda())
    gs = (torch.rand(E, generator=g) * 50 + 200).float().cuda()
    c_ref, s_ref = gm.scaled_fp4_experts_quant(gm.shuffle_rows(hidden, a_map), gs, eo, bso)
    c_new, s_new = gm.shuffle_rows_scaled_fp4_experts_quant(hidden, a_map, gs, eo, bso)
    assert torch.equal(c_ref, c_new)
    assert torch.equal(s_ref.view(torch.uint8), s_new.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scatter_quant_matches_gather_quant(dtype):
    """Token-major quantization writes the bytes of the row-major gather for every permuted row, with an
    expert_map that drops pairs (destinations < 0) and K larger than one pass of the block."""
    from dgx_vllm_b200 import grouped_moe as gm
    M, E_global, topk, K = 70, 12, 5, 4096 + 64
    _, ids = _routing(M, E_global, topk, 21)
    emap = np.full(E_global, -1, np.int32)
    emap[[0, 2, 3, 7, 8, 11]] = np.arange(6)
    E = 6
    eo, bso, a_map, c_map = _metadata(ids, E, emap)
    hidden = torch.randn(M, K, generator=torch.Generator().manual_seed(4)).to(dtype).cuda()
    gs = torch.linspace(40.0, 300.0, E).cuda()
    ref_q, ref_sf = gm.shuffle_rows_scaled_fp4_experts_quant(hidden, a_map, gs, eo, bso)
    rows = int(to_np(eo)[-1])
    assert 0 < rows < M * topk
    # with the owning expert searched for in expert_offsets, and read from the routing
    for kw in ({}, {"topk_ids": ids.cuda(), "expert_map": torch.from_numpy(emap).cuda()}):
        got_q, got_sf = gm.scatter_scaled_fp4_experts_quant(hidden, c_map, topk, gs, eo, bso, **kw)
        np.testing.assert_array_equal(to_np(got_q)[:rows], to_np(ref_q)[:rows])
        np.testing.assert_array_equal(to_np(got_sf), to_np(ref_sf))      # padding rows are zero in both
