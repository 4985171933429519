"""GPU parity on the configurations the benchmark times, at their full expert counts and shapes (the other GPU test
files use reduced expert counts).  Yardstick: the CPU oracle, evaluated only for the experts that the sampled
tokens route to; tolerance max|diff| / max|ref| <= 1e-2 (the reference's metric, sparse_fp4_kernel/bench_v7_scaled.py:127-128).
Weights are quantized by the CUDA quantizer, whose bytes the quantizer tests pin to the oracle's."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from util import bf16_bits, expert_fetch, gpu_quantize_fn, rel_err, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2
E_TOTAL, HIDDEN, INTER, TOPK = 512, 2048, 512, 10
KEYS = ("comp_T", "meta_T", "scale_T", "g_scales")


@pytest.fixture(scope="module")
def moe_weights():
    import synth
    w13 = synth.make_sparse_experts(E_TOTAL, 2 * INTER, HIDDEN, 1000, "cuda", gpu_quantize_fn)
    w2 = synth.make_sparse_experts(E_TOTAL, HIDDEN, INTER, 2000, "cuda", gpu_quantize_fn)
    return w13, w2


@pytest.mark.parametrize("B,n_check", [(32, 32), (128, 12)])
def test_decode_layer_512_experts_top10(moe_weights, B, n_check):
    # the headline configuration: 512 experts, top-10, batch 32 (two launches) and 128 (second passes per expert)
    import synth
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    w13, w2 = moe_weights
    tw, ids = synth.make_routing(B, E_TOTAL, TOPK, 5 + B, "cuda")
    hidden = synth.make_hidden(B, HIDDEN, 6 + B, "cuda")
    emap = torch.empty(0, dtype=torch.int32, device="cuda")
    out = sp7.fused_sparse_moe_v7(hidden, tw, ids, emap, *[w13[k] for k in KEYS], *[w2[k] for k in KEYS], INTER, False)
    assert sp7.last_moe_status() == 0
    rows = np.sort(np.random.default_rng(B).choice(B, n_check, replace=False))
    ref = oracle.fused_sparse_moe_by_expert(hidden.float().cpu().numpy()[rows], tw.cpu().numpy()[rows],
                                            ids.cpu().numpy()[rows], expert_fetch(w13, w2), INTER)
    assert rel_err(to_np(out)[rows], ref) < TOL
    bound = sp7.FusedSparseMoE(*[w13[k] for k in KEYS], *[w2[k] for k in KEYS], INTER)     # the object bench.py times
    assert torch.equal(bound(hidden, tw, ids), out)


def test_expert_parallel_local_call_as_eight_ranks_issue_it(moe_weights):
    # what one of eight ranks runs per step: 256 received dispatch records (32 tokens from each rank), 64 local of 512
    # experts, expert_map with -1 for the others -> eight-token passes over the local experts
    import synth
    from dgx_vllm_b200 import _lib
    from dgx_vllm_b200._torch_util import workspace
    from dgx_vllm_b200.moe_ep import expert_map_for_rank
    L = _lib.lib()
    w13, w2 = moe_weights
    G, rank, T = 8, 3, 256
    El = E_TOTAL // G
    loc13 = {k: w13[k][rank * El:(rank + 1) * El].contiguous() for k in KEYS}
    loc2 = {k: w2[k][rank * El:(rank + 1) * El].contiguous() for k in KEYS}
    tw, ids = synth.make_routing(T, E_TOTAL, TOPK, 77, "cuda")
    hidden = synth.make_hidden(T, HIDDEN, 78, "cuda")
    emap = expert_map_for_rank(E_TOTAL, G, rank, "cuda")
    R = L.b200fp4_ep_record_bytes(HIDDEN, TOPK)
    rec = torch.empty(T * R, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.b200fp4_ep_pack(hidden.data_ptr(), ids.data_ptr(), tw.data_ptr(), T, HIDDEN, TOPK, 1, rec.data_ptr(), st), "pack")
    part = torch.empty(T, HIDDEN, dtype=torch.bfloat16, device="cuda")
    ws = workspace(torch.device("cuda", torch.cuda.current_device()), L.b200fp4_fused_moe_workspace_bytes(T, TOPK, HIDDEN, INTER, El))
    _lib.check(L.b200fp4_fused_sparse_moe_records(
        rec.data_ptr(), R, _lib.BF16, emap.data_ptr(), E_TOTAL, *[loc13[k].data_ptr() for k in KEYS], loc13["scale_T"].shape[1],
        *[loc2[k].data_ptr() for k in KEYS], loc2["scale_T"].shape[1], part.data_ptr(), _lib.BF16, T, TOPK, HIDDEN, INTER, El,
        _lib.SPARSE_META_ORDERED, ws.data_ptr(), ws.numel(), st), "records")
    torch.cuda.synchronize()
    mapped = emap.cpu().numpy()[ids.cpu().numpy()]
    assert (mapped >= 0).sum() >= 4 * El                      # the eight-token-pass branch of the layer
    rows = np.sort(np.random.default_rng(1).choice(T, 24, replace=False))
    ref = oracle.fused_sparse_moe_by_expert(hidden.float().cpu().numpy()[rows], tw.cpu().numpy()[rows], mapped[rows],
                                            expert_fetch(loc13, loc2), INTER)
    assert rel_err(to_np(part)[rows], ref) < TOL


def _dense_experts(E, N, K, seed):
    """E dense NVFP4 expert matrices on the GPU: codes [E,N,K/2], swizzled scales [E, pad128(N), pad4(K/16)], gs [E]."""
    import synth
    from dgx_vllm_b200 import scaled_fp4_quant
    gen = torch.Generator(device="cuda").manual_seed(seed)
    codes = torch.empty(E, N, K // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(E, (N + 127) // 128 * 128, (K // 16 + 3) // 4 * 4, dtype=torch.uint8, device="cuda")
    gs = torch.empty(E, dtype=torch.float32, device="cuda")
    for e0 in range(0, E, 64):
        w = (0.02 * torch.randn(min(64, E - e0), N, K, generator=gen, device="cuda")).to(torch.bfloat16)
        for i in range(w.shape[0]):
            g = synth.global_scale_of(w[i])
            c, s_ = scaled_fp4_quant(w[i], g)
            codes[e0 + i], sf[e0 + i], gs[e0 + i] = c, s_.view(torch.uint8), g[0]
    return codes, sf, gs


def test_grouped_prefill_shapes_512_experts_zipf():
    # the grouped-prefill configuration's shapes (512 experts, hidden 2048, intermediate 512, Zipf(1.1) top-10) on
    # 1024 tokens: both grouped GEMM outputs against the per-expert oracle on a sample of experts that covers the
    # most loaded ones (several 128-row tiles), lightly loaded ones and single-row ones
    import synth
    from dgx_vllm_b200 import grouped_moe as gm
    from dgx_vllm_b200.ops import last_gemm_status
    T, E, H, I = 1024, E_TOTAL, HIDDEN, INTER
    w13c, w13s, w13g = _dense_experts(E, 2 * I, H, 11)
    w2c, w2s, w2g = _dense_experts(E, H, I, 12)
    hidden = synth.make_hidden(T, H, 5, "cuda")
    tw, ids = synth.make_routing(T, E, TOPK, 6, "cuda", zipf=1.1)
    a1 = (448.0 * 6.0 / hidden.float().abs().max()).repeat(E).float()
    a2 = torch.full((E,), 448.0 * 6.0 / 2.0, dtype=torch.float32, device="cuda")
    alpha1, alpha2 = gm.nvfp4_moe_alphas(w13g, w2g, a1, a2)
    P = T * TOPK
    eo = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    a_map = torch.empty(P, dtype=torch.int32, device="cuda")
    c_map = torch.empty(P, dtype=torch.int32, device="cuda")
    bso = gm.get_cutlass_moe_mm_data(ids, eo, None, None, a_map, c_map, E, I, H, pair_indices=True)
    xq, xsf = gm.scatter_scaled_fp4_experts_quant(hidden, c_map, TOPK, a1, eo, bso, ids, None)
    c1 = torch.empty((P, 2 * I), dtype=torch.bfloat16, device="cuda")
    gm.cutlass_fp4_moe_mm(c1, xq, w13c, xsf, w13s, alpha1, None, eo, bso)
    assert last_gemm_status() == 0
    hq, hsf = gm.silu_and_mul_scaled_fp4_experts_quant(c1, a2, eo, bso)
    c2 = torch.empty((P, H), dtype=torch.bfloat16, device="cuda")
    gm.cutlass_fp4_moe_mm(c2, hq, w2c, hsf, w2s, alpha2, None, eo, bso)
    assert last_gemm_status() == 0
    # the fused gate_up epilogue gives the same bytes as GEMM + SiLU-mul quantizer for every valid row
    hq2, hsf2 = gm.cutlass_fp4_moe_mm_silu_and_mul_quant(xq, w13c, xsf, w13s, alpha1, eo, bso, a2, torch.bfloat16)
    n_rows = int(eo[-1])
    assert torch.equal(hq2[:n_rows], hq[:n_rows])

    eon, bson = to_np(eo), to_np(bso)
    counts = np.diff(eon)
    order = np.argsort(-counts)
    nonempty = order[counts[order] > 0]
    rng = np.random.default_rng(3)
    sample = list(nonempty[:6]) + list(nonempty[-6:]) + list(rng.choice(nonempty[6:-6], 12, replace=False))
    assert counts[nonempty[0]] > 256 and counts[nonempty[-1]] <= 8          # the skew the configuration is about

    def check(out, a_codes, a_sf, b_codes, b_sf, alphas, N, K):
        worst = 0.0
        for e in sample:
            r0, r1 = int(eon[e]), int(eon[e + 1])
            m = r1 - r0
            sf_lin = oracle.sf_swizzled_to_linear(to_np(a_sf)[bson[e]:bson[e] + (m + 127) // 128 * 128].reshape(-1), m, K // 16)
            ad = oracle.dequantize(to_np(a_codes[r0:r1]), sf_lin, 1.0)
            bd = oracle.dequantize(to_np(b_codes[e]), oracle.sf_swizzled_to_linear(to_np(b_sf[e]).reshape(-1), N, K // 16), 1.0)
            ref = oracle.matmul_nt(ad, bd) * np.float32(alphas[e])
            worst = max(worst, rel_err(to_np(out[r0:r1]), ref))
        return worst

    assert check(c1, xq, xsf, w13c, w13s, to_np(alpha1), 2 * I, H) < TOL
    assert check(c2, hq, hsf, w2c, w2s, to_np(alpha2), H, I) < TOL
    # and the layer's last step against the same rows: un-permute + weighted sum
    out = gm.moe_unpermute_reduce(c2, c_map, tw)
    ref = (c2.float()[c_map.long()].reshape(T, TOPK, H) * tw[:, :, None]).sum(1)
    assert rel_err(to_np(out), to_np(ref)) < TOL
    full = gm.nvfp4_moe_prefill(hidden, tw, ids, w13c, w13s, w13g, w2c, w2s, w2g, a1, a2, alphas=(alpha1, alpha2))
    assert torch.equal(full, out)


def test_dense_prefill_config_m1024_sampled_rows():
    # dense prefill configuration at M=1024 (N=14336, K=4096): 32 sampled rows against the oracle
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm, scaled_fp4_quant
    from dgx_vllm_b200.ops import last_gemm_status
    g = torch.Generator().manual_seed(13)
    x = torch.randn(1024, 4096, generator=g).bfloat16()
    w = (0.02 * torch.randn(14336, 4096, generator=g)).bfloat16()
    gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
    q = lambda t, gs, swz: scaled_fp4_quant(t.cuda(), torch.tensor([gs], dtype=torch.float32, device="cuda"), swz)
    xc, xs = q(x, gx, True)
    wc, ws = q(w, gw, True)
    alpha = torch.tensor([1.0 / (np.float32(gx) * np.float32(gw))], dtype=torch.float32, device="cuda")
    out = cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16)
    assert last_gemm_status() == 0
    rows = np.sort(np.random.default_rng(0).choice(1024, 32, replace=False))
    xcl, xsl = q(x, gx, False)
    wcl, wsl = q(w, gw, False)
    ref = oracle.matmul_nt(oracle.dequantize(to_np(xcl)[rows], to_np(xsl)[rows], gx), oracle.dequantize(to_np(wcl), to_np(wsl), gw))
    assert rel_err(to_np(out)[rows], ref) < TOL


def test_reference_gpu_kernel_agrees_on_the_decode_layer(moe_weights):
    # second yardstick: the reference's own CUDA extension (sparse_fp4_kernel/sparse_fp4_v7.cu, compiled unmodified
    # for sm_100 by oracle/build_ref_v7.py), run inside its contract: identity expert_map, N >= 512, fp16 result
    from oracle import build_ref_v7
    ref_mod = build_ref_v7.load()
    if ref_mod is None:
        pytest.skip("the reference extension was not built (oracle/build_ref_v7.py needs a checkout of the reference)")
    import synth
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7
    w13, w2 = moe_weights
    B = 8
    tw, ids = synth.make_routing(B, E_TOTAL, TOPK, 91, "cuda")
    hidden = synth.make_hidden(B, HIDDEN, 92, "cuda")
    emap = torch.empty(0, dtype=torch.int32, device="cuda")
    args = (hidden, tw, ids, emap, *[w13[k] for k in KEYS], *[w2[k] for k in KEYS], INTER, False)
    theirs = ref_mod.fused_sparse_moe_v7(*args)
    ours = sp7.fused_sparse_moe_v7(*args)
    torch.cuda.synchronize()
    assert theirs.dtype == torch.float16 and ours.dtype == torch.bfloat16
    ref = oracle.fused_sparse_moe_by_expert(hidden.float().cpu().numpy(), tw.cpu().numpy(), ids.cpu().numpy(),
                                            expert_fetch(w13, w2), INTER)
    assert rel_err(to_np(ours), ref) < TOL
    assert rel_err(to_np(theirs), ref) < 2e-2        # the reference rounds 32 + 8 partial sums per output to fp16
    assert rel_err(to_np(ours), to_np(theirs)) < 2e-2
