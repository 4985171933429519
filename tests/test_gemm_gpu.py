"""GPU parity of the dense block-scaled NVFP4 GEMM (tcgen05 path, through the C ABI) against the
oracle's fp32 dequantize-then-matmul.  Tolerance: max|diff| / max|ref| <= 1e-2."""
import os

import numpy as np
import pytest
import torch

import oracle
from util import bf16_bits, from_bf16_bits, rel_err, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _quant_gpu(t, gs, swz=True):
    from dgx_vllm_b200 import scaled_fp4_quant
    return scaled_fp4_quant(t.cuda(), torch.tensor([gs], dtype=torch.float32, device="cuda"), swz)


def _run(x, w, out_dtype=torch.bfloat16, tile_n=0):
    """x [M,K], w [N,K] bf16 CPU tensors -> (gpu result, oracle result, status)."""
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm
    from dgx_vllm_b200.ops import last_gemm_status
    gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
    xc, xs = _quant_gpu(x, gx)
    wc, ws = _quant_gpu(w, gw)
    alpha = torch.tensor([1.0 / (np.float32(gx) * np.float32(gw))], dtype=torch.float32, device="cuda")
    out = cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, out_dtype, tile_n=tile_n)
    status = last_gemm_status()
    oc, osf = oracle.quantize_bf16(bf16_bits(x), gx)
    wcq, wsf = oracle.quantize_bf16(bf16_bits(w), gw)
    np.testing.assert_array_equal(to_np(xc), oc)                     # same codes as the oracle, so the
    ref = oracle.matmul_nt(oracle.dequantize(oc, osf, gx), oracle.dequantize(wcq, wsf, gw))   # yardstick is exact
    return to_np(out), ref, status


def _rand(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g).bfloat16(), (0.02 * torch.randn(N, K, generator=g)).bfloat16()


def test_c1_golden_config(golden_dir):
    # the reference's CPU-runnable case: x 8x2048, W 512x2048, against its own emulation output
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm, scaled_fp4_quant
    g = np.load(os.path.join(golden_dir, "dense_c1.npz"))
    gx, gw = float(g["gs_x"][0]), float(g["gs_w"][0])
    x = from_bf16_bits(g["x_bits"])
    xc, xs = _quant_gpu(x, gx)
    wc = torch.from_numpy(g["w_codes"]).cuda()
    ws = torch.from_numpy(oracle.sf_linear_to_swizzled(g["w_sf"])).cuda()
    alpha = torch.tensor([1.0 / (np.float32(gx) * np.float32(gw))], dtype=torch.float32, device="cuda")
    out = to_np(cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16))
    ref_emulation = oracle.bf16_bits_to_f32(g["out_bits"])
    exact = oracle.nvfp4_linear(g["x_bits"], gx, g["w_codes"], g["w_sf"], gw)
    assert rel_err(out, exact) < TOL
    assert rel_err(out, ref_emulation) < TOL


@pytest.mark.parametrize("M,N,K,tile_n", [
    (128, 128, 256, 128), (128, 256, 256, 256),       # one tile, one stage
    (128, 128, 1024, 128), (256, 512, 2048, 0),       # several stages / tiles
    (1, 128, 64, 0), (7, 384, 320, 0),                # M tail, K tail (K % 256 != 0), N = 1.5 wide tiles
    (200, 384, 320, 256), (129, 136, 192, 128),       # N not a multiple of the tile or of 128
    (300, 1024, 4096, 0),
])
def test_shapes(M, N, K, tile_n):
    out, ref, status = _run(*_rand(M, N, K, M + N + K), tile_n=tile_n)
    assert status == 0
    assert out.shape == (M, N)
    assert rel_err(out, ref) < TOL


@pytest.mark.parametrize("M,N,K", [
    (256, 256, 256),                 # one pair tile, one stage
    (128, 256, 256), (1, 128, 64),   # the second CTA's rows lie entirely past M
    (7, 384, 320), (200, 384, 320),  # M, N and K tails
    (512, 768, 1024),                # several pair tiles and stages (the rings wrap)
    (300, 1024, 4096),               # more stages than ring slots, several tiles per pair
    (2304, 2560, 1024),              # more pair tiles than pairs of SMs: every pair takes a second tile
])
def test_pair_kernel_shapes(M, N, K):
    """tile_n=512 selects the CTA-pair kernel (tcgen05 cta_group::2, 256x256 tiles)."""
    out, ref, status = _run(*_rand(M, N, K, M + N + K + 1), tile_n=512)
    assert status == 0
    assert out.shape == (M, N)
    assert rel_err(out, ref) < TOL
    out16, ref16, status16 = _run(*_rand(M, N, K, M + N + K + 2), out_dtype=torch.float16, tile_n=512)
    assert status16 == 0 and rel_err(out16, ref16) < TOL


def test_fp16_output_and_in_place_and_determinism():
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm
    x, w = _rand(64, 256, 512, 3)
    out, ref, status = _run(x, w, out_dtype=torch.float16)
    assert status == 0 and rel_err(out, ref) < TOL
    gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
    xc, xs = _quant_gpu(x, gx)
    wc, ws = _quant_gpu(w, gw)
    alpha = torch.tensor([1.0 / (gx * gw)], dtype=torch.float32, device="cuda")
    buf = torch.full((64, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    r = cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16, out=buf)
    assert r.data_ptr() == buf.data_ptr()
    r2 = cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16)
    assert torch.equal(r, r2)
    with pytest.raises(RuntimeError):
        cutlass_scaled_fp4_mm(xc[:, :24], wc[:, :24], xs, ws, alpha, torch.bfloat16)      # K % 64 != 0
    with pytest.raises(RuntimeError):
        cutlass_scaled_fp4_mm(xc, wc, xs[:64], ws, alpha, torch.bfloat16)                 # scale tensor too small


def test_linear_in_one_call_matches_the_two_ops():
    """nvfp4_linear (quantizer + GEMM queued by one library call) returns the bytes of scaled_fp4_quant followed by
    cutlass_scaled_fp4_mm, for contiguous and row-strided activations, small and pair-kernel sizes."""
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm, scaled_fp4_quant
    from dgx_vllm_b200.ops import last_gemm_status, nvfp4_linear
    for M, N, K in ((9, 384, 320), (300, 512, 1024), (2304, 2560, 1024)):
        x, w = _rand(M, N, K, 5 + M)
        gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
        wc, ws = _quant_gpu(w, gw)
        gxt = torch.tensor([gx], dtype=torch.float32, device="cuda")
        alpha = torch.tensor([1.0 / (np.float32(gx) * np.float32(gw))], dtype=torch.float32, device="cuda")
        xd = x.cuda()
        xc, xs = scaled_fp4_quant(xd, gxt)
        ref = cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16)
        assert last_gemm_status() == 0
        assert torch.equal(nvfp4_linear(xd, gxt, wc, ws, alpha), ref)
        wide = torch.zeros(M, K + 64, dtype=torch.bfloat16, device="cuda")
        wide[:, :K] = xd
        assert torch.equal(nvfp4_linear(wide[:, :K], gxt, wc, ws, alpha), ref)
    with pytest.raises(RuntimeError):
        nvfp4_linear(xd.float(), gxt, wc, ws, alpha)


def test_prefill_config_m128_full_weight():
    # dense prefill configuration at M=128: N=14336, K=4096, checked in full
    out, ref, status = _run(*_rand(128, 14336, 4096, 11))
    assert status == 0
    assert rel_err(out, ref) < TOL


def test_prefill_config_m4096_sampled_rows_and_linearity():
    # full size (M=4096): 48 sampled rows against the oracle, plus a size-independent property:
    # scaling alpha scales the output
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm
    x, w = _rand(4096, 14336, 4096, 12)
    gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
    xc, xs = _quant_gpu(x, gx)
    wc, ws = _quant_gpu(w, gw)
    a1 = torch.tensor([1.0 / (gx * gw)], dtype=torch.float32, device="cuda")
    out = cutlass_scaled_fp4_mm(xc, wc, xs, ws, a1, torch.bfloat16)
    rows = np.random.default_rng(0).choice(4096, 48, replace=False)
    xcl, xsl = _quant_gpu(x, gx, False)
    wcl, wsl = _quant_gpu(w, gw, False)
    xd = oracle.dequantize(to_np(xcl)[rows], to_np(xsl)[rows], gx)
    wd = oracle.dequantize(to_np(wcl), to_np(wsl), gw)
    ref = oracle.matmul_nt(xd, wd)
    assert rel_err(to_np(out[torch.from_numpy(rows).cuda()]), ref) < TOL
    out2 = cutlass_scaled_fp4_mm(xc, wc, xs, ws, a1 * 2, torch.bfloat16)
    assert torch.equal(out2.float(), out.float() * 2)


def test_torch_custom_ops_dispatch_to_the_library():
    import dgx_vllm_b200.torch_ops  # noqa: F401
    x, w = _rand(32, 128, 256, 9)
    gx, gw = float(oracle.global_scale(x.float().numpy())), float(oracle.global_scale(w.float().numpy()))
    g = lambda v: torch.tensor([v], dtype=torch.float32, device="cuda")
    xc, xs = torch.ops.b200_nvfp4.scaled_fp4_quant(x.cuda(), g(gx), True)
    wc, ws = torch.ops.b200_nvfp4.scaled_fp4_quant(w.cuda(), g(gw), True)
    out = torch.empty(32, 128, dtype=torch.bfloat16, device="cuda")
    torch.ops.b200_nvfp4.cutlass_scaled_fp4_mm(out, xc, wc, xs, ws, g(1.0 / (gx * gw)))
    oc, osf = oracle.quantize_bf16(bf16_bits(x), gx)
    wq, wsf = oracle.quantize_bf16(bf16_bits(w), gw)
    ref = oracle.matmul_nt(oracle.dequantize(oc, osf, gx), oracle.dequantize(wq, wsf, gw))
    assert rel_err(to_np(out), ref) < TOL
