"""The CPU oracle against the golden vectors produced by the reference's own Python
(tests/golden/make_golden.py) and against the reference's published tables."""
import os

import numpy as np
import pytest

import oracle


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_e2m1_threshold_table():
    # patch_nvfp4_utils_sw_e2m1.py:37-44 -- ties go to the even mantissa, saturate at 6
    cases = [(0.0, 0), (0.25, 0), (0.26, 1), (0.5, 1), (0.74, 1), (0.75, 2), (1.0, 2), (1.25, 2), (1.26, 3),
             (1.74, 3), (1.75, 4), (2.5, 4), (2.51, 5), (3.49, 5), (3.5, 6), (5.0, 6), (5.01, 7), (6.0, 7),
             (1e9, 7)]
    for x, code in cases:
        assert oracle.e2m1_encode(x) == code, x
        assert oracle.e2m1_encode(-x) == (code | 8), x
    assert oracle.e2m1_encode(-0.0) == 8


def test_e2m1_decode_lut():
    # sparse_fp4_kernel/sparse_fp4_v7.cu:25-28
    lut = [0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6]
    for c, v in enumerate(lut):
        assert oracle.e2m1_decode(c) == v
    assert not np.signbit(np.float32(oracle.e2m1_decode(8)))


def test_cast_to_fp4_golden(golden_dir):
    g = _load(golden_dir, "codec.npz")
    got = np.array([oracle.e2m1_decode(oracle.e2m1_encode(float(x))) for x in g["probe"]], np.float32)
    np.testing.assert_array_equal(got, g["cast"])


def test_break_fp4_bytes_golden(golden_dir):
    g = _load(golden_dir, "codec.npz")
    b = g["break_in"]
    sf = np.full((b.shape[0], b.shape[1] * 2 // 16), oracle.e4m3_encode(1.0), np.uint8)
    np.testing.assert_array_equal(oracle.dequantize(b, sf, 1.0), g["break_out"])


def test_e4m3_codec_roundtrip_and_torch():
    torch = pytest.importorskip("torch")
    lut = oracle.e4m3_lut()
    t = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    for b in range(256):
        if (b & 0x7F) == 0x7F:
            assert abs(lut[b]) == 480.0  # the reference table decodes the NaN codes as 480
            continue
        assert lut[b] == t[b], b
        assert oracle.e4m3_encode(float(lut[b])) == (b if b != 0x80 else 0x80)
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.uniform(0, 448, 20000), rng.uniform(0, 0.05, 20000), [448.0, 2 ** -9, 2 ** -10,
                        3 * 2 ** -10, 0.0]]).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([oracle.e4m3_encode(float(v)) for v in x], np.uint8)
    np.testing.assert_array_equal(got, ref)


def test_sf_swizzle_golden(golden_dir):
    g = _load(golden_dir, "codec.npz")
    M, KB = int(g["swz_M"]), int(g["swz_KB"])
    lin_idx = g["swz_linear_index"]          # lin_idx[m,kb] = byte offset in the swizzled buffer
    for m in range(M):
        for kb in range(KB):
            assert oracle.lib().orc_sf_swizzled_offset(m, kb, KB) == lin_idx[m, kb]
    lin = np.random.default_rng(0).integers(0, 255, (M, KB), dtype=np.uint8)
    swz = oracle.sf_linear_to_swizzled(lin)
    assert swz.size == oracle.sf_swizzled_bytes(M, KB)
    np.testing.assert_array_equal(oracle.sf_swizzled_to_linear(swz, M, KB), lin)


@pytest.mark.parametrize("name", ["amax", "one", "big", "tiny"])
def test_quantizer_kat_golden(golden_dir, name):
    g = _load(golden_dir, "quant_kat.npz")
    x = g["x_bits"]
    codes, sf = oracle.quantize_bf16(x, float(g[f"gs_{name}"][0]))
    np.testing.assert_array_equal(sf, g[f"sf_{name}"])
    np.testing.assert_array_equal(oracle.e4m3_lut()[sf], g[f"sf_f32_{name}"])
    # values agree everywhere; codes agree except the sign nibble of an exact -0.0 input, where
    # the reference's software E2M1 keeps the sign bit and the torch emulation drops it
    sf_one = np.full_like(sf, oracle.e4m3_encode(1.0))
    np.testing.assert_array_equal(oracle.dequantize(codes, sf_one, 1.0), g[f"values_{name}"])
    neg_zero_in = (x == 0x8000)
    lo, hi = codes & 15, codes >> 4
    glo, ghi = g[f"codes_{name}"] & 15, g[f"codes_{name}"] >> 4
    assert np.all((lo == glo) | neg_zero_in[:, 0::2])
    assert np.all((hi == ghi) | neg_zero_in[:, 1::2])
    assert np.all(lo[neg_zero_in[:, 0::2]] == 8)


def test_dense_c1_golden(golden_dir):
    g = _load(golden_dir, "dense_c1.npz")
    gs_x, gs_w = float(g["gs_x"][0]), float(g["gs_w"][0])
    codes, sf = oracle.quantize_bf16(g["x_bits"], gs_x)
    np.testing.assert_array_equal(codes, g["x_codes"])
    np.testing.assert_array_equal(sf, g["x_sf"])
    ref = oracle.bf16_bits_to_f32(g["out_bits"])
    # the reference's emulation: operands rounded to bf16, bf16 matmul, bf16 result
    emu = oracle.nvfp4_linear(g["x_bits"], gs_x, g["w_codes"], g["w_sf"], gs_w, round_bf16=True)
    assert np.max(np.abs(emu - ref)) / np.max(np.abs(ref)) < 2 ** -7      # one bf16 output rounding
    # the fp32 dequantize-then-matmul yardstick is within the path's 1e-2 tolerance of it
    exact = oracle.nvfp4_linear(g["x_bits"], gs_x, g["w_codes"], g["w_sf"], gs_w)
    assert np.max(np.abs(exact - ref)) / np.max(np.abs(ref)) < 1e-2
    # quantize_f32 on the stored fp32 weight rows reproduces the reference's weight codes
    wc, ws = oracle.quantize_f32(g["w_f32_first_rows"], gs_w)
    np.testing.assert_array_equal(wc, g["w_codes"][:4])
    np.testing.assert_array_equal(ws, g["w_sf"][:4])
    small = oracle.matmul_nt(np.ones((2, 32), np.float32), np.ones((3, 32), np.float32), exact_c_loop=True)
    np.testing.assert_array_equal(small, np.full((2, 3), 32, np.float32))


def test_sparse_convert_golden(golden_dir):
    g = _load(golden_dir, "sparse_convert.npz")
    comp, meta = oracle.sparse_2of4_pack(g["codes"])
    nib = g["nibbles"]                                   # [N,K]
    N, K = nib.shape
    mag = np.abs(oracle.E2M1_LUT[nib]).reshape(N, K // 4, 4)
    srt = np.sort(mag, axis=2)
    tie_free = (srt[:, :, 1] != srt[:, :, 2]).T          # [K/4,N]: 2nd and 3rd largest differ
    assert tie_free.mean() > 0.3
    np.testing.assert_array_equal(comp[tie_free], g["comp_T"][tie_free])
    m2 = np.stack([meta & 15, meta >> 4], axis=1).reshape(K // 4, N)
    r2 = np.stack([g["meta_T"] & 15, g["meta_T"] >> 4], axis=1).reshape(K // 4, N)
    np.testing.assert_array_equal(m2[tie_free], r2[tie_free])
    # at ties both choices keep the same magnitudes: dense expansions agree in |W|
    ones = np.full((K // 16, N), oracle.e4m3_encode(1.0), np.uint8)
    W = oracle.sparse_expand(comp, meta, ones, 1.0)
    Wr = oracle.sparse_expand(g["comp_T"], g["meta_T"], ones, 1.0)
    np.testing.assert_array_equal(np.sort(np.abs(W).reshape(N, K // 4, 4), 2), np.sort(np.abs(Wr).reshape(N, K // 4, 4), 2))
    assert np.all((W != 0).reshape(N, K // 4, 4).sum(2) <= 2)
    # kept values are the original ones at their original positions
    dense = oracle.E2M1_LUT[nib]
    assert np.all((W == 0) | (W == dense))
    np.testing.assert_array_equal(g["scale_T"], g["sf"].T)


def test_sparse_gemv_oracle_matches_reference_loop():
    # the element loop of sparse_fp4_kernel/bench_v7_scaled.py:178-201, on a tiny case
    rng = np.random.default_rng(3)
    E, K, N, P = 3, 32, 8, 4
    comp = rng.integers(0, 256, (E, K // 4, N), dtype=np.uint8)
    meta = rng.integers(0, 256, (E, K // 8, N), dtype=np.uint8)
    for G in (K // 8, K // 16):
        scale = rng.integers(56, 120, (E, G, N), dtype=np.uint8)
        gsc = (rng.random(E) * 1e-3 + 1e-4).astype(np.float32)
        ids = np.array([2, 0, 1, 2], np.int32)
        A = rng.standard_normal((P, K)).astype(np.float16).astype(np.float32)
        got = oracle.batched_sparse_gemv(A, comp, meta, scale, gsc, ids)
        ref = np.zeros((P, N))
        for p in range(P):
            e = ids[p]
            for gi in range(0, K // 4, 2):
                mi = gi // 2
                si = mi // ((K // 8) // G)
                for n in range(N):
                    c0, c1, mt = int(comp[e, gi, n]), int(comp[e, gi + 1, n]), int(meta[e, mi, n])
                    s = oracle.e4m3_decode(scale[e, si, n]) * float(gsc[e])
                    lut = oracle.E2M1_LUT
                    ref[p, n] += lut[c0 & 15] * s * A[p, gi * 4 + (mt & 3)]
                    ref[p, n] += lut[c0 >> 4] * s * A[p, gi * 4 + ((mt >> 2) & 3)]
                    ref[p, n] += lut[c1 & 15] * s * A[p, gi * 4 + 4 + ((mt >> 4) & 3)]
                    ref[p, n] += lut[c1 >> 4] * s * A[p, gi * 4 + 4 + ((mt >> 6) & 3)]
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-9)
