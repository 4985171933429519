/*
 * CPU oracle for the NVFP4 hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the arithmetic the reference (Avarok-Cybersecurity/dgx-vllm)
 * uses on its NVFP4 path.  Only the tests, the smoke check and the CPU-baseline leg of the
 * benchmark may link or call this file; the shipped library never does.
 *
 * Parity status: PINNED for the quantizer, the E2M1/E4M3 codecs, the scale-factor swizzle and
 * the dense dequantize-then-matmul, against (a) the reference's own E2M1 threshold table and
 * decode LUTs and (b) golden vectors produced by running the reference's emulation path
 * (fix_nvfp4_emulation_backend.py:60-102 on top of vLLM's ref_nvfp4_quant / break_fp4_bytes)
 * in the build container; see tests/golden/make_golden.py.  PINNED for the 2:4 sparse format
 * against goldens produced by the reference's converter (sparse_v7_moe_patch.py:39-129).
 * UNPINNED for the grouped MoE GEMM: the reference has no test or vector for that boundary;
 * the oracle there is a per-expert loop over the pinned dense oracle.
 *
 * Every function cites the reference file:line it restates (paths relative to the reference
 * project root; "vllm/..." = the third-party vLLM tree the reference patches).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ bf16 / fp16 helpers */

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even float -> bf16 (what torch .to(bfloat16) does for finite values) */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

ORC_API float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
ORC_API uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }

/* ------------------------------------------------------------------ E2M1 */

/* float -> 4-bit E2M1 code, round-to-nearest-even, saturating at 6.0, sign bit kept for -0.
 * Restates _sw_float_to_e2m1, patch_nvfp4_utils_sw_e2m1.py:31-46 (same thresholds as vLLM
 * cast_to_fp4, vllm/model_executor/layers/quantization/utils/nvfp4_emulation_utils.py:425-436). */
ORC_API uint8_t orc_e2m1_encode(float x) {
  uint32_t bits;
  memcpy(&bits, &x, 4);
  uint8_t sign = (uint8_t)((bits >> 28) & 8u);
  float ax = fabsf(x);
  uint8_t mag;
  if (ax <= 0.25f) mag = 0;
  else if (ax < 0.75f) mag = 1;
  else if (ax <= 1.25f) mag = 2;
  else if (ax < 1.75f) mag = 3;
  else if (ax <= 2.5f) mag = 4;
  else if (ax < 3.5f) mag = 5;
  else if (ax <= 5.0f) mag = 6;
  else mag = 7;
  return sign | mag;
}

/* 4-bit code -> float.  Restates c_fp4_lut, sparse_fp4_kernel/sparse_fp4_v7.cu:25-28
 * (code 8 decodes to +0.0) and kE2M1ToFloat, vllm/.../nvfp4_emulation_utils.py:20-22. */
static const float k_e2m1_lut[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                     0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
ORC_API float orc_e2m1_decode(uint8_t code) { return k_e2m1_lut[code & 15]; }

/* ------------------------------------------------------------------ E4M3FN */

/* byte -> float.  Restates fp8_e4m3fn_to_float_host, sparse_fp4_v7.cu:34-50: subnormals are
 * 2^-6 * m/8 and the two NaN encodings 0x7F/0xFF decode as +-480 exactly as that table does. */
ORC_API float orc_e4m3_decode(uint8_t b) {
  uint32_t sign = (b >> 7) & 1u, e = (b >> 3) & 0xFu, m = b & 7u;
  float v;
  if (e == 0) v = ldexpf((float)m / 8.0f, -6);
  else v = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
  return sign ? -v : v;
}

/* float -> e4m3fn byte, round-to-nearest-even, finite saturation at 448.  This is the
 * `.to(torch.float8_e4m3fn)` step of ref_nvfp4_quant (vllm/.../nvfp4_emulation_utils.py:446)
 * after its clamp to +-448. */
ORC_API uint8_t orc_e4m3_encode(float x) {
  uint32_t bits;
  memcpy(&bits, &x, 4);
  uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
  float ax = fabsf(x);
  if (ax != ax) return (uint8_t)(sign | 0x7F);
  if (ax >= 448.0f) {
    return (uint8_t)(sign | 0x7E);
  }
  if (ax < 0.015625f) { /* below 2^-6: subnormal grid of 2^-9 */
    int q = (int)nearbyintf(ax * 512.0f);
    return (uint8_t)(sign | (uint8_t)q); /* q == 8 lands on the smallest normal, code 0x08 */
  }
  int e;
  float fr = frexpf(ax, &e); /* ax = fr * 2^e, fr in [0.5,1) */
  float mant = fr * 2.0f;    /* [1,2) */
  e -= 1;
  int q = (int)nearbyintf((mant - 1.0f) * 8.0f);
  if (q == 8) {
    q = 0;
    e += 1;
  }
  int code = ((e + 7) << 3) | q;
  if (code > 0x7E) code = 0x7E;
  return (uint8_t)(sign | (uint8_t)code);
}

/* ------------------------------------------------------------------ quantizer */

/* 1/(x + (x==0)*1e8): get_reciprocal, vllm/.../nvfp4_emulation_utils.py:415-422 */
static inline float ref_reciprocal(float x) { return 1.0f / (x + (x == 0.0f ? 1.0e8f : 0.0f)); }

/* bf16 [M,K] -> packed E2M1 codes [M,K/2] (element 2i in the low nibble) + e4m3 block scales
 * [M,K/16], linear layout.  Operation order follows ref_nvfp4_quant,
 * vllm/.../nvfp4_emulation_utils.py:439-453, as called by the reference at
 * fix_nvfp4_emulation_backend.py:72; code packing follows
 * patch_nvfp4_utils_sw_e2m1.py:48-63.  gs is the "input_global_scale" (= 448*6/amax). */
ORC_API void orc_quantize_bf16(const uint16_t* x, int64_t M, int64_t K, float gs, uint8_t* codes,
                               uint8_t* sf_linear) {
  const float sixth = (float)(1.0 / 6.0);
  const float rcp_gs = ref_reciprocal(gs);
  const int64_t KB = K / 16;
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t kb = 0; kb < KB; ++kb) {
      const uint16_t* px = x + m * K + kb * 16;
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        float a = fabsf(bf16_to_f32(px[i]));
        if (a > amax) amax = a;
      }
      float scale = gs * (amax * sixth);
      if (scale > 448.0f) scale = 448.0f;
      if (scale < -448.0f) scale = -448.0f;
      uint8_t sfb = orc_e4m3_encode(scale);
      float sff = orc_e4m3_decode(sfb);
      float t = sff * rcp_gs;
      float os = ref_reciprocal(t);
      sf_linear[m * KB + kb] = sfb;
      for (int i = 0; i < 16; i += 2) {
        float v0 = bf16_to_f32(px[i]) * os;
        float v1 = bf16_to_f32(px[i + 1]) * os;
        if (v0 > 6.0f) v0 = 6.0f;
        if (v0 < -6.0f) v0 = -6.0f;
        if (v1 > 6.0f) v1 = 6.0f;
        if (v1 < -6.0f) v1 = -6.0f;
        codes[m * (K / 2) + kb * 8 + i / 2] =
            (uint8_t)(orc_e2m1_encode(v0) | (orc_e2m1_encode(v1) << 4));
      }
    }
  }
}

/* Same as above for fp32 input (used to quantize synthetic weights). */
ORC_API void orc_quantize_f32(const float* x, int64_t M, int64_t K, float gs, uint8_t* codes,
                              uint8_t* sf_linear) {
  const float sixth = (float)(1.0 / 6.0);
  const float rcp_gs = ref_reciprocal(gs);
  const int64_t KB = K / 16;
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t kb = 0; kb < KB; ++kb) {
      const float* px = x + m * K + kb * 16;
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        float a = fabsf(px[i]);
        if (a > amax) amax = a;
      }
      float scale = gs * (amax * sixth);
      if (scale > 448.0f) scale = 448.0f;
      uint8_t sfb = orc_e4m3_encode(scale);
      float os = ref_reciprocal(orc_e4m3_decode(sfb) * rcp_gs);
      sf_linear[m * KB + kb] = sfb;
      for (int i = 0; i < 16; i += 2) {
        float v0 = fminf(fmaxf(px[i] * os, -6.0f), 6.0f);
        float v1 = fminf(fmaxf(px[i + 1] * os, -6.0f), 6.0f);
        codes[m * (K / 2) + kb * 8 + i / 2] =
            (uint8_t)(orc_e2m1_encode(v0) | (orc_e2m1_encode(v1) << 4));
      }
    }
  }
}

/* Byte offset of scale factor (m, kb) inside the padded 128x4 swizzled layout
 * [ceil(M/128), ceil(KB/4), 32, 4, 4]; the inverse permutation is convert_swizzled_to_linear,
 * vllm/.../nvfp4_emulation_utils.py:348-355. */
ORC_API int64_t orc_sf_swizzled_offset(int64_t m, int64_t kb, int64_t KB) {
  int64_t KT = (KB + 3) / 4;
  return ((((m / 128) * KT + kb / 4) * 32 + (m % 32)) * 4 + (m % 128) / 32) * 4 + (kb % 4);
}

ORC_API int64_t orc_sf_swizzled_bytes(int64_t M, int64_t KB) {
  return ((M + 127) / 128) * 128 * ((KB + 3) / 4) * 4;
}

ORC_API void orc_sf_linear_to_swizzled(const uint8_t* lin, int64_t M, int64_t KB, uint8_t* swz) {
  memset(swz, 0, (size_t)orc_sf_swizzled_bytes(M, KB));
  for (int64_t m = 0; m < M; ++m)
    for (int64_t kb = 0; kb < KB; ++kb) swz[orc_sf_swizzled_offset(m, kb, KB)] = lin[m * KB + kb];
}

ORC_API void orc_sf_swizzled_to_linear(const uint8_t* swz, int64_t M, int64_t KB, uint8_t* lin) {
  for (int64_t m = 0; m < M; ++m)
    for (int64_t kb = 0; kb < KB; ++kb) lin[m * KB + kb] = swz[orc_sf_swizzled_offset(m, kb, KB)];
}

/* ------------------------------------------------------------------ dequantize + matmul */

/* codes [M,K/2] + linear e4m3 scales [M,K/16] -> fp32 [M,K], value = lut[code]*sf/gs.
 * Restates the dequantisation at fix_nvfp4_emulation_backend.py:75-77 (activations) and :89-97
 * (weights: break_fp4_bytes, linear scales, divide by the global scale).  If round_bf16 != 0
 * the result is rounded to bf16 as the reference does with `.to(output_dtype)`. */
ORC_API void orc_dequantize(const uint8_t* codes, const uint8_t* sf_linear, float gs, int64_t M,
                            int64_t K, int round_bf16, float* out) {
  const int64_t KB = K / 16;
  for (int64_t m = 0; m < M; ++m)
    for (int64_t kb = 0; kb < KB; ++kb) {
      float s = orc_e4m3_decode(sf_linear[m * KB + kb]) / gs;
      for (int i = 0; i < 8; ++i) {
        uint8_t b = codes[m * (K / 2) + kb * 8 + i];
        float v0 = k_e2m1_lut[b & 15] * s, v1 = k_e2m1_lut[b >> 4] * s;
        if (round_bf16) {
          v0 = bf16_to_f32(f32_to_bf16(v0));
          v1 = bf16_to_f32(f32_to_bf16(v1));
        }
        out[m * K + kb * 16 + 2 * i] = v0;
        out[m * K + kb * 16 + 2 * i + 1] = v1;
      }
    }
}

/* C[M,N] = A[M,K] . B[N,K]^T with double accumulation: the "FP32 dequantize-then-matmul"
 * yardstick (same formula as reference_gemm_fp4, cutlass_nvfp4/test_nvfp4_gemm.cu:22-66, and
 * torch.matmul(x_dq, w_dq.t()) at fix_nvfp4_emulation_backend.py:100). */
ORC_API void orc_matmul_nt(const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                           float* C) {
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      const float* a = A + m * K;
      const float* b = B + n * K;
      double acc = 0.0;
      for (int64_t k = 0; k < K; ++k) acc += (double)a[k] * (double)b[k];
      C[m * N + n] = (float)acc;
    }
}

/* ------------------------------------------------------------------ 2:4 sparse format */

/* NVFP4 codes [N,K/2] -> 2:4 compressed form, transposed so that N is contiguous:
 * comp_T [K/4,N] (low nibble = first kept value, high nibble = second), meta_T [K/8,N]
 * (i0g0 | i1g0<<2 | i0g1<<4 | i1g1<<6).  Restates unpack_fp4_nibbles + apply_2of4_sparsity_fast
 * + the transposes of convert_expert_to_v7_gpu, sparse_fp4_kernel/sparse_v7_moe_patch.py:39-93.
 * The reference picks the two largest magnitudes with torch.topk, whose order among equal
 * magnitudes is unspecified; this restatement fixes the rule: larger magnitude first, then the
 * lower index.  Kept indices are stored ascending, as the reference's sort does. */
ORC_API void orc_sparse_2of4_pack(const uint8_t* codes, int64_t N, int64_t K, uint8_t* comp_T,
                                  uint8_t* meta_T) {
  for (int64_t n = 0; n < N; ++n)
    for (int64_t g = 0; g < K / 4; ++g) {
      uint8_t nib[4];
      float mag[4];
      for (int j = 0; j < 4; ++j) {
        int64_t k = g * 4 + j;
        uint8_t b = codes[n * (K / 2) + k / 2];
        nib[j] = (k & 1) ? (b >> 4) : (b & 15);
        mag[j] = fabsf(k_e2m1_lut[nib[j]]);
      }
      int a = 0;
      for (int j = 1; j < 4; ++j)
        if (mag[j] > mag[a]) a = j;
      int b2 = -1;
      for (int j = 0; j < 4; ++j) {
        if (j == a) continue;
        if (b2 < 0 || mag[j] > mag[b2]) b2 = j;
      }
      int i0 = a < b2 ? a : b2, i1 = a < b2 ? b2 : a;
      comp_T[g * N + n] = (uint8_t)(nib[i0] | (nib[i1] << 4));
      uint8_t* mp = &meta_T[(g / 2) * N + n];
      if ((g & 1) == 0) *mp = (uint8_t)(i0 | (i1 << 2));
      else *mp = (uint8_t)(*mp | (i0 << 4) | (i1 << 6));
    }
}

/* Expand one expert's 2:4 tensors to a dense fp32 W[N,K]:
 * W[n, 4g+idx] = lut[nibble] * e4m3(scale_T[kb', n]) * g_scale, scale row kb' = (k/8)/((K/8)/G).
 * Restates the reference check in sparse_fp4_kernel/bench_v7_scaled.py:165-201 and
 * test_real_weights.py:239-257, and the kernel's indexing at sparse_fp4_v7.cu:187,210-235. */
ORC_API void orc_sparse_expand(const uint8_t* comp_T, const uint8_t* meta_T, const uint8_t* scale_T,
                               float g_scale, int64_t N, int64_t K, int64_t G, float* W) {
  memset(W, 0, sizeof(float) * (size_t)(N * K));
  int64_t pairs_per_scale = (K / 8) / G;
  for (int64_t g = 0; g < K / 4; ++g)
    for (int64_t n = 0; n < N; ++n) {
      uint8_t c = comp_T[g * N + n];
      uint8_t mt = meta_T[(g / 2) * N + n];
      int sh = (g & 1) ? 4 : 0;
      int i0 = (mt >> sh) & 3, i1 = (mt >> (sh + 2)) & 3;
      float s = orc_e4m3_decode(scale_T[((g / 2) / pairs_per_scale) * N + n]) * g_scale;
      /* += so that a (malformed) repeated index behaves like the kernel's sum */
      W[n * K + g * 4 + i0] += k_e2m1_lut[c & 15] * s;
      W[n * K + g * 4 + i1] += k_e2m1_lut[c >> 4] * s;
    }
}

/* Expand one expert's dense transposed tensors B_dense_T [K/2,N] (sparse_fp4_v7.cu:67-149):
 * byte (r, n) holds W[n,2r] in the low and W[n,2r+1] in the high nibble. */
ORC_API void orc_dense_T_expand(const uint8_t* dense_T, const uint8_t* scale_T, float g_scale,
                                int64_t N, int64_t K, int64_t G, float* W) {
  int64_t k_per_scale = K / G;
  for (int64_t r = 0; r < K / 2; ++r)
    for (int64_t n = 0; n < N; ++n) {
      uint8_t c = dense_T[r * N + n];
      float s = orc_e4m3_decode(scale_T[((2 * r) / k_per_scale) * N + n]) * g_scale;
      W[n * K + 2 * r] = k_e2m1_lut[c & 15] * s;
      W[n * K + 2 * r + 1] = k_e2m1_lut[c >> 4] * s;
    }
}

/* SiLU(gate)*up on [P,2I] -> [P,I] (silu_mul_kernel, sparse_fp4_v7.cu:541-554). */
ORC_API void orc_silu_mul(const float* x, int64_t P, int64_t I, float* out) {
  for (int64_t p = 0; p < P; ++p)
    for (int64_t i = 0; i < I; ++i) {
      float g = x[p * 2 * I + i], u = x[p * 2 * I + I + i];
      out[p * I + i] = g / (1.0f + expf(-g)) * u;
    }
}
