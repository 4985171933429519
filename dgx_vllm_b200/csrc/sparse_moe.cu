// 2:4-sparse NVFP4 batched GEMV and the fused MoE decode layer for sm_100a.
//
// Replaces sparse_fp4_kernel/sparse_fp4_v7.cu of the reference with a different execution plan:
//   * a one-block "plan" kernel groups the (token, expert) pairs by expert, so each expert's
//     weights are streamed from HBM once per layer instead of once per pair;
//   * a persistent GEMV kernel walks (expert, 128-column slab) work items.  Each thread owns 16
//     output columns (one 16-byte load per weight row) and one of 32 K-slices; the K reduction is
//     done in-kernel with warp shuffles plus one shared-memory pass, so no partial-sum tensor and
//     no second reduction kernel exist;
//   * E2M1 byte -> half2 and metadata byte -> byte-permute selector decoding go through two
//     bank-replicated shared-memory tables, the 2:4 gather of the activation is one PRMT, and the
//     products run as packed half2 FMAs with fp32 accumulation per 16-element scale block;
//   * SiLU(gate)*up is fused into the gate_up epilogue and the router-weighted sum is one small
//     deterministic kernel (no atomics).
#include "common.cuh"

namespace b200fp4 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSlabCols = 128;   // output columns per work item
constexpr int kKSlices = 32;     // K-slices per block (4 per warp)
constexpr int kMaxTok = 4;       // tokens of one expert processed per pass over its weights
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxExperts = 4096;

// Where one projection's weights live.  Row r of the compressed tensor for expert e and column n:
//   comp  + e*comp_e  + (r/2)*comp_pair + (r&1)*comp_odd + n
//   meta  + e*meta_e  + (r/2)*meta_row + n            (one metadata row per two compressed rows)
//   scale + e*scale_e + srow*scale_row + n
// which covers both the separate tensors (sparse_fp4_v7.cu:158-167) and the interleaved
// [E, K/8, 4N] tensor (sparse_fp4_v7.cu:246-251).
struct SparseWeights {
  const uint8_t* comp;
  const uint8_t* meta;
  const uint8_t* scale;
  const float* g;
  int64_t comp_e, comp_pair, comp_odd;
  int64_t meta_e, meta_row;
  int64_t scale_e, scale_row;
};

struct Plan {
  int* n_unique;     // [1]
  int* uniq_expert;  // [U]
  int* uniq_start;   // [U+1]
  int* pairs;        // [P]  pair indices grouped by expert
  int* mapped;       // [P]  local expert id of each pair, or -1
};

struct GemvArgs {
  SparseWeights w;
  Plan plan;
  const void* A;  // [rows, K]; the row of pair p is p / a_div
  int64_t lda;
  int a_div;
  int a_bf16;
  void* out;      // [P, N] (or [P, N/2] in SiLU mode), leading dimension ldo
  int64_t ldo;
  int out_dtype;
  int N, K;
  int n_slabs;
  int inter;      // SiLU mode: gate columns [0, inter), up columns [inter, 2*inter)
};

// ------------------------------------------------------------------------------------------ plan

__global__ void __launch_bounds__(kPlanThreads)
    moe_plan_kernel(const int32_t* __restrict__ ids, int P, const int32_t* __restrict__ expert_map, int global_E, int E,
                    Plan plan) {
  __shared__ int s_count[kPlanMaxExperts];
  __shared__ int s_warp_a[32], s_warp_b[32];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += kPlanThreads) s_count[e] = 0;
  __syncthreads();
  for (int p = tid; p < P; p += kPlanThreads) {
    int e = ids[p];
    if (expert_map != nullptr) e = (e >= 0 && e < global_E) ? expert_map[e] : -1;
    if (e < 0 || e >= E) e = -1;
    plan.mapped[p] = e;
    if (e >= 0) atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  // exclusive scan over experts of (count, count > 0); each thread owns a contiguous run
  const int per = (E + kPlanThreads - 1) / kPlanThreads;
  const int e0 = tid * per;
  int sum_c = 0, sum_f = 0;
  for (int i = 0; i < per; ++i) {
    int e = e0 + i;
    if (e < E) {
      sum_c += s_count[e];
      sum_f += s_count[e] > 0;
    }
  }
  int inc_c = sum_c, inc_f = sum_f;
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int a = __shfl_up_sync(0xffffffffu, inc_c, d);
    int b = __shfl_up_sync(0xffffffffu, inc_f, d);
    if (lane >= d) {
      inc_c += a;
      inc_f += b;
    }
  }
  if (lane == 31) {
    s_warp_a[warp] = inc_c;
    s_warp_b[warp] = inc_f;
  }
  __syncthreads();
  if (warp == 0) {
    int a = s_warp_a[lane], b = s_warp_b[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int x = __shfl_up_sync(0xffffffffu, a, d);
      int y = __shfl_up_sync(0xffffffffu, b, d);
      if (lane >= d) {
        a += x;
        b += y;
      }
    }
    s_warp_a[lane] = a;
    s_warp_b[lane] = b;
  }
  __syncthreads();
  int base_c = inc_c - sum_c + (warp > 0 ? s_warp_a[warp - 1] : 0);
  int base_f = inc_f - sum_f + (warp > 0 ? s_warp_b[warp - 1] : 0);
  for (int i = 0; i < per; ++i) {
    int e = e0 + i;
    if (e < E) {
      int c = s_count[e];
      if (c > 0) {
        plan.uniq_expert[base_f] = e;
        plan.uniq_start[base_f] = base_c;
        ++base_f;
      }
      s_count[e] = base_c;  // becomes the scatter cursor
      base_c += c;
    }
  }
  if (tid == kPlanThreads - 1) {
    plan.n_unique[0] = base_f;
    plan.uniq_start[base_f] = base_c;
  }
  __syncthreads();
  for (int p = tid; p < P; p += kPlanThreads) {
    int e = plan.mapped[p];
    if (e >= 0) plan.pairs[atomicAdd(&s_count[e], 1)] = p;
  }
}

// ------------------------------------------------------------------------------------------ tables

__device__ __forceinline__ uint32_t e2m1_to_half_bits(uint32_t nib) {
  const uint32_t c = nib & 7u;
  uint32_t h = (c == 0) ? 0u : (c == 1 ? 0x3800u : 0x3800u + c * 0x200u);
  if (c != 0) h |= (nib & 8u) << 12;
  return h;
}

// table[b][lane]: 32 copies of every entry, one per bank, so that 32 lanes looking up 32 different
// bytes never conflict.  Writes are rotated by the thread index for the same reason.
__device__ __forceinline__ void fill_tables(uint32_t* lut_c, uint32_t* lut_m, int tid) {
  for (int b = tid; b < 256; b += kThreads) {
    const uint32_t vc = e2m1_to_half_bits(b & 15) | (e2m1_to_half_bits(b >> 4) << 16);
    const uint32_t i0 = b & 3, i1 = (b >> 2) & 3, i2 = (b >> 4) & 3, i3 = (b >> 6) & 3;
    const uint32_t s0 = (2 * i0) | ((2 * i0 + 1) << 4) | ((2 * i1) << 8) | ((2 * i1 + 1) << 12);
    const uint32_t s1 = (2 * i2) | ((2 * i2 + 1) << 4) | ((2 * i3) << 8) | ((2 * i3 + 1) << 12);
    const uint32_t vm = s0 | (s1 << 16);
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
      const int l = (i + tid) & 31;
      lut_c[b * 32 + l] = vc;
      lut_m[b * 32 + l] = vm;
    }
  }
}

// ------------------------------------------------------------------------------------------ GEMV

struct BlockLoads {
  uint4 c[4];  // four compressed rows (16 k) x 16 columns
  uint4 m[2];  // two metadata rows
  uint4 s[2];  // scale row(s): s[1] is used only with one scale per 8 k
};

template <bool kScale8>
__device__ __forceinline__ void load_block(BlockLoads& L, const uint8_t* comp, const uint8_t* meta,
                                           const uint8_t* scale, const SparseWeights& w, int kb, bool ok) {
  if (ok) {
    const uint8_t* c0 = comp + (int64_t)(2 * kb) * w.comp_pair;
    L.c[0] = ldg_stream_u4(c0);
    L.c[1] = ldg_stream_u4(c0 + w.comp_odd);
    L.c[2] = ldg_stream_u4(c0 + w.comp_pair);
    L.c[3] = ldg_stream_u4(c0 + w.comp_pair + w.comp_odd);
    const uint8_t* m0 = meta + (int64_t)(2 * kb) * w.meta_row;
    L.m[0] = ldg_stream_u4(m0);
    L.m[1] = ldg_stream_u4(m0 + w.meta_row);
    if (kScale8) {
      const uint8_t* s0 = scale + (int64_t)(2 * kb) * w.scale_row;
      L.s[0] = ldg_stream_u4(s0);
      L.s[1] = ldg_stream_u4(s0 + w.scale_row);
    } else {
      L.s[0] = ldg_stream_u4(scale + (int64_t)kb * w.scale_row);
    }
  } else {
    L.c[0] = L.c[1] = L.c[2] = L.c[3] = L.m[0] = L.m[1] = L.s[0] = L.s[1] = make_uint4(0, 0, 0, 0);
  }
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int q) {
  return q == 0 ? v.x : (q == 1 ? v.y : (q == 2 ? v.z : v.w));
}

// byte j of w, shifted left by 7 (the row pitch of the replicated tables), masked.
template <int J>
__device__ __forceinline__ uint32_t byte_shl7(uint32_t w, uint32_t mask) {
  return (J == 0 ? (w << 7) : (w >> (8 * J - 7))) & mask;
}

__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

template <int T, bool kScale8>
__device__ __forceinline__ void compute_block(const BlockLoads& L, const uint4 (&a)[T][2], const uint32_t* lut_c,
                                              const uint32_t* lut_m, float (&acc)[T][16]) {
  // lut_c / lut_m already include this lane's bank offset.
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t c0 = word_of(L.c[0], q), c1 = word_of(L.c[1], q), c2 = word_of(L.c[2], q), c3 = word_of(L.c[3], q);
    const uint32_t m0 = word_of(L.m[0], q), m1 = word_of(L.m[1], q);
    const uint32_t s0 = word_of(L.s[0], q), s1 = kScale8 ? word_of(L.s[1], q) : 0u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t i0, i1, i2, i3, im0, im1, hs0, hs1 = 0;
      // clang-format off
      if (j == 0) { i0 = byte_shl7<0>(c0, 0x7F80u); i1 = byte_shl7<0>(c1, 0x7F80u); i2 = byte_shl7<0>(c2, 0x7F80u); i3 = byte_shl7<0>(c3, 0x7F80u);
                    im0 = byte_shl7<0>(m0, 0x7F80u); im1 = byte_shl7<0>(m1, 0x7F80u); hs0 = byte_shl7<0>(s0, 0x3F80u); if (kScale8) hs1 = byte_shl7<0>(s1, 0x3F80u); }
      if (j == 1) { i0 = byte_shl7<1>(c0, 0x7F80u); i1 = byte_shl7<1>(c1, 0x7F80u); i2 = byte_shl7<1>(c2, 0x7F80u); i3 = byte_shl7<1>(c3, 0x7F80u);
                    im0 = byte_shl7<1>(m0, 0x7F80u); im1 = byte_shl7<1>(m1, 0x7F80u); hs0 = byte_shl7<1>(s0, 0x3F80u); if (kScale8) hs1 = byte_shl7<1>(s1, 0x3F80u); }
      if (j == 2) { i0 = byte_shl7<2>(c0, 0x7F80u); i1 = byte_shl7<2>(c1, 0x7F80u); i2 = byte_shl7<2>(c2, 0x7F80u); i3 = byte_shl7<2>(c3, 0x7F80u);
                    im0 = byte_shl7<2>(m0, 0x7F80u); im1 = byte_shl7<2>(m1, 0x7F80u); hs0 = byte_shl7<2>(s0, 0x3F80u); if (kScale8) hs1 = byte_shl7<2>(s1, 0x3F80u); }
      if (j == 3) { i0 = byte_shl7<3>(c0, 0x7F80u); i1 = byte_shl7<3>(c1, 0x7F80u); i2 = byte_shl7<3>(c2, 0x7F80u); i3 = byte_shl7<3>(c3, 0x7F80u);
                    im0 = byte_shl7<3>(m0, 0x7F80u); im1 = byte_shl7<3>(m1, 0x7F80u); hs0 = byte_shl7<3>(s0, 0x3F80u); if (kScale8) hs1 = byte_shl7<3>(s1, 0x3F80u); }
      // clang-format on
      const __half2 w0 = as_h2(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut_c) + i0));
      const __half2 w1 = as_h2(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut_c) + i1));
      const __half2 w2 = as_h2(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut_c) + i2));
      const __half2 w3 = as_h2(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut_c) + i3));
      const uint32_t sel01 = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut_m) + im0);
      const uint32_t sel23 = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(lut_m) + im1);
      const uint32_t sel1 = sel01 >> 16, sel3 = sel23 >> 16;
      // e4m3 bits placed in a half give scale * 2^-8; the 2^8 is folded into the final multiplier
      const float sc0 = __half2float(__ushort_as_half((unsigned short)hs0));
      const float sc1 = kScale8 ? __half2float(__ushort_as_half((unsigned short)hs1)) : 0.f;
      const int col = q * 4 + j;
#pragma unroll
      for (int t = 0; t < T; ++t) {
        __half2 p = __hmul2(w0, as_h2(prmt(a[t][0].x, a[t][0].y, sel01)));
        p = __hfma2(w1, as_h2(prmt(a[t][0].z, a[t][0].w, sel1)), p);
        if (kScale8) {
          __half2 r = __hmul2(w2, as_h2(prmt(a[t][1].x, a[t][1].y, sel23)));
          r = __hfma2(w3, as_h2(prmt(a[t][1].z, a[t][1].w, sel3)), r);
          acc[t][col] = fmaf(__low2float(p) + __high2float(p), sc0, acc[t][col]);
          acc[t][col] = fmaf(__low2float(r) + __high2float(r), sc1, acc[t][col]);
        } else {
          p = __hfma2(w2, as_h2(prmt(a[t][1].x, a[t][1].y, sel23)), p);
          p = __hfma2(w3, as_h2(prmt(a[t][1].z, a[t][1].w, sel3)), p);
          acc[t][col] = fmaf(__low2float(p) + __high2float(p), sc0, acc[t][col]);
        }
      }
    }
  }
}

template <int T, bool kScale8>
__device__ __forceinline__ void gemv_pass(const GemvArgs& g, const uint8_t* comp, const uint8_t* meta,
                                          const uint8_t* scale, bool col_ok, int kslice, int cg, int ksub, int warp,
                                          const __half* sA, const uint32_t* lut_c, const uint32_t* lut_m, float* red) {
  const int KB = g.K >> 4;
  float acc[T][16];
#pragma unroll
  for (int t = 0; t < T; ++t)
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[t][c] = 0.f;

  BlockLoads cur, nxt;
  int kb = kslice;
  load_block<kScale8>(cur, comp, meta, scale, g.w, kb, col_ok && kb < KB);
  for (; kb < KB; kb += kKSlices) {
    const int kn = kb + kKSlices;
    load_block<kScale8>(nxt, comp, meta, scale, g.w, kn, col_ok && kn < KB);
    uint4 a[T][2];
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const uint4* pa = reinterpret_cast<const uint4*>(sA + (size_t)t * g.K + (size_t)kb * 16);
      a[t][0] = pa[0];
      a[t][1] = pa[1];
    }
    compute_block<T, kScale8>(cur, a, lut_c, lut_m, acc);
    cur = nxt;
  }
  // K reduction: the four K-slices of a warp through shuffles, the eight warps through shared memory
#pragma unroll
  for (int t = 0; t < T; ++t)
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      float v = acc[t][c];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      acc[t][c] = v;
    }
  if (ksub == 0) {
#pragma unroll
    for (int t = 0; t < T; ++t) {
      float4* dst = reinterpret_cast<float4*>(red + ((size_t)warp * kMaxTok + t) * kSlabCols + cg * 16);
#pragma unroll
      for (int c = 0; c < 4; ++c) dst[c] = make_float4(acc[t][4 * c], acc[t][4 * c + 1], acc[t][4 * c + 2], acc[t][4 * c + 3]);
    }
  }
}

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
  if (dtype == B200FP4_DTYPE_F16) reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
  else if (dtype == B200FP4_DTYPE_BF16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[idx] = v;
}

template <bool kScale8, bool kSilu>
__global__ void __launch_bounds__(kThreads, 1) sparse_gemv_kernel(const GemvArgs g) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* lut_c = reinterpret_cast<uint32_t*>(smem);
  uint32_t* lut_m = lut_c + 256 * 32;
  float* red = reinterpret_cast<float*>(lut_m + 256 * 32);            // [kWarps][kMaxTok][kSlabCols]
  __half* sA = reinterpret_cast<__half*>(red + kWarps * kMaxTok * kSlabCols);  // [kMaxTok][K]

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int cg = lane & 7, ksub = lane >> 3;
  const int kslice = warp * 4 + ksub;
  fill_tables(lut_c, lut_m, tid);
  const uint32_t* lut_c_lane = lut_c + lane;
  const uint32_t* lut_m_lane = lut_m + lane;

  const int n_unique = g.plan.n_unique[0];
  const int n_work = n_unique * g.n_slabs;
  for (int work = blockIdx.x; work < n_work; work += gridDim.x) {
    const int u = work / g.n_slabs, slab = work - u * g.n_slabs;
    const int e = g.plan.uniq_expert[u];
    const int p0 = g.plan.uniq_start[u];
    const int np = g.plan.uniq_start[u + 1] - p0;
    // column owned by this thread
    int col0;
    if (kSilu) col0 = (cg < 4) ? slab * 64 + cg * 16 : g.inter + slab * 64 + (cg - 4) * 16;
    else col0 = slab * kSlabCols + cg * 16;
    const bool col_ok = kSilu ? ((cg < 4 ? col0 : col0 - g.inter) < g.inter) : (col0 < g.N);
    const uint8_t* comp = g.w.comp + (int64_t)e * g.w.comp_e + col0;
    const uint8_t* meta = g.w.meta + (int64_t)e * g.w.meta_e + col0;
    const uint8_t* scale = g.w.scale + (int64_t)e * g.w.scale_e + col0;
    const float gmul = g.w.g[e] * 256.0f;

    for (int tc = 0; tc < np; tc += kMaxTok) {
      const int nt = min(kMaxTok, np - tc);
      __syncthreads();  // tables ready (first pass) / previous pass done with sA and red
      // stage the activations of this pass as fp16: sA[t][k]
      const int chunks = g.K >> 3;
      for (int i = tid; i < kMaxTok * chunks; i += kThreads) {
        const int t = i / chunks, ch = i - t * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < nt) {
          const int p = g.plan.pairs[p0 + tc + t];
          const int64_t row = p / g.a_div;
          if (g.a_bf16) {
            const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g.A) + row * g.lda + ch * 8);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            __half2 h[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) h[k] = __float22half2_rn(__bfloat1622float2(b2[k]));
            v = *reinterpret_cast<uint4*>(h);
          } else {
            v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(g.A) + row * g.lda + ch * 8);
          }
        }
        *reinterpret_cast<uint4*>(sA + (size_t)t * g.K + ch * 8) = v;
      }
      __syncthreads();
      if (nt == 1) gemv_pass<1, kScale8>(g, comp, meta, scale, col_ok, kslice, cg, ksub, warp, sA, lut_c_lane, lut_m_lane, red);
      else if (nt == 2) gemv_pass<2, kScale8>(g, comp, meta, scale, col_ok, kslice, cg, ksub, warp, sA, lut_c_lane, lut_m_lane, red);
      else gemv_pass<4, kScale8>(g, comp, meta, scale, col_ok, kslice, cg, ksub, warp, sA, lut_c_lane, lut_m_lane, red);
      __syncthreads();
      // epilogue: sum the eight warps, apply the expert's global scale, write
      if (kSilu) {
        for (int i = tid; i < nt * 64; i += kThreads) {
          const int t = i >> 6, j = i & 63;
          const int n = slab * 64 + j;
          if (n < g.inter) {
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
              gate += red[((size_t)w * kMaxTok + t) * kSlabCols + j];
              up += red[((size_t)w * kMaxTok + t) * kSlabCols + 64 + j];
            }
            gate *= gmul;
            up *= gmul;
            const float act = gate / (1.0f + __expf(-gate)) * up;
            const int p = g.plan.pairs[p0 + tc + t];
            store_out(g.out, g.out_dtype, (int64_t)p * g.ldo + n, act);
          }
        }
      } else {
        for (int i = tid; i < nt * kSlabCols; i += kThreads) {
          const int t = i >> 7, j = i & 127;
          const int n = slab * kSlabCols + j;
          if (n < g.N) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) v += red[((size_t)w * kMaxTok + t) * kSlabCols + j];
            const int p = g.plan.pairs[p0 + tc + t];
            store_out(g.out, g.out_dtype, (int64_t)p * g.ldo + n, v * gmul);
          }
        }
      }
    }
  }
}

// Rows of pairs whose expert is not local are never touched by the GEMV; this writes zeros there.
__global__ void zero_unmapped_rows_kernel(const int* __restrict__ mapped, int P, void* out, int out_dtype, int64_t ldo,
                                          int N) {
  const int p = blockIdx.x;
  if (p >= P || mapped[p] >= 0) return;
  for (int n = threadIdx.x; n < N; n += blockDim.x) store_out(out, out_dtype, (int64_t)p * ldo + n, 0.f);
}

// ------------------------------------------------------------------------------------------ generic

// Scalar kernel for shapes the vectorised kernel does not take (N % 16 != 0, unusual scale group
// counts) and for the dense [E, K/2, N] layout: one thread per (pair, column), fp32 throughout.
// mode 0: 2:4 compressed (SparseWeights addressing); mode 1: dense transposed codes.
__global__ void generic_gemv_kernel(SparseWeights w, int mode, const void* A, int a_bf16, int64_t lda,
                                    const int32_t* __restrict__ expert_ids, int E, void* out, int out_dtype, int P,
                                    int N, int K, int G) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int p = blockIdx.y;
  if (n >= N || p >= P) return;
  const int e = expert_ids[p];
  if (e < 0 || e >= E) {
    store_out(out, out_dtype, (int64_t)p * N + n, 0.f);
    return;
  }
  const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  auto dec = [&](uint32_t nib) { float v = lut[nib & 7]; return (nib & 8) ? -v : v; };
  auto a_at = [&](int k) {
    return a_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(A)[(int64_t)p * lda + k])
                  : __half2float(reinterpret_cast<const __half*>(A)[(int64_t)p * lda + k]);
  };
  float acc = 0.f;
  if (mode == 0) {
    const int pairs_per_scale = (K / 8) / G;
    const uint8_t* comp = w.comp + (int64_t)e * w.comp_e + n;
    const uint8_t* meta = w.meta + (int64_t)e * w.meta_e + n;
    const uint8_t* scale = w.scale + (int64_t)e * w.scale_e + n;
    for (int pr = 0; pr < K / 8; ++pr) {
      const uint32_t c0 = comp[(int64_t)pr * w.comp_pair], c1 = comp[(int64_t)pr * w.comp_pair + w.comp_odd];
      const uint32_t mt = meta[(int64_t)pr * w.meta_row];
      const float s = e4m3_to_f32(scale[(int64_t)(pr / pairs_per_scale) * w.scale_row] & 0x7F);
      const int k0 = pr * 8;
      float sum = dec(c0 & 15) * a_at(k0 + (mt & 3)) + dec(c0 >> 4) * a_at(k0 + ((mt >> 2) & 3)) +
                  dec(c1 & 15) * a_at(k0 + 4 + ((mt >> 4) & 3)) + dec(c1 >> 4) * a_at(k0 + 4 + ((mt >> 6) & 3));
      acc = fmaf(sum, s, acc);
    }
  } else {
    const int k_per_scale = K / G;
    const uint8_t* dense = w.comp + (int64_t)e * w.comp_e + n;
    const uint8_t* scale = w.scale + (int64_t)e * w.scale_e + n;
    for (int r = 0; r < K / 2; ++r) {
      const uint32_t c = dense[(int64_t)r * N];
      const float s = e4m3_to_f32(scale[(int64_t)((2 * r) / k_per_scale) * w.scale_row] & 0x7F);
      acc = fmaf(dec(c & 15) * a_at(2 * r) + dec(c >> 4) * a_at(2 * r + 1), s, acc);
    }
  }
  store_out(out, out_dtype, (int64_t)p * N + n, acc * w.g[e]);
}

// out[m, h] = sum_t weight(m,t) * down[m*topk + t, h] over pairs whose expert is local.
__global__ void weighted_reduce_kernel(const float* __restrict__ down, const float* __restrict__ topk_w,
                                       const int* __restrict__ mapped, void* out, int out_dtype, int M, int topk, int H,
                                       int unweighted) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  const int m = blockIdx.y;
  if (h >= H || m >= M) return;
  float acc = 0.f;
  for (int t = 0; t < topk; ++t) {
    const int p = m * topk + t;
    if (mapped[p] < 0) continue;
    const float v = down[(int64_t)p * H + h];
    acc += unweighted ? v : v * topk_w[p];
  }
  store_out(out, out_dtype, (int64_t)m * H + h, acc);
}

// ------------------------------------------------------------------------------------------ host

// Optional CUDA events recorded around the two GEMV launches of the fused layer (benchmark hook).
cudaEvent_t g_prof_events[3] = {nullptr, nullptr, nullptr};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t plan_bytes(int64_t P, int64_t E) {
  const int64_t U = P < E ? P : E;
  return align_up(sizeof(int) * (size_t)(4 + U + (U + 1) + 2 * P), 256);
}

Plan carve_plan(void* ws, int64_t P, int64_t E) {
  const int64_t U = P < E ? P : E;
  int* base = reinterpret_cast<int*>(ws);
  Plan pl;
  pl.n_unique = base;
  pl.uniq_expert = base + 4;
  pl.uniq_start = pl.uniq_expert + U;
  pl.pairs = pl.uniq_start + (U + 1);
  pl.mapped = pl.pairs + P;
  return pl;
}

size_t gemv_smem_bytes(int K) {
  return (size_t)2 * 256 * 32 * 4 + (size_t)kWarps * kMaxTok * kSlabCols * 4 + (size_t)kMaxTok * K * 2;
}

template <bool kScale8, bool kSilu>
int launch_gemv(const GemvArgs& g, int64_t P, int64_t E, cudaStream_t st) {
  static bool attr_set[64] = {false};
  const size_t smem = gemv_smem_bytes(g.K);
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sparse_gemv_kernel<kScale8, kSilu>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  const int64_t U = P < E ? P : E;
  int64_t grid = U * g.n_slabs;
  const int64_t cap = (int64_t)sm_count();
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  sparse_gemv_kernel<kScale8, kSilu><<<(unsigned)grid, kThreads, smem, st>>>(g);
  return B200FP4_STATUS_SUCCESS;
}

bool vector_ok(int64_t N, int64_t K, int64_t G, const SparseWeights& w, const void* A, int64_t lda) {
  if (N % 16 != 0 || K % 16 != 0 || K > 8192) return false;
  if (G != K / 16 && G != K / 8) return false;
  if (!aligned(w.comp, 16) || !aligned(w.meta, 16) || !aligned(w.scale, 16) || !aligned(A, 16)) return false;
  if ((w.comp_e | w.comp_pair | w.comp_odd | w.meta_e | w.meta_row | w.scale_e | w.scale_row) % 16 != 0) return false;
  if (lda % 8 != 0) return false;
  return true;
}

int check_common(const void* A, int a_dtype, const void* out, int out_dtype, int64_t P, int64_t N, int64_t K,
                 int64_t G, int64_t E) {
  if (P < 0 || N <= 0 || K <= 0 || E <= 0 || G <= 0 || (K % 8) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if ((K / 8) % G != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (a_dtype != B200FP4_DTYPE_F16 && a_dtype != B200FP4_DTYPE_BF16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (out_dtype != B200FP4_DTYPE_F16 && out_dtype != B200FP4_DTYPE_BF16 && out_dtype != B200FP4_DTYPE_F32)
    return B200FP4_STATUS_NOT_SUPPORTED;
  if (P > 0 && (!A || !out)) return B200FP4_STATUS_INVALID_VALUE;
  if (P > 65535 || N > (int64_t)1 << 24 || K > (int64_t)1 << 20) return B200FP4_STATUS_NOT_SUPPORTED;
  return B200FP4_STATUS_SUCCESS;
}

// Runs one projection for P pairs with a plan already in `plan`.
int run_projection(const SparseWeights& w, const Plan& plan, const void* A, int a_bf16, int64_t lda, int a_div,
                   void* out, int out_dtype, int64_t ldo, int64_t P, int64_t N, int64_t K, int64_t G, int64_t E,
                   int inter_silu, cudaStream_t st) {
  GemvArgs g;
  g.w = w;
  g.plan = plan;
  g.A = A;
  g.lda = lda;
  g.a_div = a_div;
  g.a_bf16 = a_bf16;
  g.out = out;
  g.ldo = ldo;
  g.out_dtype = out_dtype;
  g.N = (int)N;
  g.K = (int)K;
  g.inter = inter_silu;
  const bool s8 = (G == K / 8);
  if (inter_silu > 0) {
    g.n_slabs = (inter_silu + 63) / 64;
    return s8 ? launch_gemv<true, true>(g, P, E, st) : launch_gemv<false, true>(g, P, E, st);
  }
  g.n_slabs = (int)((N + kSlabCols - 1) / kSlabCols);
  return s8 ? launch_gemv<true, false>(g, P, E, st) : launch_gemv<false, false>(g, P, E, st);
}

int gemv_entry(const SparseWeights& w, int mode, const void* A, int a_dtype, const int32_t* expert_ids, void* out,
               int out_dtype, int64_t P, int64_t N, int64_t K, int64_t G, int64_t E, void* workspace, size_t ws_bytes,
               void* stream) {
  int rc = check_common(A, a_dtype, out, out_dtype, P, N, K, G, E);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (P == 0) return B200FP4_STATUS_SUCCESS;
  if (!w.comp || !w.scale || !w.g || !expert_ids || (mode == 0 && !w.meta)) return B200FP4_STATUS_INVALID_VALUE;
  cudaStream_t st = (cudaStream_t)stream;
  const int a_bf16 = a_dtype == B200FP4_DTYPE_BF16;
  if (mode == 0 && E <= kPlanMaxExperts && vector_ok(N, K, G, w, A, K)) {
    if (!workspace || ws_bytes < plan_bytes(P, E) || !aligned(workspace, 16)) return B200FP4_STATUS_ALLOC_FAILED;
    Plan plan = carve_plan(workspace, P, E);
    moe_plan_kernel<<<1, kPlanThreads, 0, st>>>(expert_ids, (int)P, nullptr, 0, (int)E, plan);
    zero_unmapped_rows_kernel<<<(unsigned)P, 128, 0, st>>>(plan.mapped, (int)P, out, out_dtype, N, (int)N);
    rc = run_projection(w, plan, A, a_bf16, K, 1, out, out_dtype, N, P, N, K, G, E, 0, st);
    if (rc != B200FP4_STATUS_SUCCESS) return rc;
    return finish_launch(3);
  }
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)P);
  generic_gemv_kernel<<<grid, 128, 0, st>>>(w, mode, A, a_bf16, K, expert_ids, (int)E, out, out_dtype, (int)P, (int)N,
                                            (int)K, (int)G);
  return finish_launch(1);
}

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" size_t b200fp4_sparse_workspace_bytes(int64_t P, int64_t E) {
  if (P < 0 || E < 0) return 0;
  return plan_bytes(P, E);
}

extern "C" int b200fp4_sparse_gemv(const void* A, int a_dtype, const uint8_t* B_comp_T, const uint8_t* Meta_T_pk,
                                   const uint8_t* scales_T, const float* g_scales, const int32_t* expert_ids, void* out,
                                   int out_dtype, int64_t P, int64_t N, int64_t K, int64_t G, int64_t E, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  SparseWeights w;
  w.comp = B_comp_T;
  w.meta = Meta_T_pk;
  w.scale = scales_T;
  w.g = g_scales;
  w.comp_e = (K / 4) * N;
  w.comp_pair = 2 * N;
  w.comp_odd = N;
  w.meta_e = (K / 8) * N;
  w.meta_row = N;
  w.scale_e = G * N;
  w.scale_row = N;
  return gemv_entry(w, 0, A, a_dtype, expert_ids, out, out_dtype, P, N, K, G, E, workspace, workspace_bytes, stream);
}

extern "C" int b200fp4_dense_gemv(const void* A, int a_dtype, const uint8_t* B_dense_T, const uint8_t* scales_T,
                                  const float* g_scales, const int32_t* expert_ids, void* out, int out_dtype, int64_t P,
                                  int64_t N, int64_t K, int64_t G, int64_t E, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  if (K > 0 && G > 0 && (K % 2 != 0 || K % G != 0 || (K / G) % 2 != 0)) return B200FP4_STATUS_INVALID_VALUE;
  SparseWeights w = {};
  w.comp = B_dense_T;
  w.scale = scales_T;
  w.g = g_scales;
  w.comp_e = (K / 2) * N;
  w.scale_e = G * N;
  w.scale_row = N;
  // the dense layout has no constraint tying G to K/8; validate with a G that passes the shared check
  int rc = check_common(A, a_dtype, out, out_dtype, P, N, K, (K % 8 == 0) ? K / 8 : 1, E);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (P == 0) return B200FP4_STATUS_SUCCESS;
  if (!B_dense_T || !scales_T || !g_scales || !expert_ids) return B200FP4_STATUS_INVALID_VALUE;
  (void)workspace;
  (void)workspace_bytes;
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)P);
  generic_gemv_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(w, 1, A, a_dtype == B200FP4_DTYPE_BF16, K, expert_ids,
                                                              (int)E, out, out_dtype, (int)P, (int)N, (int)K, (int)G);
  return finish_launch(1);
}

extern "C" int b200fp4_sparse_packed_gemv(const void* A, int a_dtype, const uint8_t* B_packed_T, const float* g_scales,
                                          const int32_t* expert_ids, void* out, int out_dtype, int64_t P, int64_t N,
                                          int64_t K, int64_t E, void* workspace, size_t workspace_bytes, void* stream) {
  SparseWeights w;
  w.comp = B_packed_T;
  w.meta = B_packed_T ? B_packed_T + 2 * N : nullptr;
  w.scale = B_packed_T ? B_packed_T + 3 * N : nullptr;
  w.g = g_scales;
  w.comp_e = (K / 8) * 4 * N;
  w.comp_pair = 4 * N;
  w.comp_odd = N;
  w.meta_e = w.comp_e;
  w.meta_row = 4 * N;
  w.scale_e = w.comp_e;
  w.scale_row = 4 * N;
  return gemv_entry(w, 0, A, a_dtype, expert_ids, out, out_dtype, P, N, K, K / 8, E, workspace, workspace_bytes, stream);
}

extern "C" void b200fp4_fused_moe_profile_events(void* before_gate_up, void* after_gate_up, void* after_down) {
  g_prof_events[0] = (cudaEvent_t)before_gate_up;
  g_prof_events[1] = (cudaEvent_t)after_gate_up;
  g_prof_events[2] = (cudaEvent_t)after_down;
}

extern "C" size_t b200fp4_fused_moe_workspace_bytes(int64_t M, int64_t topk, int64_t H, int64_t I, int64_t E) {
  if (M < 0 || topk <= 0 || H <= 0 || I <= 0 || E <= 0) return 0;
  const int64_t P = M * topk;
  return plan_bytes(P, E) + align_up((size_t)P * I * sizeof(__half), 256) + align_up((size_t)P * H * sizeof(float), 256);
}

extern "C" int b200fp4_fused_sparse_moe(const void* hidden, int h_dtype, const float* topk_weights,
                                        const int32_t* topk_ids, const int32_t* expert_map, int64_t global_E,
                                        const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale,
                                        const float* w13_g, int64_t G13, const uint8_t* w2_comp, const uint8_t* w2_meta,
                                        const uint8_t* w2_scale, const float* w2_g, int64_t G2, void* out, int out_dtype,
                                        int64_t M, int64_t topk, int64_t H, int64_t I, int64_t E,
                                        int apply_router_weight_on_input, void* workspace, size_t workspace_bytes,
                                        void* stream) {
  if (M < 0 || topk <= 0 || H <= 0 || I <= 0 || E <= 0) return B200FP4_STATUS_INVALID_VALUE;
  const int64_t P = M * topk;
  int rc = check_common(hidden, h_dtype, out, out_dtype, P, 2 * I, H, G13, E);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  rc = check_common(hidden, h_dtype, out, out_dtype, P, H, I, G2, E);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!topk_weights || !topk_ids || !w13_comp || !w13_meta || !w13_scale || !w13_g || !w2_comp || !w2_meta ||
      !w2_scale || !w2_g)
    return B200FP4_STATUS_INVALID_VALUE;
  if (expert_map && global_E <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (E > kPlanMaxExperts || out_dtype == B200FP4_DTYPE_F32) return B200FP4_STATUS_NOT_SUPPORTED;
  SparseWeights w13, w2;
  w13.comp = w13_comp; w13.meta = w13_meta; w13.scale = w13_scale; w13.g = w13_g;
  w13.comp_e = (H / 4) * 2 * I; w13.comp_pair = 4 * I; w13.comp_odd = 2 * I;
  w13.meta_e = (H / 8) * 2 * I; w13.meta_row = 2 * I; w13.scale_e = G13 * 2 * I; w13.scale_row = 2 * I;
  w2.comp = w2_comp; w2.meta = w2_meta; w2.scale = w2_scale; w2.g = w2_g;
  w2.comp_e = (I / 4) * H; w2.comp_pair = 2 * H; w2.comp_odd = H;
  w2.meta_e = (I / 8) * H; w2.meta_row = H; w2.scale_e = G2 * H; w2.scale_row = H;
  // the fused layer only exists in vectorised form
  if (I % 16 != 0 || !vector_ok(2 * I, H, G13, w13, hidden, H) || !vector_ok(H, I, G2, w2, hidden, I))
    return B200FP4_STATUS_NOT_SUPPORTED;
  if (!workspace || !aligned(workspace, 256) || workspace_bytes < b200fp4_fused_moe_workspace_bytes(M, topk, H, I, E))
    return B200FP4_STATUS_ALLOC_FAILED;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  Plan plan = carve_plan(ws, P, E);
  __half* act = reinterpret_cast<__half*>(ws + plan_bytes(P, E));
  float* down = reinterpret_cast<float*>(ws + plan_bytes(P, E) + align_up((size_t)P * I * sizeof(__half), 256));

  moe_plan_kernel<<<1, kPlanThreads, 0, st>>>(topk_ids, (int)P, expert_map, (int)global_E, (int)E, plan);
  if (g_prof_events[0]) cudaEventRecord(g_prof_events[0], st);
  rc = run_projection(w13, plan, hidden, h_dtype == B200FP4_DTYPE_BF16, H, (int)topk, act, B200FP4_DTYPE_F16, I, P,
                      2 * I, H, G13, E, (int)I, st);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (g_prof_events[1]) cudaEventRecord(g_prof_events[1], st);
  rc = run_projection(w2, plan, act, 0, I, 1, down, B200FP4_DTYPE_F32, H, P, H, I, G2, E, 0, st);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (g_prof_events[2]) cudaEventRecord(g_prof_events[2], st);
  dim3 grid((unsigned)((H + 255) / 256), (unsigned)M);
  weighted_reduce_kernel<<<grid, 256, 0, st>>>(down, topk_weights, plan.mapped, out, out_dtype, (int)M, (int)topk,
                                               (int)H, apply_router_weight_on_input ? 1 : 0);
  return finish_launch(4);
}
