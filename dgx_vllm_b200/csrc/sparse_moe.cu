// 2:4-sparse NVFP4 batched GEMV and the fused MoE decode layer for sm_100a.
//
// Replaces sparse_fp4_kernel/sparse_fp4_v7.cu of the reference with a different execution plan:
//   * a "plan" kernel groups the (token, expert) pairs by expert and cuts them into passes of at
//     most four (or eight) tokens, so an expert's weights are streamed from HBM once per layer (per
//     pass) instead of once per pair;
//   * two persistent GEMV kernels (one block per SM) walk (pass, column slab) work items: the
//     tensor-core kernel further down (mma.sp; needs ordered metadata indices and one scale per 16 k)
//     and the general kernel described here, which takes any metadata.  In the general kernel a thread
//     owns 16 output columns and one K-slice.  Its weight bytes (four compressed rows, two
//     metadata rows, one scale row per 16 k) arrive through a private multi-stage cp.async ring in
//     shared memory that keeps running across work-item boundaries, so HBM latency is hidden
//     without holding prefetched data in registers;
//   * E2M1 byte -> half2 and metadata byte -> byte-permute selector decoding are table look-ups in
//     shared memory (32 copies per entry, one per bank: conflict free); the table index is built by
//     a single PRMT that merges the byte with the lane's bank offset;
//   * the 2:4 gather of the activation is one PRMT, products are packed half2 FMAs, and every
//     16-element scale block is folded into an fp32 accumulator;
//   * the K reduction is done in-kernel (warp shuffles, then one shared-memory pass), so there is
//     no partial-sum tensor and no separate reduction kernel; SiLU(gate)*up is fused into the
//     gate_up epilogue; the router-weighted sum is a small deterministic kernel (no atomics).
#include <type_traits>

#include <mutex>

#include "common.cuh"

extern "C" size_t b200fp4_sparse_workspace_bytes(int64_t P, int64_t K, int64_t E);

namespace b200fp4 {
namespace {

constexpr int kThreads = 256;      // block size of the 16-columns-per-thread variant
constexpr int kMaxTok = 4;       // tokens of one expert processed per pass over its weights
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxExperts = 4096;
constexpr int kLutBytes = 256 * 256;   // 256 rows of [32 x comp entry | 32 x meta entry]

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
  int* hdr;        // [0] = number of unique experts, [1] = number of passes, [2] and [4] = work-item counters of the
                   // warp-scheduled GEMV (one per projection), [3] = status word of the one-launch layer
  int* pairs;      // [P]  pair indices grouped by expert
  int* mapped;     // [P]  local expert id of each pair, or -1
  int4* pass_rec;  // [passes][2]: {expert, n_tokens, pair0, pair1}, {pair2, pair3, index of pair0 in pairs[], -}
};

struct GemvArgs {
  SparseWeights w;
  Plan plan;
  const __half* A;  // [rows, K] fp16; the row of pair p is p / a_div
  int64_t lda;
  int a_div;
  uint32_t a_magic; // 0 if a_div == 1, else floor(2^32 / a_div) + 1: pair / a_div == umulhi(pair, a_magic) for pair < 2^16
  void* out;        // [P, N] (or [P, N/2] in SiLU mode), leading dimension ldo
  int64_t ldo;
  int out_dtype;
  int N, K;
  int n_slabs;
  int inter;        // SiLU mode: gate columns [0, inter), up columns [inter, 2*inter)
  long long wait_cycles;   // one-launch layer: clock64 budget of a wait on a pass counter
};

// ------------------------------------------------------------------------------------------ plan

// Activation copy modes of the plan kernel's extra blocks.
//   kConvBf16      bf16 -> fp16, same element order
//   kConvBf16Frag  bf16 -> fp16 in "fragment order" (below)
//   kConvF16Frag   fp16 copy in fragment order
// Fragment order: inside every group of 32 elements (16 words of two halves) word 4i + t is stored at position
// 4t + i (a 4 x 4 transpose of words).  The 16 bytes at offset 16t of a group are then exactly the four B-operand
// registers of lane t of a quad for one 32-wide k-step of mma.m16n8k32, which the warp-scheduled GEMV fetches with a
// single 16-byte asynchronous copy per lane.
enum { kConvNone = 0, kConvBf16 = 1, kConvBf16Frag = 2, kConvF16Frag = 3 };

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w) {
  const __half2 h = __float22half2_rn(__bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w)));
  return *reinterpret_cast<const uint32_t*>(&h);
}


// Block 0 builds the plan; the remaining blocks (if any) copy / convert the activation matrix to fp16.
__global__ void __launch_bounds__(kPlanThreads)
    moe_plan_kernel(const int32_t* __restrict__ ids, int P, const int32_t* __restrict__ expert_map, int global_E, int E,
                    Plan plan, const void* __restrict__ conv_src_v, __half* __restrict__ conv_dst,
                    int64_t conv_chunks, int ids_topk, int64_t ids_ld, int64_t conv_row_chunks, int64_t conv_ld_chunks,
                    int* zero_buf, int zero_count, int max_tok, int conv_mode) {
  pdl_wait();                 // the kernel before this one may still be reading the workspace this one rewrites
  pdl_launch_dependents();
  if (blockIdx.x > 0) {
    const uint4* conv_src = reinterpret_cast<const uint4*>(conv_src_v);
    const int64_t stride = (int64_t)(gridDim.x - 1) * kPlanThreads;
    if (conv_mode == kConvBf16) {
      for (int64_t i = (int64_t)(blockIdx.x - 1) * kPlanThreads + threadIdx.x; i < conv_chunks; i += stride) {
        // rows of the source may be strided (conv_ld_chunks 16-byte chunks apart); the copy is dense
        const int64_t row = i / conv_row_chunks, col = i - row * conv_row_chunks;
        const uint4 raw = conv_src[row * conv_ld_chunks + col];
        reinterpret_cast<uint4*>(conv_dst)[i] =
            make_uint4(bf16x2_to_f16x2(raw.x), bf16x2_to_f16x2(raw.y), bf16x2_to_f16x2(raw.z), bf16x2_to_f16x2(raw.w));
      }
    } else {
      // one thread per group of 32 elements: four 16-byte loads, a 4 x 4 word transpose, four 16-byte stores
      const int64_t groups = conv_chunks >> 2, row_groups = conv_row_chunks >> 2;
      for (int64_t i = (int64_t)(blockIdx.x - 1) * kPlanThreads + threadIdx.x; i < groups; i += stride) {
        const int64_t row = i / row_groups, col = i - row * row_groups;
        uint4 r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          r[k] = conv_src[row * conv_ld_chunks + col * 4 + k];
          if (conv_mode == kConvBf16Frag)
            r[k] = make_uint4(bf16x2_to_f16x2(r[k].x), bf16x2_to_f16x2(r[k].y), bf16x2_to_f16x2(r[k].z), bf16x2_to_f16x2(r[k].w));
        }
        uint4* dst = reinterpret_cast<uint4*>(conv_dst) + i * 4;
        dst[0] = make_uint4(r[0].x, r[1].x, r[2].x, r[3].x);
        dst[1] = make_uint4(r[0].y, r[1].y, r[2].y, r[3].y);
        dst[2] = make_uint4(r[0].z, r[1].z, r[2].z, r[3].z);
        dst[3] = make_uint4(r[0].w, r[1].w, r[2].w, r[3].w);
      }
    }
    return;
  }
  __shared__ int s_count[kPlanMaxExperts];
  __shared__ int s_warp[3][32];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += kPlanThreads) s_count[e] = 0;
  for (int i = tid; i < zero_count; i += kPlanThreads) zero_buf[i] = 0;   // per-pass counters of the one-launch layer
  if (tid == 0) plan.hdr[2] = plan.hdr[3] = plan.hdr[4] = 0;
  __syncthreads();
  for (int p = tid; p < P; p += kPlanThreads) {
    int e = ids[(int64_t)(p / ids_topk) * ids_ld + (p % ids_topk)];   // ids rows may be strided
    if (expert_map != nullptr) e = (e >= 0 && e < global_E) ? expert_map[e] : -1;
    if (e < 0 || e >= E) e = -1;
    plan.mapped[p] = e;
    if (e >= 0) atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  // exclusive scans over experts of (pairs, present, passes); each thread owns a contiguous run
  const int per = (E + kPlanThreads - 1) / kPlanThreads;
  const int e0 = tid * per;
  int sum[3] = {0, 0, 0};
  for (int i = 0; i < per; ++i) {
    const int e = e0 + i;
    if (e < E) {
      const int c = s_count[e];
      sum[0] += c;
      sum[1] += c > 0;
      sum[2] += (c + max_tok - 1) / max_tok;
    }
  }
  int inc[3] = {sum[0], sum[1], sum[2]};
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1)
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const int v = __shfl_up_sync(0xffffffffu, inc[k], d);
      if (lane >= d) inc[k] += v;
    }
  if (lane == 31)
#pragma unroll
    for (int k = 0; k < 3; ++k) s_warp[k][warp] = inc[k];
  __syncthreads();
  if (warp == 0) {
    int v[3] = {s_warp[0][lane], s_warp[1][lane], s_warp[2][lane]};
#pragma unroll
    for (int d = 1; d < 32; d <<= 1)
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        const int x = __shfl_up_sync(0xffffffffu, v[k], d);
        if (lane >= d) v[k] += x;
      }
#pragma unroll
    for (int k = 0; k < 3; ++k) s_warp[k][lane] = v[k];
  }
  __syncthreads();
  int base[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) base[k] = inc[k] - sum[k] + (warp > 0 ? s_warp[k][warp - 1] : 0);
  const int my_pair_base = base[0], my_pass_base = base[2];
  {
    int bc = base[0];
    for (int i = 0; i < per; ++i) {
      const int e = e0 + i;
      if (e < E) {
        const int c = s_count[e];
        s_count[e] = bc;  // becomes the scatter cursor
        bc += c;
      }
    }
  }
  if (tid == kPlanThreads - 1) {
    plan.hdr[0] = base[1] + sum[1];
    plan.hdr[1] = base[2] + sum[2];
  }
  __syncthreads();
  for (int p = tid; p < P; p += kPlanThreads) {
    const int e = plan.mapped[p];
    if (e >= 0) plan.pairs[atomicAdd(&s_count[e], 1)] = p;
  }
  __syncthreads();  // pairs[] (global) written by this block are visible to it after the barrier
  // pass records of the experts this thread owns; after the scatter s_count[e] is the END of e's run
  {
    int start = my_pair_base, pass = my_pass_base;
    for (int i = 0; i < per; ++i) {
      const int e = e0 + i;
      if (e < E) {
        const int end = s_count[e];
        for (int s0 = start; s0 < end; s0 += max_tok) {
          const int nt = min(max_tok, end - s0);
          int pr[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) pr[t] = t < nt ? plan.pairs[s0 + t] : 0;
          // pairs 4.. of an 8-token pass are read from pairs[] (the run of an expert is contiguous there)
          plan.pass_rec[2 * pass] = make_int4(e, nt, pr[0], pr[1]);
          plan.pass_rec[2 * pass + 1] = make_int4(pr[2], pr[3], s0, 0);
          ++pass;
        }
        start = end;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ tables

__device__ __forceinline__ uint32_t e2m1_to_half_bits(uint32_t nib) {
  const uint32_t c = nib & 7u;
  uint32_t h = (c == 0) ? 0u : (c == 1 ? 0x3800u : 0x3800u + c * 0x200u);
  if (c != 0) h |= (nib & 8u) << 12;
  return h;
}

// Row b (256 bytes) of the table: words 0..31 hold 32 copies of the half2 pair decoded from the
// compressed byte b, words 32..63 hold 32 copies of the two PRMT selectors decoded from the
// metadata byte b.  A lane always reads word `lane` (or 32+lane), i.e. its own bank.
__device__ __forceinline__ void fill_tables(uint32_t* lut, int tid, int nthreads) {
  for (int b = tid; b < 256; b += nthreads) {
    const uint32_t vc = e2m1_to_half_bits(b & 15) | (e2m1_to_half_bits(b >> 4) << 16);
    const uint32_t i0 = b & 3, i1 = (b >> 2) & 3, i2 = (b >> 4) & 3, i3 = (b >> 6) & 3;
    const uint32_t s0 = (2 * i0) | ((2 * i0 + 1) << 4) | ((2 * i1) << 8) | ((2 * i1 + 1) << 12);
    const uint32_t s1 = (2 * i2) | ((2 * i2 + 1) << 4) | ((2 * i3) << 8) | ((2 * i3 + 1) << 12);
    const uint32_t vm = s0 | (s1 << 16);
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
      const int l = (i + tid) & 31;  // rotate so that the 32 threads of a warp hit 32 banks
      lut[b * 64 + l] = vc;
      lut[b * 64 + 32 + l] = vm;
    }
  }
}

// ------------------------------------------------------------------------------------------ GEMV

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
}
// COLS bytes (16 or 8) of one weight row
template <int COLS>
__device__ __forceinline__ void cp_async_cols(void* smem_dst, const void* gmem_src) {
  if (COLS == 16) cp_async16(smem_dst, gmem_src);
  else cp_async8(smem_dst, gmem_src);
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int q) {
  return q == 0 ? v.x : (q == 1 ? v.y : (q == 2 ? v.z : v.w));
}
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t lds32(const unsigned char* p) { return *reinterpret_cast<const uint32_t*>(p); }

// One scale block (16 k) x 16 columns for T tokens.  v[] = 4 compressed rows, 2 metadata rows,
// 1 (or 2) scale rows; a[t] = the 16 activations of token t as 8 half2.
template <int T, int COLS, bool kScale8>
__device__ __forceinline__ void compute_block(const uint4 (&v)[8], const uint4 (&a)[T][2], const unsigned char* lut,
                                              uint32_t lane4, float (&acc)[T][COLS]) {
  // PRMT selectors: (table row = byte j of the word) << 8 | lane*4
  constexpr uint32_t kIdx[4] = {0x5504u, 0x5514u, 0x5524u, 0x5534u};
  // PRMT selectors: bytes (j, j+1) of the scale word to the high bytes of two halves
  constexpr uint32_t kSc[2] = {0x1404u, 0x3424u};
#pragma unroll
  for (int q = 0; q < COLS / 4; ++q) {
    const uint32_t c0 = word_of(v[0], q), c1 = word_of(v[1], q), c2 = word_of(v[2], q), c3 = word_of(v[3], q);
    const uint32_t m0 = word_of(v[4], q), m1 = word_of(v[5], q);
    const uint32_t s0 = word_of(v[6], q) & 0x7F7F7F7Fu;
    const uint32_t s1 = kScale8 ? (word_of(v[7], q) & 0x7F7F7F7Fu) : 0u;
#pragma unroll
    for (int jp = 0; jp < 2; ++jp) {
      // e4m3 bits moved into a half give scale * 2^-8; the 2^8 is folded into the final multiplier
      const float2 sc0 = __half22float2(as_h2(prmt(s0, 0u, kSc[jp]) >> 1));
      float2 sc1 = make_float2(0.f, 0.f);
      if (kScale8) sc1 = __half22float2(as_h2(prmt(s1, 0u, kSc[jp]) >> 1));
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = jp * 2 + jj;
        const int col = q * 4 + j;
        const __half2 w0 = as_h2(lds32(lut + prmt(c0, lane4, kIdx[j])));
        const __half2 w1 = as_h2(lds32(lut + prmt(c1, lane4, kIdx[j])));
        const __half2 w2 = as_h2(lds32(lut + prmt(c2, lane4, kIdx[j])));
        const __half2 w3 = as_h2(lds32(lut + prmt(c3, lane4, kIdx[j])));
        const uint32_t sel01 = lds32(lut + 128 + prmt(m0, lane4, kIdx[j]));
        const uint32_t sel23 = lds32(lut + 128 + prmt(m1, lane4, kIdx[j]));
        const uint32_t sel1 = sel01 >> 16, sel3 = sel23 >> 16;
        const float f0 = jj == 0 ? sc0.x : sc0.y;
        const float f1 = jj == 0 ? sc1.x : sc1.y;
#pragma unroll
        for (int t = 0; t < T; ++t) {
          __half2 p = __hmul2(w0, as_h2(prmt(a[t][0].x, a[t][0].y, sel01)));
          p = __hfma2(w1, as_h2(prmt(a[t][0].z, a[t][0].w, sel1)), p);
          if (kScale8) {
            __half2 r = __hmul2(w2, as_h2(prmt(a[t][1].x, a[t][1].y, sel23)));
            r = __hfma2(w3, as_h2(prmt(a[t][1].z, a[t][1].w, sel3)), r);
            acc[t][col] = fmaf(__half2float(__hadd(__low2half(p), __high2half(p))), f0, acc[t][col]);
            acc[t][col] = fmaf(__half2float(__hadd(__low2half(r), __high2half(r))), f1, acc[t][col]);
          } else {
            p = __hfma2(w2, as_h2(prmt(a[t][1].x, a[t][1].y, sel23)), p);
            p = __hfma2(w3, as_h2(prmt(a[t][1].z, a[t][1].w, sel3)), p);
            acc[t][col] = fmaf(__half2float(__hadd(__low2half(p), __high2half(p))), f0, acc[t][col]);
          }
        }
      }
    }
  }
}

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
  if (dtype == B200FP4_DTYPE_F16) reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
  else if (dtype == B200FP4_DTYPE_BF16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[idx] = v;
}

struct Rec {
  int e, nt;
  int p0, p1, p2, p3;
  __device__ __forceinline__ int pair(int t) const { return t == 0 ? p0 : (t == 1 ? p1 : (t == 2 ? p2 : p3)); }
};
__device__ __forceinline__ Rec load_rec(const int4* recs, int pass) {
  const int4 x = recs[2 * pass], y = recs[2 * pass + 1];
  Rec r;
  r.e = x.x; r.nt = x.y; r.p0 = x.z; r.p1 = x.w; r.p2 = y.x; r.p3 = y.y;
  return r;
}
__device__ __forceinline__ Rec empty_rec() {
  Rec r;
  r.e = -1; r.nt = 0; r.p0 = r.p1 = r.p2 = r.p3 = 0;
  return r;
}

// NT      threads per block: 256 with COLS = 16 columns per thread, or 512 with COLS = 8 (twice the
//         warps per SM for latency hiding, half the accumulators per thread)
// CG      column groups per slab: slab = COLS*CG columns, NT/CG K-slices
// S       cp.async ring stages; every thread must own at least S-1 scale blocks per item
// kScale8 one scale per 8 k instead of per 16 k
// kSilu   slab = CG*8 gate columns + the matching CG*8 up columns; epilogue writes SiLU(gate)*up
template <int NT, int COLS, int CG, int S, bool kScale8, bool kSilu>
__global__ void __launch_bounds__(NT, 1) sparse_gemv_kernel(const GemvArgs g) {
  constexpr int kThreads = NT;
  constexpr int kWarps = NT / 32;
  constexpr int KS = kThreads / CG;
  constexpr int SLAB = CG * COLS;
  constexpr int NV = kScale8 ? 8 : 7;
  using Vec = typename std::conditional<COLS == 16, uint4, uint2>::type;   // COLS bytes of one weight row
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* lut_w = reinterpret_cast<uint32_t*>(smem);
  Vec* ring = reinterpret_cast<Vec*>(smem + kLutBytes);                          // [S][NV][NT]
  float* red = reinterpret_cast<float*>(ring + S * NV * kThreads);               // [kWarps][kMaxTok][SLAB]
  __half* sA = reinterpret_cast<__half*>(red + kWarps * kMaxTok * SLAB);         // [2][kMaxTok][K]

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int cg = lane % CG, ksub = lane / CG;
  const int kslice = warp * (32 / CG) + ksub;
  const uint32_t lane4 = (uint32_t)lane * 4u;
  const int K = g.K, KB = K >> 4;
  const int nblk = (KB - kslice + KS - 1) / KS;   // scale blocks this thread owns in every item (>= S-1)
  const int grid = gridDim.x;
  fill_tables(lut_w, tid, kThreads);

  const int n_items = g.plan.hdr[1] * g.n_slabs;
  int item = blockIdx.x;
  if (item >= n_items) return;
  Rec rc = load_rec(g.plan.pass_rec, item / g.n_slabs);
  Rec rn = (item + grid < n_items) ? load_rec(g.plan.pass_rec, (item + grid) / g.n_slabs) : empty_rec();

  // this thread's share of the activation rows of a pass -> sA[buf]
  const int chunks = K >> 3;
  auto issue_A = [&](const Rec& r, int buf) {
    for (int i = tid; i < r.nt * chunks; i += kThreads) {
      const int t = i / chunks, ch = i - t * chunks;
      const int64_t row = r.pair(t) / g.a_div;
      cp_async16(sA + ((size_t)(buf * kMaxTok + t) * K + ch * 8), g.A + row * g.lda + ch * 8);
    }
  };

  // ---- weight fetch stream: runs S-1 blocks ahead of the compute and crosses item boundaries
  int f_item = item, f_j = 0, f_slot = 0;
  const uint8_t *f_comp = nullptr, *f_meta = nullptr, *f_scale = nullptr;
  bool f_ok = false;
  auto fetch_next = [&](const Rec& cur, const Rec& nxt) {
    if (f_item < n_items) {
      if (f_j == 0) {
        const int e = (f_item == item) ? cur.e : nxt.e;
        const int slab = f_item % g.n_slabs;
        int col0;
        if (kSilu) col0 = (cg < CG / 2) ? slab * (SLAB / 2) + cg * COLS : g.inter + slab * (SLAB / 2) + (cg - CG / 2) * COLS;
        else col0 = slab * SLAB + cg * COLS;
        f_ok = kSilu ? ((cg < CG / 2 ? col0 : col0 - g.inter) < g.inter) : (col0 < g.N);
        f_comp = g.w.comp + (int64_t)e * g.w.comp_e + col0;
        f_meta = g.w.meta + (int64_t)e * g.w.meta_e + col0;
        f_scale = g.w.scale + (int64_t)e * g.w.scale_e + col0;
      }
      if (f_ok) {
        const int kb = kslice + KS * f_j;
        Vec* dst = ring + (size_t)f_slot * NV * kThreads + tid;
        const uint8_t* c0 = f_comp + (int64_t)(2 * kb) * g.w.comp_pair;
        cp_async_cols<COLS>(dst, c0);
        cp_async_cols<COLS>(dst + kThreads, c0 + g.w.comp_odd);
        cp_async_cols<COLS>(dst + 2 * kThreads, c0 + g.w.comp_pair);
        cp_async_cols<COLS>(dst + 3 * kThreads, c0 + g.w.comp_pair + g.w.comp_odd);
        const uint8_t* m0 = f_meta + (int64_t)(2 * kb) * g.w.meta_row;
        cp_async_cols<COLS>(dst + 4 * kThreads, m0);
        cp_async_cols<COLS>(dst + 5 * kThreads, m0 + g.w.meta_row);
        if (kScale8) {
          const uint8_t* s0 = f_scale + (int64_t)(2 * kb) * g.w.scale_row;
          cp_async_cols<COLS>(dst + 6 * kThreads, s0);
          cp_async_cols<COLS>(dst + 7 * kThreads, s0 + g.w.scale_row);
        } else {
          cp_async_cols<COLS>(dst + 6 * kThreads, f_scale + (int64_t)kb * g.w.scale_row);
        }
      }
      if (++f_j == nblk) {
        f_j = 0;
        f_item += grid;
      }
    }
    cp_async_commit();
    f_slot = (f_slot + 1 == S) ? 0 : f_slot + 1;
  };

  // prologue: activations of the first item, then S-1 weight blocks
  issue_A(rc, 0);
  cp_async_commit();
#pragma unroll
  for (int s = 0; s < S - 1; ++s) fetch_next(rc, rn);

  int c_slot = 0, abuf = 0;
  for (; item < n_items; item += grid) {
    const int slab = item % g.n_slabs;
    // record of the item after next; activations of the next item ride on the next weight group
    Rec rnn = (item + 2 * grid < n_items) ? load_rec(g.plan.pass_rec, (item + 2 * grid) / g.n_slabs) : empty_rec();
    const float gmul = g.w.g[rc.e] * 256.0f;
    cp_async_wait<S - 2>();   // oldest group: first weight block of this item and (older) its activations
    __syncthreads();          // sA[abuf] complete for all threads; red and sA[abuf^1] free
    issue_A(rn, abuf ^ 1);

    float accs[kMaxTok][COLS];
    auto run = [&](auto tconst) {
      constexpr int T = decltype(tconst)::value;
      float acc[T][COLS];
#pragma unroll
      for (int t = 0; t < T; ++t)
#pragma unroll
        for (int c = 0; c < COLS; ++c) acc[t][c] = 0.f;
      for (int j = 0; j < nblk; ++j) {
        cp_async_wait<S - 2>();
        uint4 v[8];
        const Vec* src = ring + (size_t)c_slot * NV * kThreads + tid;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const Vec x = src[i * kThreads];
          v[i].x = x.x;
          v[i].y = x.y;
          if (COLS == 16) {
            v[i].z = reinterpret_cast<const uint32_t*>(&x)[COLS == 16 ? 2 : 0];
            v[i].w = reinterpret_cast<const uint32_t*>(&x)[COLS == 16 ? 3 : 0];
          } else {
            v[i].z = v[i].w = 0u;
          }
        }
        if (!kScale8) v[7] = make_uint4(0, 0, 0, 0);
        fetch_next(rc, rn);
        const int kb = kslice + KS * j;
        uint4 a[T][2];
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const uint4* pa = reinterpret_cast<const uint4*>(sA + ((size_t)(abuf * kMaxTok + t) * K + (size_t)kb * 16));
          a[t][0] = pa[0];
          a[t][1] = pa[1];
        }
        compute_block<T, COLS, kScale8>(v, a, smem, lane4, acc);
        c_slot = (c_slot + 1 == S) ? 0 : c_slot + 1;
      }
      // K reduction: the K-slices of a warp through shuffles, then the warps through shared memory
#pragma unroll
      for (int t = 0; t < T; ++t)
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          float x = acc[t][c];
#pragma unroll
          for (int d = CG; d < 32; d <<= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
          accs[t][c] = x;
        }
      if (ksub == 0) {
#pragma unroll
        for (int t = 0; t < T; ++t) {
          float4* dst = reinterpret_cast<float4*>(red + ((size_t)warp * kMaxTok + t) * SLAB + cg * COLS);
#pragma unroll
          for (int c = 0; c < COLS / 4; ++c)
            dst[c] = make_float4(accs[t][4 * c], accs[t][4 * c + 1], accs[t][4 * c + 2], accs[t][4 * c + 3]);
        }
      }
    };
    if (rc.nt == 1) run(std::integral_constant<int, 1>{});
    else if (rc.nt == 2) run(std::integral_constant<int, 2>{});
    else if (rc.nt == 3) run(std::integral_constant<int, 3>{});
    else run(std::integral_constant<int, 4>{});
    __syncthreads();
    // epilogue: sum the warps, apply the expert's global scale, write
    if (kSilu) {
      constexpr int HALF = SLAB / 2;
      for (int i = tid; i < rc.nt * HALF; i += kThreads) {
        const int t = i / HALF, j = i - t * HALF;
        const int n = slab * HALF + j;
        if (n < g.inter) {
          float gate = 0.f, up = 0.f;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            gate += red[((size_t)w * kMaxTok + t) * SLAB + j];
            up += red[((size_t)w * kMaxTok + t) * SLAB + HALF + j];
          }
          gate *= gmul;
          up *= gmul;
          const float act = gate / (1.0f + __expf(-gate)) * up;
          store_out(g.out, g.out_dtype, (int64_t)rc.pair(t) * g.ldo + n, act);
        }
      }
    } else {
      for (int i = tid; i < rc.nt * SLAB; i += kThreads) {
        const int t = i / SLAB, j = i - t * SLAB;
        const int n = slab * SLAB + j;
        if (n < g.N) {
          float x = 0.f;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) x += red[((size_t)w * kMaxTok + t) * SLAB + j];
          store_out(g.out, g.out_dtype, (int64_t)rc.pair(t) * g.ldo + n, x * gmul);
        }
      }
    }
    rc = rn;
    rn = rnn;
    abuf ^= 1;
  }
  cp_async_wait<0>();
}

// Rows of pairs whose expert is not local are never touched by the GEMV; this writes zeros there.
__global__ void zero_unmapped_rows_kernel(const int* __restrict__ mapped, int P, void* out, int out_dtype, int64_t ldo,
                                          int N) {
  const int p = blockIdx.x;
  if (p >= P || mapped[p] >= 0) return;
  for (int n = threadIdx.x; n < N; n += blockDim.x) store_out(out, out_dtype, (int64_t)p * ldo + n, 0.f);
}

// Pass record of the tensor-core kernel: up to TM (4 or 8) pairs.
template <int TM>
struct RecT {
  int e, nt;
  int p[TM];
  __device__ __forceinline__ int pair(int t) const {
    int v = p[0];
#pragma unroll
    for (int i = 1; i < TM; ++i) v = (t == i) ? p[i] : v;
    return v;
  }
};
template <int TM>
__device__ __forceinline__ RecT<TM> load_rec_t(const Plan& plan, int pass) {
  const int4 x = plan.pass_rec[2 * pass], y = plan.pass_rec[2 * pass + 1];
  RecT<TM> r;
  r.e = x.x; r.nt = x.y; r.p[0] = x.z; r.p[1] = x.w; r.p[2] = y.x; r.p[3] = y.y;
  if (TM == 8) {
#pragma unroll
    for (int i = 4; i < TM; ++i) r.p[i] = (i < r.nt) ? plan.pairs[y.z + i] : 0;
  }
  return r;
}
template <int TM>
__device__ __forceinline__ RecT<TM> empty_rec_t() {
  RecT<TM> r;
  r.e = -1; r.nt = 0;
#pragma unroll
  for (int i = 0; i < TM; ++i) r.p[i] = 0;
  return r;
}

// ------------------------------------------------------------------------------------------ tensor-core GEMV
//
// Same work items as sparse_gemv_kernel, but the 2:4 gather and the multiply-accumulate run on the
// tensor cores: the weights are the sparse A operand of mma.sp m16n8k32 (f16, fp32 accumulate), the
// reference's metadata bytes are -- after one byte permute -- the instruction's metadata operand, and
// the (up to four, or eight) tokens of the pass are columns of B.  What is left for the CUDA cores is the
// E2M1 -> half2 decode (cvt.rn.f16x2.e2m1x2 straight from a byte of the loaded word), the E4M3 ->
// half2 decode of the block scales (cvt.rn.f16x2.e4m3x2) and one half2 multiply per pair of weights
// (E2M1 x E4M3 is exact in fp16).
//
// Requires every 4-group's two indices in increasing order (the instruction's rule), which is how
// the reference's converter writes them (sparse_v7_moe_patch.py:59-60); callers promise it.
//
// A block is 16 warps.  An item is (pass, slab of 128*CG columns); warp w owns column group w % CG
// and K-slice w / CG and walks its K-slice in steps of 32 k.  One step of one warp reads 8 compressed
// rows, 4 metadata rows and 2 scale rows of 128 columns (1792 bytes) from a private cp.async ring
// that keeps running across items, and issues 8 mma.sp (16 columns x 32 k each):
//   * quad q = lane / 4 owns columns 16q..16q+15 of the warp's 128; mma j takes columns 2h, 2h+1 of
//     every quad (h = 4*(j%2) + j/2) as its rows q and q+8;
//   * lane t = lane % 4 of the quad reads compressed rows t and t+4 (the instruction's 4-groups t and
//     t+4), so byte 2h (2h+1) of those two 16-byte vectors decodes to the fragment registers of row q
//     (q+8) -- no shuffles;
//   * metadata: for mma j the lanes with t/2 == j%2 supply it; their register is [row q | row q+8] x
//     [metadata rows 2(t%2), 2(t%2)+1], i.e. bytes (2h, 2h+1) of two 8-byte loads interleaved by PRMT.
constexpr int kMmaThreads = 512;
constexpr int kMmaWarps = 16;
constexpr int kMmaStageBytes = 1792;
constexpr int kMmaRedBytes = kMmaWarps * 128 * 4 * 4;   // K-slice partial sums [warp][column][token] fp32

__device__ __forceinline__ uint32_t shared_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t lds32_at(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint2 lds64_at(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint4 lds128_at(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ float4 lds128f_at(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void sts64f_at(uint32_t a, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(a), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ void cp_async16_s(uint32_t smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

template <int SEL>
__device__ __forceinline__ void mma_sp_m16n8k32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                const uint32_t (&b)[4], uint32_t e) {
  asm volatile(
      "mma.sp::ordered_metadata.sync.aligned.m16n8k32.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9,%10,%11}, {%0,%1,%2,%3}, %12, %13;"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(e), "n"(SEL));
}

// byte B of a word holds two E2M1 values -> half2 (low nibble in the low half)
template <int B>
__device__ __forceinline__ __half2 e2m1x2_to_h2(uint32_t w) {
  uint32_t r;
  if (B == 0) asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b0; }" : "=r"(r) : "r"(w));
  else if (B == 1) asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b1; }" : "=r"(r) : "r"(w));
  else if (B == 2) asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b2; }" : "=r"(r) : "r"(w));
  else asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %1; cvt.rn.f16x2.e2m1x2 %0, b3; }" : "=r"(r) : "r"(w));
  return as_h2(r);
}
// half H (16 bits) of a word holds two E4M3 values -> half2
template <int H>
__device__ __forceinline__ __half2 e4m3x2_to_h2(uint32_t w) {
  uint32_t r;
  if (H == 0) asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(r) : "r"(w));
  else asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, hi; }" : "=r"(r) : "r"(w));
  return as_h2(r);
}

// One projection over all items of this block.  kDep links the two projections of the MoE layer when
// they run in one launch: 1 = producer (done[pass] is incremented once an item's output is stored and
// fenced), 2 = consumer (the activations of a pass are staged only after done[pass] has reached
// `need` = producer slabs per pass), 0 = stand-alone.
// TM = tokens per pass (4 or 8; the instruction's B operand has 8 columns either way, but the
// activation buffers and the partial-sum scratch double with 8).
template <int CG, int S, bool kSilu, int kDep, int TM>
__device__ __forceinline__ void gemv_mma_phase(const GemvArgs& g, unsigned char* smem, int* done, int need) {
  using Rec = RecT<TM>;
  constexpr int KSL = kMmaWarps / CG;          // K-slices per item
  constexpr int VCOLS = 128 * CG;              // columns of a slab (SiLU: 64*CG gate + 64*CG up)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q = lane >> 2, t = lane & 3;
  const int cgw = warp % CG, ks = warp / CG;
  const int K = g.K;
  const int nstep = K / (32 * KSL);
  const int grid = gridDim.x;

  // ---- shared memory map (shared-window addresses)
  //   activations of the current and the next pass [2][TM][K + 8] fp16 | partial sums (one block of
  //   kMmaRedBytes per four tokens) | 16 rings of S stages
  const uint32_t a_pitch = 2u * (uint32_t)K + 16u;
  const uint32_t sa = (shared_addr(smem) + 1023u) & ~1023u;
  const uint32_t red = sa + ((2u * TM * a_pitch + 1023u) & ~1023u);
  const uint32_t ring_bytes = S * kMmaStageBytes;
  const uint32_t ring = red + (TM / 4) * kMmaRedBytes + (uint32_t)warp * ring_bytes;
  const uint32_t ring_end = ring + ring_bytes;

  // ---- items of this block: blockIdx.x, + grid, ...
  const int n_slabs = g.n_slabs;
  const int n_items = g.plan.hdr[1] * n_slabs;
  const int my_items = (int)blockIdx.x < n_items ? (n_items - 1 - (int)blockIdx.x) / grid + 1 : 0;
  if (my_items == 0) return;
  auto pass_of = [&](int i) { return ((int)blockIdx.x + i * grid) / n_slabs; };
  Rec rc = load_rec_t<TM>(g.plan, pass_of(0));
  Rec rn = my_items > 1 ? load_rec_t<TM>(g.plan, pass_of(1)) : empty_rec_t<TM>();
  int e_nn = my_items > 2 ? g.plan.pass_rec[2 * pass_of(2)].x : -1;

  const int chunks = K >> 3;
  auto issue_A = [&](const Rec& r, int buf) {
#pragma unroll
    for (int tk = 0; tk < TM; ++tk)
      if (tk < r.nt) {
        const uint32_t pr = (uint32_t)r.p[tk];
        const int64_t row = g.a_magic ? (int64_t)__umulhi(pr, g.a_magic) : (int64_t)pr;
        const __half* src = g.A + row * g.lda;
        const uint32_t dst = sa + (uint32_t)(buf * TM + tk) * a_pitch;
        for (int ch = tid; ch < chunks; ch += kMmaThreads) cp_async16_s(dst + (uint32_t)ch * 16u, src + ch * 8);
      }
  };

  // ---- weight fetch stream of this warp: lane = (row fr, 16-byte chunk fc) of every tensor's tile.
  // It runs S-1 stages ahead of the compute and crosses item boundaries (at most two items ahead).
  const int fr = lane >> 3, fc = lane & 7;
  const int64_t comp_step = 4 * g.w.comp_pair * KSL, meta_step = 4 * g.w.meta_row * KSL, scale_step = 2 * g.w.scale_row * KSL;
  const int64_t comp_row4 = 2 * g.w.comp_pair;
  const int64_t lane_comp = (int64_t)(4 * ks + (fr >> 1)) * g.w.comp_pair + (fr & 1) * g.w.comp_odd;
  const int64_t lane_meta = (int64_t)(4 * ks + fr) * g.w.meta_row;
  const int64_t lane_scale = (int64_t)(2 * ks + fr) * g.w.scale_row;
  const int lane_v = cgw * 128 + fc * 16;   // virtual column of this lane's chunk in the slab
  int i_cur = 0;                            // ordinal of the item being computed
  int f_i = 0, f_j = 0;
  uint32_t f_dst = ring + (uint32_t)lane * 16u;
  const uint8_t *f_comp = nullptr, *f_meta = nullptr, *f_scale = nullptr;
  auto fetch_next = [&]() {
    if (f_i < my_items) {
      if (f_j == 0) {
        const int rel = f_i - i_cur;
        const int e = rel == 0 ? rc.e : (rel == 1 ? rn.e : e_nn);
        const int slab = ((int)blockIdx.x + f_i * grid) % n_slabs;
        int col;
        if (kSilu) col = lane_v < 64 * CG ? slab * (64 * CG) + lane_v : g.inter + slab * (64 * CG) + (lane_v - 64 * CG);
        else col = slab * VCOLS + lane_v;
        f_comp = g.w.comp + ((int64_t)e * g.w.comp_e + col + lane_comp);
        f_meta = g.w.meta + ((int64_t)e * g.w.meta_e + col + lane_meta);
        f_scale = g.w.scale + ((int64_t)e * g.w.scale_e + col + lane_scale);
      }
      cp_async16_s(f_dst, f_comp);
      cp_async16_s(f_dst + 512u, f_comp + comp_row4);
      cp_async16_s(f_dst + 1024u, f_meta);
      if (lane < 16) cp_async16_s(f_dst + 1536u, f_scale);
      f_comp += comp_step;
      f_meta += meta_step;
      f_scale += scale_step;
      if (++f_j == nstep) {
        f_j = 0;
        ++f_i;
      }
    }
    cp_async_commit();
    f_dst += kMmaStageBytes;
    if (f_dst >= ring_end) f_dst -= ring_bytes;
  };

  // consumer side of the dependency: thread 0 reads a pass's counter (acquire) one item ahead, so the
  // load's latency is hidden; only a counter that is still short is polled (bounded), and the block's
  // next barrier releases the other threads
  auto load_count = [&](int pass) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(done + pass) : "memory");
    return v;
  };
  // A wait that runs out of its clock budget records B200FP4_MOE_STATUS_WAIT_EXPIRED in the plan header (the layer's
  // status word) and carries on with whatever the activation buffer holds; once the word is set no later wait of the
  // launch polls at all, so a broken launch still ends promptly.
  auto wait_pass = [&](int pass, int seen) {
    if (kDep == 2 && tid == 0 && pass >= 0 && seen < need) {
      volatile int* status = g.plan.hdr + 3;
      if (*status == 0) {
        const long long t0 = clock64();
        while (load_count(pass) < need) {
          if (clock64() - t0 > g.wait_cycles) {
            *status = B200FP4_MOE_STATUS_WAIT_EXPIRED;
            break;
          }
        }
      }
    }
  };
  // producer side: an item's output is complete for the whole block at the next block-wide barrier;
  // thread 0 then fences (cumulative over the barrier) and counts the item
  int finished_pass = -1;
  auto signal_finished = [&]() {
    if (kDep == 1 && tid == 0 && finished_pass >= 0) {
      __threadfence();
      atomicAdd(done + finished_pass, 1);
    }
  };
  int seen_next = 0;      // thread 0: counter of the next item's pass, read during the previous item
  wait_pass(pass_of(0), 0);
  if (kDep == 2) __syncthreads();
  if (kDep == 2 && tid == 0 && my_items > 1) seen_next = load_count(pass_of(1));
  issue_A(rc, 0);
  cp_async_commit();
#pragma unroll
  for (int s = 0; s < S - 1; ++s) fetch_next();

  // lane-constant pieces of the addresses used in a step
  const uint32_t off_comp = (uint32_t)t * 128u + (uint32_t)q * 16u;
  const uint32_t off_meta = 1024u + (uint32_t)(2 * (t & 1)) * 128u + (uint32_t)q * 16u + (uint32_t)(t >> 1) * 8u;
  const uint32_t off_scale = 1536u + (uint32_t)q * 16u;
  // B column q = token q (with four tokens per pass columns 4..7 repeat them; their results are never read),
  // k = 32*ks + 2t (+8i)
  const uint32_t off_b = (uint32_t)(TM == 8 ? q : (q & 3)) * a_pitch + (uint32_t)t * 4u + (uint32_t)ks * 64u;
  // scratch [warp][column 0..127][token 0..3]; the 16-byte token groups of a column are XOR-swizzled
  // by the column's quad so that neither side has bank conflicts
  // (tokens 4..7 of an 8-token pass, held by lanes t = 2, 3, go to a second block of the same shape)
  const uint32_t red_w = red + (uint32_t)(t >> 1) * kMmaRedBytes + (uint32_t)warp * 2048u + (uint32_t)q * 256u +
                         8u * (uint32_t)(t & 1) + 16u * (uint32_t)((q ^ ((cgw & 1) << 2)) & 7);

  uint32_t c_st = ring;
  int abuf = 0;
  for (; i_cur < my_items; ++i_cur) {
    const int slab = ((int)blockIdx.x + i_cur * grid) % n_slabs;
    Rec rnn = i_cur + 2 < my_items ? load_rec_t<TM>(g.plan, pass_of(i_cur + 2)) : empty_rec_t<TM>();
    const int e_n3 = i_cur + 3 < my_items ? g.plan.pass_rec[2 * pass_of(i_cur + 3)].x : -1;
    const float gmul = g.w.g[rc.e];
    // the group that carried this pass's activations is followed by nstep - 1 newer ones
    if (nstep >= S - 1) cp_async_wait<S - 2>();
    else if (nstep == 2) cp_async_wait<1>();
    else cp_async_wait<(S > 3 ? 2 : 1)>();
    wait_pass(i_cur + 1 < my_items ? pass_of(i_cur + 1) : -1, seen_next);
    __syncthreads();   // activations of this pass complete for all threads; scratch and the other buffer free
    signal_finished();
    issue_A(rn, abuf ^ 1);   // rides on the next committed weight stage
    if (kDep == 2 && tid == 0 && i_cur + 2 < my_items) seen_next = load_count(pass_of(i_cur + 2));

    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[j][k] = 0.f;
    uint32_t ab = sa + (uint32_t)abuf * TM * a_pitch + off_b;

    for (int js = 0; js < nstep; ++js) {
      cp_async_wait<S - 2>();
      __syncwarp();
      const uint32_t st = c_st;
      const uint4 v0 = lds128_at(st + off_comp), v1 = lds128_at(st + off_comp + 512u);
      const uint2 m0 = lds64_at(st + off_meta), m1 = lds64_at(st + off_meta + 128u);
      const uint4 s0 = lds128_at(st + off_scale), s1 = lds128_at(st + off_scale + 128u);
      uint32_t b[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) b[k] = lds32_at(ab + 16u * k);
      ab += 64u * KSL;
      c_st += kMmaStageBytes;
      if (c_st >= ring_end) c_st -= ring_bytes;
      fetch_next();   // into the slot read in the previous step (all lanes are past this step's __syncwarp)
      uint32_t em[4];
      em[0] = prmt(m0.x, m1.x, 0x5140u);
      em[1] = prmt(m0.x, m1.x, 0x7362u);
      em[2] = prmt(m0.y, m1.y, 0x5140u);
      em[3] = prmt(m0.y, m1.y, 0x7362u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // mma j: columns 2h, 2h+1 of the quad = bytes (2hf, 2hf+1) of word wi of every loaded vector
        constexpr int kH[8] = {0, 4, 1, 5, 2, 6, 3, 7};
        const int h = kH[j];
        const int wi = h >> 1, hf = h & 1;
        const uint32_t c0 = word_of(v0, wi), c1 = word_of(v1, wi);
        const __half2 sc0 = hf ? e4m3x2_to_h2<1>(word_of(s0, wi)) : e4m3x2_to_h2<0>(word_of(s0, wi));
        const __half2 sc1 = hf ? e4m3x2_to_h2<1>(word_of(s1, wi)) : e4m3x2_to_h2<0>(word_of(s1, wi));
        const __half2 a0 = __hmul2(hf ? e2m1x2_to_h2<2>(c0) : e2m1x2_to_h2<0>(c0), __low2half2(sc0));
        const __half2 a1 = __hmul2(hf ? e2m1x2_to_h2<3>(c0) : e2m1x2_to_h2<1>(c0), __high2half2(sc0));
        const __half2 a2 = __hmul2(hf ? e2m1x2_to_h2<2>(c1) : e2m1x2_to_h2<0>(c1), __low2half2(sc1));
        const __half2 a3 = __hmul2(hf ? e2m1x2_to_h2<3>(c1) : e2m1x2_to_h2<1>(c1), __high2half2(sc1));
        if ((j & 1) == 0)
          mma_sp_m16n8k32<0>(acc[j], *reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
                             *reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&a3), b, em[j >> 1]);
        else
          mma_sp_m16n8k32<1>(acc[j], *reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
                             *reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&a3), b, em[j >> 1]);
      }
    }

    // partial sums of this K-slice -> scratch
    if (2 * t < rc.nt) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        constexpr int kH[8] = {0, 4, 1, 5, 2, 6, 3, 7};
        const uint32_t c0 = 2u * kH[j], c1 = 2u * kH[j] + 1u;   // columns of the quad: rows q and q+8 of mma j
        sts64f_at((red_w ^ ((c0 & 7u) << 4)) + (c0 >> 3) * 128u, acc[j][0], acc[j][1]);
        sts64f_at((red_w ^ ((c1 & 7u) << 4)) + (c1 >> 3) * 128u, acc[j][2], acc[j][3]);
      }
    }
    __syncthreads();
    // epilogue, spread over all warps: one (column, token) sum per lane and round.  The warp of
    // K-slice s and column group cw is s * CG + cw.
    auto slice_sum = [&](int v, int tok) {
      const int cw = v >> 7, col = v & 127;
      const uint32_t a = red + (uint32_t)(tok >> 2) * kMmaRedBytes + (uint32_t)cw * 2048u +
                         (((uint32_t)col * 16u) ^ ((uint32_t)(((col >> 4) ^ ((cw & 1) << 2)) & 7) << 4)) + (uint32_t)(tok & 3) * 4u;
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < KSL; ++s) sum += __uint_as_float(lds32_at(a + (uint32_t)(s * CG) * 2048u));
      return sum;
    };
    if (kSilu) {
#pragma unroll
      for (int r = 0; r < CG * (TM / 4); ++r) {
        const int idx = (r % CG) * 256 + warp * 16 + (lane & 15);
        const int col_g = idx >> 2, tok = (idx & 3) + 4 * (r / CG);
        const float sum = slice_sum(col_g + (lane >> 4) * (64 * CG), tok);
        const float other = __shfl_down_sync(0xffffffffu, sum, 16);
        if (lane < 16 && tok < rc.nt) {
          const float gate = sum * gmul, up = other * gmul;
          store_out(g.out, g.out_dtype, (int64_t)rc.pair(tok) * g.ldo + slab * (64 * CG) + col_g,
                    gate / (1.0f + __expf(-gate)) * up);
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < CG * (TM / 4); ++r) {
        const int x = (r % CG) * 512 + tid;
        const int v = x >> 2, tok = (x & 3) + 4 * (r / CG);
        const float sum = slice_sum(v, tok);
        if (tok < rc.nt) store_out(g.out, g.out_dtype, (int64_t)rc.pair(tok) * g.ldo + slab * VCOLS + v, sum * gmul);
      }
    }
    if (kDep == 1) finished_pass = pass_of(i_cur);   // counted after the next block-wide barrier
    rc = rn;
    rn = rnn;
    e_nn = e_n3;
    abuf ^= 1;
  }
  cp_async_wait<0>();
  if (kDep == 1) {
    __syncthreads();
    signal_finished();
  }
}

// Programmatic dependent launch: the GEMV and reduce kernels of a layer are launched with the stream-serialization
// attribute, so their blocks may become resident while the kernel before them drains; pdl_wait() returns once that
// kernel has completed and its writes are visible (at once when the launch carried no such attribute).


template <int CG, int S, bool kSilu, int TM>
__global__ void __launch_bounds__(kMmaThreads, 1) sparse_gemv_mma_kernel(const GemvArgs g) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch_dependents();
  gemv_mma_phase<CG, S, kSilu, 0, TM>(g, smem, nullptr, 0);
}

// Both projections of the MoE layer in one launch: every block first walks its gate_up items, then its
// down items.  A down item only needs the activations of its own pass, so blocks that run out of
// gate_up items start on the down projection of passes finished long ago instead of idling through
// the last, partial round and a second kernel's ramp-up.  Launched cooperatively (all blocks
// co-resident), so a block polling for a pass can never keep the block that produces it off the GPU.
template <int CGA, int SA, int CGB, int SB, int TM>
__global__ void __launch_bounds__(kMmaThreads, 1)
    fused_moe_mma_kernel(const GemvArgs ga, const GemvArgs gb, int* done, int need) {
  extern __shared__ __align__(16) unsigned char smem[];
  gemv_mma_phase<CGA, SA, true, 1, TM>(ga, smem, done, need);
  __syncthreads();              // the second phase lays shared memory out anew
  gemv_mma_phase<CGB, SB, false, 2, TM>(gb, smem, done, need);
}

// ------------------------------------------------------------------------------------------ warp-scheduled tensor-core GEMV
//
// The same arithmetic as gemv_mma_phase (mma.sp m16n8k32, hardware E2M1 / E4M3 decode), organised so that a warp
// never has to meet another warp:
//   * a work item is (pass of up to eight tokens, group of 128 output columns) over the WHOLE K, owned by one warp:
//     no K-slices, so no partial sums in shared memory, no block-wide barrier and no block-wide epilogue;
//   * warps take items from a global counter (atomicAdd by lane 0), always holding the next item while they
//     compute the current one, so the tail of the launch is at most one item long whatever the routing;
//   * the activations are not staged per block: the plan kernel (or the gate_up epilogue) leaves them in
//     "fragment order" (see kConv*), and each lane copies the 16 bytes that are its own B-operand registers for a
//     k-step asynchronously into its ring stage, next to the weights of that step;
//   * a ring stage is one 32-wide k-step: 8 compressed rows, 4 metadata rows and 2 scale rows of 128 columns
//     (1792 bytes) + 512 bytes of B fragments.  Four stages per warp; the copy for step j+4 is issued into the slot
//     of step j as soon as step j's shared-memory reads are done, so that four steps are in flight per warp and the
//     slot of every step is a compile-time constant in the loop unrolled by four (K is a multiple of 128).  The
//     stream runs across item boundaries.
//   * 16-byte chunks are XOR-swizzled inside the compressed and metadata rows so that the fragment loads
//     (rows t and t+4 for lane t of a quad; metadata rows 2(t%2), 2(t%2)+1) touch every bank once.
// Epilogue from registers: the lane that holds 16 consecutive columns of a token writes them with 16-byte stores;
// with SiLU the warp's 128 columns are 64 gate + the matching 64 up columns, the two halves of the warp swap one
// token's values through shuffles, and SiLU(gate)*up leaves in fragment order for the down projection.
// Two shapes of the same ring budget: 8 warps x 8 stages per block (the default where K is a multiple of 256: two warps
// per scheduler, each with twice the bytes in flight, measured faster at every batch size tried), or 16 warps x 4 stages.
constexpr int kWsStages = 4;
constexpr int kWsWarps = 16;
constexpr int kWsThreads = 32 * kWsWarps;
constexpr int kWsStageBytes = 14 * 128 + 512;     // 8 compressed + 4 metadata + 2 scale rows of 128 bytes, B fragments of 8 tokens
constexpr size_t kWsSmemBytes = (size_t)kWsWarps * kWsStages * kWsStageBytes + 128;
// (warps per block = 64 / stages, so both shapes use the same shared memory)

// Lane-constant shared-memory offsets of the warp-scheduled kernel.
// Stage layout: compressed rows 0..7 | metadata rows 0..3 | scale rows 0..1 (128 bytes each) | B fragments.  The 16-byte
// chunks of a compressed row r sit at chunk ^ 2(r%4), those of a metadata row at chunk ^ 4(r/2), so that the fragment
// loads (rows t and t+4 for lane t of a quad; metadata rows 2(t%2), 2(t%2)+1) spread over all banks.
struct WsLane {
  uint32_t ring;                                   // this warp's ring
  uint32_t d_comp, d_meta, d_scale, d_b;           // where this lane's copies land (compressed rows fr and fr+4, metadata / scale row fr)
  uint32_t off_comp, off_meta, off_scale;          // where its fragments are read from
  int lane, q, t, fr, fc;
};

template <int kS = kWsStages>
__device__ __forceinline__ WsLane ws_lane(unsigned char* smem) {
  WsLane L;
  L.lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  L.q = L.lane >> 2;
  L.t = L.lane & 3;
  L.fr = L.lane >> 3;
  L.fc = L.lane & 7;
  L.ring = ((shared_addr(smem) + 127u) & ~127u) + (uint32_t)warp * (kS * kWsStageBytes);
  L.d_comp = (uint32_t)L.fr * 128u + (uint32_t)((L.fc ^ (2 * (L.fr & 3))) << 4);
  L.d_meta = 1024u + (uint32_t)L.fr * 128u + (uint32_t)((L.fc ^ (4 * (L.fr >> 1))) << 4);
  L.d_scale = 1536u + (uint32_t)L.fr * 128u + (uint32_t)L.fc * 16u;
  L.d_b = 1792u + (uint32_t)L.lane * 16u;
  L.off_comp = (uint32_t)L.t * 128u + (uint32_t)((L.q ^ (2 * L.t)) << 4);
  L.off_meta = 1024u + (uint32_t)(2 * (L.t & 1)) * 128u + (uint32_t)((L.q ^ (4 * (L.t & 1))) << 4) + (uint32_t)(L.t >> 1) * 8u;
  L.off_scale = 1536u + (uint32_t)L.q * 16u;
  return L;
}

// One projection for this warp: the items [base, base + passes * groups) of the claim sequence that `counter` hands out.
// `first` is an index this warp has already claimed; the return value is the first index it claimed that lies past
// this projection (the caller passes it on to the next one).
// kDep links the two projections of the MoE layer when they run in one launch: 1 = producer (done[pass] counts the
// finished items of a pass, fenced), 2 = consumer (the B fragments of an item -- the activations the producer wrote
// for that pass -- are fetched only once done[pass] has reached `need`), 0 = stand-alone.
// A consumer only ever waits for items of the first projection, and each of those is held either by a running warp (it
// was claimed before any item of the second projection) or by the warp of this grid it is statically assigned to (index <
// number of warps; the grid has at most one block per SM, so that warp becomes resident without anyone's help): the wait
// cannot deadlock; it is bounded all the same and reports through the status word.
template <bool kSilu, int kN, int kDep, int kS = kWsStages>
__device__ __forceinline__ int ws_phase(const GemvArgs& g, int* counter, const int base, int first, const WsLane& L,
                                        int* done, const int need) {
  const int lane = L.lane, q = L.q, t = L.t;
  const int N = kN ? kN : g.N;
  const int nblk = g.K / (32 * kS);          // blocks of kS 32-wide k-steps (one turn of the ring)
  const int groups = g.n_slabs;              // 128-column groups per pass
  const int n_items = g.plan.hdr[1] * groups;
  if (first - base >= n_items) return first;

  // warp w of the grid starts on item w without asking (one round trip to the counter less before the first byte is
  // requested); the counter hands out the items after those
  const int n_warps = (int)(gridDim.x * (blockDim.x >> 5));
  auto claim = [&]() {
    int v = 0;
    if (lane == 0) v = atomicAdd(counter, 1) + n_warps;
    return __shfl_sync(0xffffffffu, v, 0);
  };
  // An item as read from its pass record: expert, group, and the pairs this lane deals with (B column q; the one or two
  // tokens whose outputs it stores).  Pairs 0..3 sit in the record, later ones in pairs[].
  struct Item {
    int e, grp, pass, pb, ps0, ps1;
    bool valid;
  };
  auto pair_of = [&](const int4& x, const int4& y, int tok) {
    if (tok >= 4) return g.plan.pairs[y.z + tok];
    return tok == 0 ? x.z : (tok == 1 ? x.w : (tok == 2 ? y.x : y.y));
  };
  auto describe = [&](int claimed) {
    Item d;
    const int it = claimed - base;
    d.valid = it < n_items;
    d.e = d.grp = d.pass = d.pb = 0;
    d.ps0 = d.ps1 = -1;
    if (!d.valid) return d;
    d.pass = it / groups;
    d.grp = it - d.pass * groups;
    const int4 x = g.plan.pass_rec[2 * d.pass], y = g.plan.pass_rec[2 * d.pass + 1];
    d.e = x.x;
    const int nt = x.y;
    // B column q = token q of the pass; columns past the last token repeat token 0 (their results are never stored)
    d.pb = pair_of(x, y, q < nt ? q : 0);
    const int s0 = kSilu ? 2 * t + (lane >> 4) : 2 * t;
    if (s0 < nt) d.ps0 = pair_of(x, y, s0);
    if (!kSilu && s0 + 1 < nt) d.ps1 = pair_of(x, y, s0 + 1);
    return d;
  };
  // this lane's copy sources at k-step 0 of an item
  struct Fetch {
    const uint8_t *pc, *pm, *ps;
    const __half* pb;
    bool valid;
  };
  auto sources = [&](const Item& d) {
    Fetch f;
    f.valid = d.valid;
    f.pc = f.pm = f.ps = nullptr;
    f.pb = nullptr;
    if (!d.valid) return f;
    if (kDep == 2) {
      // the activations of this pass must be complete before any lane asks for them
      if (lane == 0) {
        volatile int* status = g.plan.hdr + 3;
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(done + d.pass) : "memory");
        if (v < need && *status == 0) {
          const long long t0 = clock64();
          do {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(done + d.pass) : "memory");
            if (clock64() - t0 > g.wait_cycles) {
              *status = B200FP4_MOE_STATUS_WAIT_EXPIRED;
              break;
            }
          } while (v < need);
        }
      }
      __syncwarp();
    }
    const uint32_t pr = (uint32_t)d.pb;
    const int64_t row = g.a_magic ? (int64_t)__umulhi(pr, g.a_magic) : (int64_t)pr;
    f.pb = g.A + row * g.lda + t * 8;
    int col;
    if (kSilu) col = L.fc < 4 ? d.grp * 64 + L.fc * 16 : g.inter + d.grp * 64 + (L.fc - 4) * 16;
    else col = d.grp * 128 + L.fc * 16;
    const int64_t lane_off = (int64_t)L.fr * N + col;
    f.pc = g.w.comp + ((int64_t)d.e * g.w.comp_e + lane_off);
    f.pm = g.w.meta + ((int64_t)d.e * g.w.meta_e + lane_off);
    f.ps = g.w.scale + ((int64_t)d.e * g.w.scale_e + lane_off);
    return f;
  };
  // copies of k-step `u` (relative to f) into ring slot u; always one commit group, so that the wait counts stay fixed
  auto fetch = [&](const Fetch& f, int u) {
    if (f.valid) {
      const uint32_t dst = L.ring + (uint32_t)u * kWsStageBytes;
      const uint8_t* c = f.pc + (int64_t)u * 8 * N;
      cp_async16_s(dst + L.d_comp, c);
      cp_async16_s(dst + 512u + L.d_comp, c + (int64_t)4 * N);
      cp_async16_s(dst + L.d_meta, f.pm + (int64_t)u * 4 * N);
      if (lane < 16) cp_async16_s(dst + L.d_scale, f.ps + (int64_t)u * 2 * N);
      cp_async16_s(dst + L.d_b, f.pb + u * 32);
    }
    cp_async_commit();
  };
  auto advance = [&](Fetch& f) {     // kS k-steps on
    f.pc += (int64_t)(8 * kS) * N;
    f.pm += (int64_t)(4 * kS) * N;
    f.ps += (int64_t)(2 * kS) * N;
    f.pb += 32 * kS;
  };

  Item cur = describe(first);
  Fetch F = sources(cur);
#pragma unroll
  for (int u = 0; u < kS; ++u) fetch(F, u);     // the first kS k-steps of the first item
  advance(F);
  int carry;

  while (true) {
    carry = claim();
    const Item nxt = describe(carry);
    const float gmul = g.w.g[cur.e];
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[j][k] = 0.f;

    for (int b = 0; b < nblk; ++b) {
      if (b == nblk - 1) F = sources(nxt);     // the last block of an item prefetches the first block of the next one
#pragma unroll
      for (int u = 0; u < kS; ++u) {
        cp_async_wait<kS - 1>();
        __syncwarp();
        const uint32_t st = L.ring + (uint32_t)u * kWsStageBytes;
        const uint4 v0 = lds128_at(st + L.off_comp), v1 = lds128_at(st + L.off_comp + 512u);
        const uint2 m0 = lds64_at(st + L.off_meta), m1 = lds64_at(st + L.off_meta + 128u);
        const uint4 s0 = lds128_at(st + L.off_scale), s1 = lds128_at(st + L.off_scale + 128u);
        const uint4 bv = lds128_at(st + L.d_b);
        const uint32_t bf[4] = {bv.x, bv.y, bv.z, bv.w};
        fetch(F, u);                 // k-step kS ahead, into the slot that was just read
        uint32_t em[4];
        em[0] = prmt(m0.x, m1.x, 0x5140u);
        em[1] = prmt(m0.x, m1.x, 0x7362u);
        em[2] = prmt(m0.y, m1.y, 0x5140u);
        em[3] = prmt(m0.y, m1.y, 0x7362u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // mma j takes columns 2h, 2h+1 of every quad as its rows q and q+8: bytes (2hf, 2hf+1) of word wi of the
          // loaded vectors.  Even j: metadata from lanes t = 0, 1 (first half of the quad's columns), odd j: t = 2, 3.
          constexpr int kH[8] = {0, 4, 1, 5, 2, 6, 3, 7};
          const int h = kH[j];
          const int wi = h >> 1, hf = h & 1;
          const uint32_t c0 = word_of(v0, wi), c1 = word_of(v1, wi);
          const __half2 sc0 = hf ? e4m3x2_to_h2<1>(word_of(s0, wi)) : e4m3x2_to_h2<0>(word_of(s0, wi));
          const __half2 sc1 = hf ? e4m3x2_to_h2<1>(word_of(s1, wi)) : e4m3x2_to_h2<0>(word_of(s1, wi));
          const __half2 a0 = __hmul2(hf ? e2m1x2_to_h2<2>(c0) : e2m1x2_to_h2<0>(c0), __low2half2(sc0));
          const __half2 a1 = __hmul2(hf ? e2m1x2_to_h2<3>(c0) : e2m1x2_to_h2<1>(c0), __high2half2(sc0));
          const __half2 a2 = __hmul2(hf ? e2m1x2_to_h2<2>(c1) : e2m1x2_to_h2<0>(c1), __low2half2(sc1));
          const __half2 a3 = __hmul2(hf ? e2m1x2_to_h2<3>(c1) : e2m1x2_to_h2<1>(c1), __high2half2(sc1));
          if ((j & 1) == 0)
            mma_sp_m16n8k32<0>(acc[j], *reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
                               *reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&a3), bf, em[j >> 1]);
          else
            mma_sp_m16n8k32<1>(acc[j], *reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
                               *reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&a3), bf, em[j >> 1]);
        }
      }
      advance(F);
    }

    // ---- epilogue from registers.  Column 2h + r of the quad's 16 columns for token 2t + b is acc[kJ[h]][2r + b].
    constexpr int kJ[8] = {0, 2, 4, 6, 1, 3, 5, 7};
    if (kSilu) {
      const int hi = lane >> 4;                       // lanes 0..15 hold gate columns, lanes 16..31 the matching up columns
      uint32_t words[8];
#pragma unroll
      for (int h = 0; h < 8; ++h) {
        float a[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          // each half of the warp finishes one of the quad's two tokens: it keeps its own value for that token and
          // sends the other token's value to the lane that holds the matching gate / up column
          const float keep = hi ? acc[kJ[h]][2 * r + 1] : acc[kJ[h]][2 * r];
          const float send = hi ? acc[kJ[h]][2 * r] : acc[kJ[h]][2 * r + 1];
          const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
          const float gate = (hi ? recv : keep) * gmul, up = (hi ? keep : recv) * gmul;
          a[r] = gate / (1.0f + __expf(-gate)) * up;
        }
        const __half2 hv = __floats2half2_rn(a[0], a[1]);
        words[h] = *reinterpret_cast<const uint32_t*>(&hv);
      }
      if (cur.ps0 >= 0) {
        // fragment order: this lane's 16 gate columns are words 8(q%2) + m, m = 0..7, of the 32-column group
        // 2 grp + (q%4)/2; word w goes to position 4(w%4) + w/4, so words m and m+4 are neighbours
        __half* dst = reinterpret_cast<__half*>(g.out) + (int64_t)cur.ps0 * g.ldo + (cur.grp * 2 + ((q & 3) >> 1)) * 32 + 4 * (q & 1);
#pragma unroll
        for (int m = 0; m < 4; ++m) *reinterpret_cast<uint2*>(dst + 8 * m) = make_uint2(words[m], words[m + 4]);
      }
    } else {
#pragma unroll
      for (int b2 = 0; b2 < 2; ++b2) {
        const int pair = b2 ? cur.ps1 : cur.ps0;
        if (pair >= 0) {
          const int64_t o = (int64_t)pair * g.ldo + cur.grp * 128 + q * 16;
          float v[16];
#pragma unroll
          for (int h = 0; h < 8; ++h) {
            v[2 * h] = acc[kJ[h]][b2] * gmul;
            v[2 * h + 1] = acc[kJ[h]][2 + b2] * gmul;
          }
          if (g.out_dtype == B200FP4_DTYPE_F32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(g.out) + o);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (g.out_dtype == B200FP4_DTYPE_F16) {
                const __half2 hv = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&hv);
              } else {
                const __nv_bfloat162 bv2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&bv2);
              }
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(g.out) + o);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
          }
        }
      }
    }
    if (kDep == 1) {
      // this item's activations are stored: make them visible, then count the item for its pass
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        atomicAdd(done + cur.pass, 1);
      }
    }
    if (!nxt.valid) break;
    cur = nxt;
  }
  cp_async_wait<0>();
  __syncwarp();
  return carry;
}

template <bool kSilu, int kN, int kS = kWsStages, int kW = kWsWarps>
__global__ void __launch_bounds__(32 * kW, 1) sparse_gemv_ws_kernel(const GemvArgs g, int* counter) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch_dependents();
  const WsLane L = ws_lane<kS>(smem);
  int first = (int)(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5));
  ws_phase<kSilu, kN, 0, kS>(g, counter, 0, first, L, nullptr, 0);
}

// Both projections of the MoE layer in one launch: the claim sequence runs through the gate_up items and on into the
// down items, so a warp that finds no gate_up item left starts on the down projection of passes that are complete
// instead of idling until the slowest warp of a first launch has finished and a second launch has ramped up.
template <int kNA, int kNB, int kS = kWsStages, int kW = kWsWarps>
__global__ void __launch_bounds__(32 * kW, 1)
    fused_moe_ws_kernel(const GemvArgs ga, const GemvArgs gb, int* counter, int* done, int need) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch_dependents();
  const WsLane L = ws_lane<kS>(smem);
  int first = (int)(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5));
  const int n_a = ga.plan.hdr[1] * ga.n_slabs;
  first = ws_phase<true, kNA, 1, kS>(ga, counter, 0, first, L, done, need);
  ws_phase<false, kNB, 2, kS>(gb, counter, n_a, first, L, done, need);
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

// Where the rows of the layer's result go when they are not one [M, H] tensor: row m is row dest_row0 + m % rows_per_dest
// of the buffer ptrs[m / rows_per_dest] (expert parallelism over peer memory: the partial rows of the tokens of rank g go
// straight into rank g's buffer).  ptrs == nullptr: the plain tensor.
struct OutScatter {
  void* const* ptrs;
  int rows_per_dest, dest_row0;
  // the layer's status word, forwarded by its last kernel (status_out may be host memory the device can address)
  int* status_out = nullptr;
  const int* status_src = nullptr;
};

// out[m, h] = sum_t weight(m,t) * down[m*topk + t, h] over pairs whose expert is local.
// One thread = four columns of one token; the rows of eight slots are requested before the first is used (the kernel is
// pure latency: 2.6 MB at batch 32), the sum runs in slot order.  H % 4 == 0.
constexpr int kRedThreads = 128;
__global__ void __launch_bounds__(kRedThreads)
    weighted_reduce_kernel(const float* __restrict__ down, const float* __restrict__ topk_w, const int* __restrict__ mapped,
                           void* out, int out_dtype, int M, int topk, int H, int unweighted, int64_t ld_w, OutScatter sc) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = (blockIdx.x * kRedThreads + threadIdx.x) * 4;
  int m = blockIdx.y;
  if (sc.status_out != nullptr && h == 0 && m == 0) *sc.status_out = *sc.status_src;
  if (h >= H || m >= M) return;
  const int m_src = m;
  if (sc.ptrs != nullptr) {
    out = sc.ptrs[m / sc.rows_per_dest];
    m = sc.dest_row0 + m % sc.rows_per_dest;
  }
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int t0 = 0; t0 < topk; t0 += 8) {
    float4 v[8];
    float w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = t0 + i;
      const int p = m_src * topk + t;
      const bool on = t < topk && mapped[p] >= 0;
      v[i] = on ? *reinterpret_cast<const float4*>(down + (int64_t)p * H + h) : make_float4(0.f, 0.f, 0.f, 0.f);
      w[i] = on ? (unweighted ? 1.0f : topk_w[(int64_t)m_src * ld_w + t]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a.x += v[i].x * w[i];
      a.y += v[i].y * w[i];
      a.z += v[i].z * w[i];
      a.w += v[i].w * w[i];
    }
  }
  const int64_t o = (int64_t)m * H + h;
  if (out_dtype == B200FP4_DTYPE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o) = a;
  } else if (out_dtype == B200FP4_DTYPE_F16) {
    const __half2 lo = __floats2half2_rn(a.x, a.y), hi = __floats2half2_rn(a.z, a.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + o) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  } else {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + o) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  }
}

inline dim3 reduce_grid(int64_t H, int64_t M) { return dim3((unsigned)((H + 4 * kRedThreads - 1) / (4 * kRedThreads)), (unsigned)M); }

// ------------------------------------------------------------------------------------------ host

// Optional CUDA events recorded around the two GEMV launches of the fused layer (benchmark hook).
cudaEvent_t g_prof_events[3] = {nullptr, nullptr, nullptr};

// One-launch layer: clock64 budget of a wait on a pass counter (~1 s at 2 GHz) and a diagnostic surplus added to the
// count a down-projection item waits for (b200fp4_fused_moe_set_wait_limit).
constexpr long long kDefaultWaitCycles = 2000000000LL;
long long g_wait_cycles = kDefaultWaitCycles;
int g_wait_extra_need = 0;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int64_t max_passes(int64_t P, int64_t E) { return (P < E ? P : E) + P / kMaxTok + 1; }

// plan layout: hdr[8] | pairs[P] | mapped[P] | (16-byte aligned) pass_rec[max_passes][2] int4
size_t plan_bytes(int64_t P, int64_t E) {
  return align_up(sizeof(int) * (size_t)(8 + 2 * P), 16) + (size_t)max_passes(P, E) * 2 * sizeof(int4);
}

Plan carve_plan(void* ws, int64_t P, int64_t E) {
  (void)E;
  int* base = reinterpret_cast<int*>(ws);
  Plan pl;
  pl.hdr = base;
  pl.pairs = base + 8;
  pl.mapped = pl.pairs + P;
  pl.pass_rec = reinterpret_cast<int4*>(reinterpret_cast<unsigned char*>(ws) + align_up(sizeof(int) * (size_t)(8 + 2 * P), 16));
  return pl;
}

struct GemvCfg {
  int nt, cols, cg, stages;
  size_t smem;
  bool ok;
};

size_t gemv_smem(int nt, int cols, int cg, int stages, bool scale8, int64_t K) {
  const int nv = scale8 ? 8 : 7;
  return (size_t)kLutBytes + (size_t)stages * nv * nt * cols + (size_t)(nt / 32) * kMaxTok * cg * cols * 4 +
         (size_t)2 * kMaxTok * K * 2;
}

// Picks slab shape and ring depth for a K.  Every thread must own >= stages-1 scale blocks per item.
// (The kernel template also builds as 512 threads x 8 columns per thread; on B200 that variant
// measured 20 % slower at batch 32 -- 177 vs 148 us per layer -- so it is not instantiated.)
GemvCfg pick_cfg(int64_t K, bool scale8) {
  GemvCfg c = {0, 0, 0, 0, 0, false};
  const int64_t KB = K / 16;
  c.nt = kThreads;
  c.cols = 16;
  c.cg = KB >= 96 ? 8 : (KB >= 16 ? 16 : 32);
  const int64_t KS = c.nt / c.cg;
  const int64_t min_blocks = KB / KS;
  if (min_blocks < 1) return c;
  for (int s = (c.cg == 32 ? 2 : 4); s >= 2; --s) {
    if (min_blocks < s - 1) continue;
    const size_t smem = gemv_smem(c.nt, c.cols, c.cg, s, scale8, K);
    if (smem <= 227 * 1024) {
      c.stages = s;
      c.smem = smem;
      c.ok = true;
      return c;
    }
  }
  return c;
}

template <int NT, int COLS, int CG, int S, bool kScale8, bool kSilu>
int launch_gemv_t(const GemvArgs& g, int64_t grid, size_t smem, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sparse_gemv_kernel<NT, COLS, CG, S, kScale8, kSilu>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  sparse_gemv_kernel<NT, COLS, CG, S, kScale8, kSilu><<<(unsigned)grid, NT, smem, st>>>(g);
  return B200FP4_STATUS_SUCCESS;
}

// ---- tensor-core kernel: configuration and launch
struct MmaCfg {
  int cg, stages, tm;
  bool ok;
};

size_t mma_smem_bytes(int64_t K, int stages, int tm) {
  const size_t a_bytes = align_up((size_t)2 * tm * (2 * (size_t)K + 16), 1024);
  return 1024 + a_bytes + (size_t)(tm / 4) * kMmaRedBytes + (size_t)kMmaWarps * stages * kMmaStageBytes;
}

// `passes` is an upper bound of the number of passes (the real number is only known on the device).
// Wide items (more column groups) have less per-item work to amortise, but with few passes they leave
// SMs without an item, so small batches take the narrowest shape that is allowed.
MmaCfg pick_mma_cfg(int64_t N, int64_t K, int64_t G, int inter_silu, int64_t passes, int tm) {
  MmaCfg c = {0, 0, tm, false};
  if (G != K / 16 || K % 32 != 0) return c;
  const int order_silu[3] = {2, 4, 1}, order_plain[3] = {4, 2, 1};
  const int order_small[3] = {1, 2, 4};
  const int64_t slabs_wide = inter_silu > 0 ? inter_silu / 128 : N / 512;     // slabs per pass of the preferred wide shape
  const bool small = passes * (slabs_wide > 0 ? slabs_wide : 1) < 2 * (int64_t)sm_count();
  for (int i = 0; i < 3; ++i) {
    const int cg = small ? order_small[i] : (inter_silu > 0 ? order_silu[i] : order_plain[i]);
    const int ksl = kMmaWarps / cg;
    const bool cols_ok = inter_silu > 0 ? (inter_silu % (64 * cg) == 0 && N == 2 * (int64_t)inter_silu) : (N % (128 * cg) == 0);
    if (cols_ok && K % (32 * ksl) == 0 && K / (32 * ksl) >= 2) {
      for (int s = 5; s >= 3; s -= 2)
        if (mma_smem_bytes(K, s, tm) <= 227 * 1024 && (s - 2 < 2 * (int)(K / (32 * ksl)))) {
          c.cg = cg;
          c.stages = s;
          c.ok = true;
          return c;
        }
    }
  }
  return c;
}

template <int CG, int S, bool kSilu, int TM>
int launch_mma_t(const GemvArgs& g, int64_t grid, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sparse_gemv_mma_kernel<CG, S, kSilu, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  launch_pdl(sparse_gemv_mma_kernel<CG, S, kSilu, TM>, dim3((unsigned)grid), dim3(kMmaThreads), mma_smem_bytes(g.K, S, TM), st,
             g);
  return B200FP4_STATUS_SUCCESS;
}

template <bool kSilu>
int launch_mma(const GemvArgs& g, const MmaCfg& c, int64_t grid, cudaStream_t st) {
  if (c.tm == 8) {
    if (c.stages == 5) {
      if (c.cg == 1) return launch_mma_t<1, 5, kSilu, 8>(g, grid, st);
      if (c.cg == 2) return launch_mma_t<2, 5, kSilu, 8>(g, grid, st);
      return launch_mma_t<4, 5, kSilu, 8>(g, grid, st);
    }
    if (c.cg == 1) return launch_mma_t<1, 3, kSilu, 8>(g, grid, st);
    if (c.cg == 2) return launch_mma_t<2, 3, kSilu, 8>(g, grid, st);
    return launch_mma_t<4, 3, kSilu, 8>(g, grid, st);
  }
  if (c.stages == 5) {
    if (c.cg == 1) return launch_mma_t<1, 5, kSilu, 4>(g, grid, st);
    if (c.cg == 2) return launch_mma_t<2, 5, kSilu, 4>(g, grid, st);
    return launch_mma_t<4, 5, kSilu, 4>(g, grid, st);
  }
  if (c.cg == 1) return launch_mma_t<1, 3, kSilu, 4>(g, grid, st);
  if (c.cg == 2) return launch_mma_t<2, 3, kSilu, 4>(g, grid, st);
  return launch_mma_t<4, 3, kSilu, 4>(g, grid, st);
}

// ---- warp-scheduled tensor-core kernel: conditions and launch
// One scale per 16 k, K in whole blocks of four 32-wide steps, whole 128-column groups (SiLU: 64 gate + 64 up), and the
// reference's separate [E, rows, N] tensors (the interleaved layout goes to the general kernel).
bool ws_ok(int64_t N, int64_t K, int64_t G, int64_t inter_silu, const SparseWeights& w) {
  if (G != K / 16 || K % 128 != 0) return false;
  if (inter_silu > 0) {
    if (inter_silu % 64 != 0 || N != 2 * inter_silu) return false;
  } else if (N % 128 != 0) {
    return false;
  }
  return w.comp_pair == 2 * N && w.comp_odd == N && w.meta_row == N && w.scale_row == N;
}

// Opt a kernel in to the large dynamic shared memory, once per device; `attr_set` belongs to the caller, one array per
// kernel instantiation (instantiations share their function type, so a static in here would be shared between them).
template <typename Kernel>
bool ws_prepare(Kernel kernel, bool* attr_set, size_t smem_bytes = kWsSmemBytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return false;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    attr_set[dev] = true;
  }
  return true;
}

int64_t ws_grid(int64_t max_items) {
  int64_t grid = (max_items + kWsWarps - 1) / kWsWarps;
  if (grid > (int64_t)sm_count()) grid = sm_count();
  return grid < 1 ? 1 : grid;
}

template <bool kSilu, int kN, int kS = kWsStages, int kW = kWsWarps>
int launch_ws_t(const GemvArgs& g, int* counter, int64_t max_items, cudaStream_t st) {
  static bool attr_set[64] = {false};
  constexpr size_t smem = (size_t)kW * kS * kWsStageBytes + 128;
  if (!ws_prepare(sparse_gemv_ws_kernel<kSilu, kN, kS, kW>, attr_set, smem)) return B200FP4_STATUS_EXECUTION_FAILED;
  int64_t grid = (max_items + kW - 1) / kW;
  if (grid > (int64_t)sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  launch_pdl(sparse_gemv_ws_kernel<kSilu, kN, kS, kW>, dim3((unsigned)grid), dim3(32 * kW), smem, st, g, counter);
  return B200FP4_STATUS_SUCCESS;
}

GemvArgs make_args(const SparseWeights& w, const Plan& plan, const __half* A, int64_t lda, int a_div, void* out,
                   int out_dtype, int64_t ldo, int64_t N, int64_t K, int inter_silu);

// A in fragment order, plan cut into passes of eight tokens, *counter zero (the plan kernel clears it).
int run_projection_ws(const SparseWeights& w, const Plan& plan, const __half* A, int64_t lda, int a_div, void* out,
                      int out_dtype, int64_t ldo, int64_t P, int64_t N, int64_t K, int64_t E, int inter_silu,
                      int* counter, cudaStream_t st) {
  GemvArgs g = make_args(w, plan, A, lda, a_div, out, out_dtype, ldo, N, K, inter_silu);
  g.n_slabs = inter_silu > 0 ? inter_silu / 64 : (int)(N / 128);
  const int64_t items = max_passes(P, E) * g.n_slabs;
  if (K % 256 == 0) {      // 8 warps x 8-stage rings (see the fused layer for the measurements)
    if (inter_silu > 0)
      return N == 1024 ? launch_ws_t<true, 1024, 8, 8>(g, counter, items, st) : launch_ws_t<true, 0, 8, 8>(g, counter, items, st);
    return N == 2048 ? launch_ws_t<false, 2048, 8, 8>(g, counter, items, st) : launch_ws_t<false, 0, 8, 8>(g, counter, items, st);
  }
  if (inter_silu > 0) return N == 1024 ? launch_ws_t<true, 1024>(g, counter, items, st) : launch_ws_t<true, 0>(g, counter, items, st);
  return N == 2048 ? launch_ws_t<false, 2048>(g, counter, items, st) : launch_ws_t<false, 0>(g, counter, items, st);
}

template <int kNA, int kNB, int kS = kWsStages, int kW = kWsWarps>
int launch_fused_ws_t(const GemvArgs& ga, const GemvArgs& gb, int* counter, int* done, int need, int64_t max_items,
                      cudaStream_t st) {
  static bool attr_set[64] = {false};
  constexpr size_t smem = (size_t)kW * kS * kWsStageBytes + 128;
  static_assert(smem <= 227 * 1024, "shared memory of the ring");
  if (!ws_prepare(fused_moe_ws_kernel<kNA, kNB, kS, kW>, attr_set, smem)) return B200FP4_STATUS_EXECUTION_FAILED;
  int64_t grid = (max_items + kW - 1) / kW;
  if (grid > (int64_t)sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  launch_pdl(fused_moe_ws_kernel<kNA, kNB, kS, kW>, dim3((unsigned)grid), dim3(32 * kW), smem, st, ga, gb, counter, done, need);
  return B200FP4_STATUS_SUCCESS;
}

template <bool kScale8, bool kSilu>
int launch_gemv(const GemvArgs& g, const GemvCfg& c, int64_t grid, cudaStream_t st) {
  if (c.cg == 32) return launch_gemv_t<256, 16, 32, 2, kScale8, kSilu>(g, grid, c.smem, st);
  if (c.cg == 8) {
    if (c.stages == 4) return launch_gemv_t<256, 16, 8, 4, kScale8, kSilu>(g, grid, c.smem, st);
    if (c.stages == 3) return launch_gemv_t<256, 16, 8, 3, kScale8, kSilu>(g, grid, c.smem, st);
    return launch_gemv_t<256, 16, 8, 2, kScale8, kSilu>(g, grid, c.smem, st);
  }
  if (c.stages == 4) return launch_gemv_t<256, 16, 16, 4, kScale8, kSilu>(g, grid, c.smem, st);
  if (c.stages == 3) return launch_gemv_t<256, 16, 16, 3, kScale8, kSilu>(g, grid, c.smem, st);
  return launch_gemv_t<256, 16, 16, 2, kScale8, kSilu>(g, grid, c.smem, st);
}

bool vector_ok(int64_t N, int64_t K, int64_t G, const SparseWeights& w, const void* A, int64_t lda) {
  if (N % 16 != 0 || K % 16 != 0) return false;
  if (G != K / 16 && G != K / 8) return false;
  if (!pick_cfg(K, G == K / 8).ok) return false;
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

// Plan + (for bf16 activations) conversion to fp16 in one launch.
// conv_mode: what the extra blocks do with the activation matrix a_src (kConv*); kConvNone = nothing.
void launch_plan(const int32_t* ids, int64_t P, int64_t ids_topk, int64_t ids_ld, const int32_t* expert_map,
                 int64_t global_E, int64_t E, const Plan& plan, const void* a_src, __half* a_f16, int64_t a_rows,
                 int64_t a_cols, int64_t a_ld, cudaStream_t st, int* zero_buf = nullptr, int zero_count = 0,
                 int max_tok = kMaxTok, int conv_mode = kConvBf16) {
  int64_t chunks = 0;
  unsigned blocks = 1;
  if (a_src == nullptr) conv_mode = kConvNone;
  if (conv_mode != kConvNone) {
    chunks = a_rows * a_cols / 8;
    int64_t nb = (chunks + kPlanThreads - 1) / kPlanThreads;
    if (nb > 2 * (int64_t)sm_count()) nb = 2 * (int64_t)sm_count();
    blocks += (unsigned)(nb < 1 ? 1 : nb);
  }
  launch_pdl(moe_plan_kernel, dim3(blocks), dim3(kPlanThreads), 0, st, ids, (int)P, expert_map, (int)global_E, (int)E, plan,
             a_src, a_f16, chunks, (int)ids_topk, ids_ld, a_cols / 8 > 0 ? a_cols / 8 : (int64_t)1, a_ld / 8, zero_buf, zero_count,
             max_tok, conv_mode);
}

// Runs one projection for P pairs with a plan already in `plan`.  A is fp16.
GemvArgs make_args(const SparseWeights& w, const Plan& plan, const __half* A, int64_t lda, int a_div, void* out,
                   int out_dtype, int64_t ldo, int64_t N, int64_t K, int inter_silu) {
  GemvArgs g;
  g.w = w;
  g.plan = plan;
  g.A = A;
  g.lda = lda;
  g.a_div = a_div;
  g.a_magic = a_div > 1 ? (uint32_t)(((uint64_t)1 << 32) / (uint64_t)a_div) + 1u : 0u;
  g.out = out;
  g.ldo = ldo;
  g.out_dtype = out_dtype;
  g.N = (int)N;
  g.K = (int)K;
  g.inter = inter_silu;
  g.n_slabs = 1;
  g.wait_cycles = g_wait_cycles;
  return g;
}

// Both projections of the layer in one cooperative launch (tensor-core kernel).  Returns
// NOT_SUPPORTED when the shapes do not map to one of the instantiated pairs of configurations or the
// device cannot keep all blocks resident; the caller then launches the projections one by one.
template <int CGA, int SA, int CGB, int SB, int TM>
int launch_fused_pair(GemvArgs ga, GemvArgs gb, int* done, int64_t P, int64_t E, cudaStream_t st) {
  const void* fn = reinterpret_cast<const void*>(&fused_moe_mma_kernel<CGA, SA, CGB, SB, TM>);
  const size_t sa = mma_smem_bytes(ga.K, SA, TM), sb = mma_smem_bytes(gb.K, SB, TM);
  const size_t smem = sa > sb ? sa : sb;
  static int state[64] = {0};     // per device: 0 unknown, 1 usable, -1 not usable
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200FP4_STATUS_NOT_SUPPORTED;
  if (state[dev] == 0) {
    int coop = 0, per_sm = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    bool ok = coop != 0 && cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess &&
              cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kMmaThreads, 227 * 1024) == cudaSuccess && per_sm >= 1;
    if (!ok) cudaGetLastError();
    state[dev] = ok ? 1 : -1;
  }
  if (state[dev] < 0) return B200FP4_STATUS_NOT_SUPPORTED;
  ga.n_slabs = ga.inter / (64 * CGA);
  gb.n_slabs = gb.N / (128 * CGB);
  int need = ga.n_slabs + g_wait_extra_need;
  const int64_t slabs = ga.n_slabs > gb.n_slabs ? ga.n_slabs : gb.n_slabs;
  int64_t grid = max_passes(P, E) * slabs;
  if (grid > (int64_t)sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  void* args[4] = {&ga, &gb, &done, &need};
  if (cudaLaunchCooperativeKernel(fn, dim3((unsigned)grid), dim3(kMmaThreads), args, smem, st) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_NOT_SUPPORTED;
  }
  return B200FP4_STATUS_SUCCESS;
}

int run_projection(const SparseWeights& w, const Plan& plan, const __half* A, int64_t lda, int a_div, void* out,
                   int out_dtype, int64_t ldo, int64_t P, int64_t N, int64_t K, int64_t G, int64_t E, int inter_silu,
                   bool meta_ordered, cudaStream_t st, int tm = kMaxTok) {
  GemvArgs g = make_args(w, plan, A, lda, a_div, out, out_dtype, ldo, N, K, inter_silu);
  const bool s8 = (G == K / 8);
  if (meta_ordered) {
    // tensor-core kernel where the shape allows it (one scale per 16 k, whole 128-column groups)
    const MmaCfg mc = pick_mma_cfg(N, K, G, inter_silu, P < E ? P : E, tm);
    if (mc.ok) {
      g.n_slabs = inter_silu > 0 ? inter_silu / (64 * mc.cg) : (int)(N / (128 * mc.cg));
      int64_t grid = max_passes(P, E) * g.n_slabs;
      if (grid > (int64_t)sm_count()) grid = sm_count();
      if (grid < 1) grid = 1;
      return inter_silu > 0 ? launch_mma<true>(g, mc, grid, st) : launch_mma<false>(g, mc, grid, st);
    }
  }
  if (tm != kMaxTok) return B200FP4_STATUS_NOT_SUPPORTED;   // the general kernel only knows four-token passes
  const GemvCfg c = pick_cfg(K, s8);
  if (!c.ok) return B200FP4_STATUS_NOT_SUPPORTED;
  const int slab = c.cg * c.cols;
  g.n_slabs = inter_silu > 0 ? (inter_silu + slab / 2 - 1) / (slab / 2) : (int)((N + slab - 1) / slab);
  int64_t grid = max_passes(P, E) * g.n_slabs;
  if (grid > (int64_t)sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  if (inter_silu > 0) return s8 ? launch_gemv<true, true>(g, c, grid, st) : launch_gemv<false, true>(g, c, grid, st);
  return s8 ? launch_gemv<true, false>(g, c, grid, st) : launch_gemv<false, false>(g, c, grid, st);
}

int gemv_entry(const SparseWeights& w, int mode, const void* A, int a_dtype, const int32_t* expert_ids, void* out,
               int out_dtype, int64_t P, int64_t N, int64_t K, int64_t G, int64_t E, int flags, void* workspace,
               size_t ws_bytes, void* stream) {
  int rc = check_common(A, a_dtype, out, out_dtype, P, N, K, G, E);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (P == 0) return B200FP4_STATUS_SUCCESS;
  if (!w.comp || !w.scale || !w.g || !expert_ids || (mode == 0 && !w.meta)) return B200FP4_STATUS_INVALID_VALUE;
  cudaStream_t st = (cudaStream_t)stream;
  const int a_bf16 = a_dtype == B200FP4_DTYPE_BF16;
  if (mode == 0 && E <= kPlanMaxExperts && vector_ok(N, K, G, w, A, K)) {
    if (!workspace || ws_bytes < b200fp4_sparse_workspace_bytes(P, K, E) || !aligned(workspace, 16))
      return B200FP4_STATUS_ALLOC_FAILED;
    Plan plan = carve_plan(workspace, P, E);
    __half* a16 = reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(workspace) + align_up(plan_bytes(P, E), 256));
    if ((flags & B200FP4_SPARSE_META_ORDERED) != 0 && ws_ok(N, K, G, 0, w)) {
      // warp-scheduled tensor-core kernel: activations copied into fragment order, eight-token passes
      launch_plan(expert_ids, P, 1, 1, nullptr, 0, E, plan, A, a16, P, K, K, st, nullptr, 0, 8,
                  a_bf16 ? kConvBf16Frag : kConvF16Frag);
      zero_unmapped_rows_kernel<<<(unsigned)P, 128, 0, st>>>(plan.mapped, (int)P, out, out_dtype, N, (int)N);
      rc = run_projection_ws(w, plan, a16, K, 1, out, out_dtype, N, P, N, K, E, 0, plan.hdr + 2, st);
      if (rc != B200FP4_STATUS_SUCCESS) return rc;
      return finish_launch(3);
    }
    launch_plan(expert_ids, P, 1, 1, nullptr, 0, E, plan, a_bf16 ? A : nullptr, a16, P, K, K, st);
    zero_unmapped_rows_kernel<<<(unsigned)P, 128, 0, st>>>(plan.mapped, (int)P, out, out_dtype, N, (int)N);
    rc = run_projection(w, plan, a_bf16 ? a16 : reinterpret_cast<const __half*>(A), K, 1, out, out_dtype, N, P, N, K,
                        G, E, 0, (flags & B200FP4_SPARSE_META_ORDERED) != 0, st);
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

extern "C" size_t b200fp4_sparse_workspace_bytes(int64_t P, int64_t K, int64_t E) {
  if (P < 0 || E < 0 || K < 0) return 0;
  return align_up(plan_bytes(P, E), 256) + align_up((size_t)P * K * sizeof(__half), 256);
}

extern "C" int b200fp4_sparse_gemv(const void* A, int a_dtype, const uint8_t* B_comp_T, const uint8_t* Meta_T_pk,
                                   const uint8_t* scales_T, const float* g_scales, const int32_t* expert_ids, void* out,
                                   int out_dtype, int64_t P, int64_t N, int64_t K, int64_t G, int64_t E, int flags,
                                   void* workspace, size_t workspace_bytes, void* stream) {
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
  return gemv_entry(w, 0, A, a_dtype, expert_ids, out, out_dtype, P, N, K, G, E, flags, workspace, workspace_bytes, stream);
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant of b200fp4_sparse_gemv.
//
// Some hosts must not (or cannot) hand this library a workspace: plug-ins loaded into an inference
// server whose memory pool has already claimed nearly all device memory (a late cudaMalloc fails or
// fragments the pool), and latency-critical loops that ban allocator calls because cudaMalloc and
// cudaFree synchronise the whole device.  For them the scratch of the GEMV (the pair plan and the
// fp16 copy of bf16 activations) lives in a fixed array inside the library image instead.
//
// The array exists once per GPU that loads the library and stays resident until the process exits.
// All calls on a GPU share it: it still holds the previous call's plan when the next call starts
// (harmless -- the plan kernel rewrites every word the GEMV reads, so nothing has to be cleared), and
// two calls that overlap on the GPU (different streams, or different host threads) would overwrite
// each other's plan: serialise them.
constexpr int64_t kStaticMaxPairs = 512;
constexpr int64_t kStaticMaxK = 4096;
constexpr int64_t kStaticMaxExperts = 4096;
constexpr size_t static_align(size_t v, size_t a) { return (v + a - 1) / a * a; }
constexpr size_t kStaticPlanBytes =
    static_align(sizeof(int) * (size_t)(8 + 2 * kStaticMaxPairs), 16) +
    (size_t)(kStaticMaxPairs + kStaticMaxPairs / 4 + 1) * 2 * sizeof(int4);
constexpr size_t kStaticScratchBytes =
    static_align(kStaticPlanBytes, 256) + static_align((size_t)kStaticMaxPairs * kStaticMaxK * sizeof(__half), 256);

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device.  In host code the symbol's name is only
// a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
static int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return B200FP4_STATUS_NOT_INITIALIZED;
  }
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return B200FP4_STATUS_INTERNAL_ERROR;
    }
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return B200FP4_STATUS_SUCCESS;
}

extern "C" int b200fp4_sparse_gemv_static(const void* A, int a_dtype, const uint8_t* B_comp_T, const uint8_t* Meta_T_pk,
                                          const uint8_t* scales_T, const float* g_scales, const int32_t* expert_ids,
                                          void* out, int out_dtype, int64_t P, int64_t N, int64_t K, int64_t G, int64_t E,
                                          void* stream) {
  // sizes the fixed scratch cannot hold are refused before anything is enqueued
  if (P > kStaticMaxPairs || K > kStaticMaxK || E > kStaticMaxExperts) return B200FP4_STATUS_NOT_SUPPORTED;
  void* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  return b200fp4_sparse_gemv(A, a_dtype, B_comp_T, Meta_T_pk, scales_T, g_scales, expert_ids, out, out_dtype, P, N, K, G,
                             E, 0, scratch, kStaticScratchBytes, stream);
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
  return gemv_entry(w, 0, A, a_dtype, expert_ids, out, out_dtype, P, N, K, K / 8, E, 0, workspace, workspace_bytes, stream);
}

extern "C" void b200fp4_fused_moe_profile_events(void* before_gate_up, void* after_gate_up, void* after_down) {
  g_prof_events[0] = (cudaEvent_t)before_gate_up;
  g_prof_events[1] = (cudaEvent_t)after_gate_up;
  g_prof_events[2] = (cudaEvent_t)after_down;
}

extern "C" void b200fp4_fused_moe_set_wait_limit(int64_t cycles, int extra_need) {
  g_wait_cycles = cycles > 0 ? (long long)cycles : kDefaultWaitCycles;
  g_wait_extra_need = extra_need > 0 ? extra_need : 0;
}

extern "C" int b200fp4_fused_moe_last_status(const void* workspace, void* stream, int* status) {
  if (!workspace || !status) return B200FP4_STATUS_INVALID_VALUE;
  cudaStream_t st = (cudaStream_t)stream;
  // the status word is hdr[3] of the plan at the start of the layer's workspace
  if (cudaMemcpyAsync(status, reinterpret_cast<const int*>(workspace) + 3, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  return B200FP4_STATUS_SUCCESS;
}

extern "C" size_t b200fp4_fused_moe_workspace_bytes(int64_t M, int64_t topk, int64_t H, int64_t I, int64_t E) {
  if (M < 0 || topk <= 0 || H <= 0 || I <= 0 || E <= 0) return 0;
  const int64_t P = M * topk;
  return align_up(plan_bytes(P, E), 256) + align_up((size_t)M * H * sizeof(__half), 256) +
         align_up((size_t)P * I * sizeof(__half), 256) + align_up((size_t)P * H * sizeof(float), 256) +
         align_up((size_t)max_passes(P, E) * sizeof(int), 256);
}

// ld_h / ld_w / ld_ids: row strides (in elements) of hidden, topk_weights and topk_ids.
static int fused_moe_impl(const void* hidden, int64_t ld_h, int h_dtype, const float* topk_weights, int64_t ld_w,
                          const int32_t* topk_ids, int64_t ld_ids, const int32_t* expert_map, int64_t global_E,
                          const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale, const float* w13_g,
                          int64_t G13, const uint8_t* w2_comp, const uint8_t* w2_meta, const uint8_t* w2_scale,
                          const float* w2_g, int64_t G2, void* out, int out_dtype, int64_t M, int64_t topk, int64_t H,
                          int64_t I, int64_t E, int flags, void* workspace, size_t workspace_bytes, void* stream,
                          OutScatter sc = OutScatter{nullptr, 1, 0}) {
  if (M < 0 || topk <= 0 || H <= 0 || I <= 0 || E <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (ld_h < H || ld_w < topk || ld_ids < topk || (ld_h % 8) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (sc.ptrs != nullptr && (sc.rows_per_dest <= 0 || sc.dest_row0 < 0)) return B200FP4_STATUS_INVALID_VALUE;
  if (sc.ptrs != nullptr && !out) out = workspace;      // the checks below want a non-null result pointer; it is not written
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
  if (E > kPlanMaxExperts) return B200FP4_STATUS_NOT_SUPPORTED;
  SparseWeights w13, w2;
  w13.comp = w13_comp; w13.meta = w13_meta; w13.scale = w13_scale; w13.g = w13_g;
  w13.comp_e = (H / 4) * 2 * I; w13.comp_pair = 4 * I; w13.comp_odd = 2 * I;
  w13.meta_e = (H / 8) * 2 * I; w13.meta_row = 2 * I; w13.scale_e = G13 * 2 * I; w13.scale_row = 2 * I;
  w2.comp = w2_comp; w2.meta = w2_meta; w2.scale = w2_scale; w2.g = w2_g;
  w2.comp_e = (I / 4) * H; w2.comp_pair = 2 * H; w2.comp_odd = H;
  w2.meta_e = (I / 8) * H; w2.meta_row = H; w2.scale_e = G2 * H; w2.scale_row = H;
  // the fused layer only exists in vectorised form
  if (I % 16 != 0 || !vector_ok(2 * I, H, G13, w13, hidden, ld_h) || !vector_ok(H, I, G2, w2, hidden, I))
    return B200FP4_STATUS_NOT_SUPPORTED;
  if (!workspace || !aligned(workspace, 256) || workspace_bytes < b200fp4_fused_moe_workspace_bytes(M, topk, H, I, E))
    return B200FP4_STATUS_ALLOC_FAILED;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  Plan plan = carve_plan(ws, P, E);
  sc.status_src = plan.hdr + 3;
  size_t off = align_up(plan_bytes(P, E), 256);
  __half* h16 = reinterpret_cast<__half*>(ws + off);
  off += align_up((size_t)M * H * sizeof(__half), 256);
  __half* act = reinterpret_cast<__half*>(ws + off);
  off += align_up((size_t)P * I * sizeof(__half), 256);
  float* down = reinterpret_cast<float*>(ws + off);
  const bool bf = h_dtype == B200FP4_DTYPE_BF16;
  const bool ordered = (flags & B200FP4_SPARSE_META_ORDERED) != 0;
  off += align_up((size_t)P * H * sizeof(float), 256);
  int* done = reinterpret_cast<int*>(ws + off);
  const int64_t n_done = max_passes(P, E);

  // More than 256 pairs: the warp-scheduled tensor-core kernel (passes of eight tokens, activations in fragment order
  // from the plan kernel and from the gate_up epilogue).  Both projections share one launch and one claim sequence
  // unless B200FP4_MOE_SEPARATE_LAUNCHES asks for one launch each.
  if (ordered && P > 256 && ws_ok(2 * I, H, G13, I, w13) && ws_ok(H, I, G2, 0, w2)) {
    launch_plan(topk_ids, P, topk, ld_ids, expert_map, global_E, E, plan, hidden, h16, M, H, ld_h, st, done, (int)n_done, 8,
                bf ? kConvBf16Frag : kConvF16Frag);
    if (g_prof_events[0]) cudaEventRecord(g_prof_events[0], st);
    if (!(flags & B200FP4_MOE_SEPARATE_LAUNCHES)) {
      GemvArgs ga = make_args(w13, plan, h16, H, (int)topk, act, B200FP4_DTYPE_F16, I, 2 * I, H, (int)I);
      GemvArgs gb = make_args(w2, plan, act, I, 1, down, B200FP4_DTYPE_F32, H, H, I, 0);
      ga.n_slabs = (int)(I / 64);
      gb.n_slabs = (int)(H / 128);
      const int need = ga.n_slabs + g_wait_extra_need;
      const int64_t items = max_passes(P, E) * (ga.n_slabs + gb.n_slabs);
      // Block shape: 8 warps with 8-stage rings where K allows (both K multiples of 256), else 16 warps x 4 stages.
      // Measured on B200 (layer step / fraction of the copy bandwidth of the launch, batch 32, 512 experts):
      // 8 x 8: 72.4 us / 0.745; 7 x 8: 73.5 / 0.73; 8 warps x 4 stages: 73.7 / 0.72; 16 x 4: 76.0 / 0.705; 6 x 8: 78.2; 12 x 4:
      // 79.6; 9, 10, 12 warps x 8: 79-82; 6 or 5 warps x 16 stages: 78.5 / 82.5; 4 x 8: 87.4; 24 x 4: 93.7.  With the 64
      // local experts of one of eight expert-parallel ranks: 16 x 4 49.7 us for the launch, 8 x 8 37.6 us, 4 x 16 44.7 us.
      const bool deep = H % 256 == 0 && I % 256 == 0;
      if (2 * I == 1024 && H == 2048) {
        rc = deep ? launch_fused_ws_t<1024, 2048, 8, 8>(ga, gb, plan.hdr + 2, done, need, items, st)
                  : launch_fused_ws_t<1024, 2048>(ga, gb, plan.hdr + 2, done, need, items, st);
      } else {
        rc = deep ? launch_fused_ws_t<0, 0, 8, 8>(ga, gb, plan.hdr + 2, done, need, items, st)
                  : launch_fused_ws_t<0, 0>(ga, gb, plan.hdr + 2, done, need, items, st);
      }
      if (rc != B200FP4_STATUS_SUCCESS) return rc;
      if (g_prof_events[1]) cudaEventRecord(g_prof_events[1], st);
    } else {
      rc = run_projection_ws(w13, plan, h16, H, (int)topk, act, B200FP4_DTYPE_F16, I, P, 2 * I, H, E, (int)I, plan.hdr + 2, st);
      if (rc != B200FP4_STATUS_SUCCESS) return rc;
      if (g_prof_events[1]) cudaEventRecord(g_prof_events[1], st);
      rc = run_projection_ws(w2, plan, act, I, 1, down, B200FP4_DTYPE_F32, H, P, H, I, E, 0, plan.hdr + 4, st);
      if (rc != B200FP4_STATUS_SUCCESS) return rc;
    }
    if (g_prof_events[2]) cudaEventRecord(g_prof_events[2], st);
    launch_pdl(weighted_reduce_kernel, reduce_grid(H, M), dim3(kRedThreads), 0, st, (const float*)down, topk_weights, (const int*)plan.mapped,
               out, out_dtype, (int)M, (int)topk, (int)H, (flags & B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT) ? 1 : 0, ld_w, sc);
    return finish_launch((flags & B200FP4_MOE_SEPARATE_LAUNCHES) ? 4 : 3);
  }

  // Tokens per pass: eight when the local experts see four or more tokens each on average (large
  // batches, expert parallelism with many source ranks) and both projections have a tensor-core
  // configuration for it; four otherwise.
  const int64_t pb = P < E ? P : E;
  const int64_t local_pairs = (expert_map && global_E > 0) ? P * E / global_E : P;
  int tm = kMaxTok;
  if (ordered && local_pairs >= 4 * E) {
    const MmaCfg a8 = pick_mma_cfg(2 * I, H, G13, (int)I, pb, 8), b8 = pick_mma_cfg(H, I, G2, 0, pb, 8);
    if (a8.ok && b8.ok) tm = 8;
  }
  launch_plan(topk_ids, P, topk, ld_ids, expert_map, global_E, E, plan, bf ? hidden : nullptr, h16, M, H, ld_h, st, done,
              (int)n_done, tm);
  if (g_prof_events[0]) cudaEventRecord(g_prof_events[0], st);
  // One cooperative launch for both projections pays for small batches (measured on B200: 24.6 vs 27.2 us
  // per layer at 10 pairs, 67.7 vs 68.2 us at 160); from 320 pairs on two launches are faster (100.6 vs
  // 102.3 us, 185.6 vs 193.8 us at 1280 pairs), so it is used up to 256 pairs.
  if (ordered && !(flags & B200FP4_MOE_SEPARATE_LAUNCHES) && P <= 256) {
    const MmaCfg ca = pick_mma_cfg(2 * I, H, G13, (int)I, pb, tm), cb = pick_mma_cfg(H, I, G2, 0, pb, tm);
    if (ca.ok && cb.ok) {
      const GemvArgs ga = make_args(w13, plan, bf ? h16 : reinterpret_cast<const __half*>(hidden), bf ? H : ld_h, (int)topk,
                                    act, B200FP4_DTYPE_F16, I, 2 * I, H, (int)I);
      const GemvArgs gb = make_args(w2, plan, act, I, 1, down, B200FP4_DTYPE_F32, H, H, I, 0);
      int frc = B200FP4_STATUS_NOT_SUPPORTED;
      if (tm == 4 && ca.stages == 5 && cb.stages == 5) {
        if (ca.cg == 2 && cb.cg == 4) frc = launch_fused_pair<2, 5, 4, 5, 4>(ga, gb, done, P, E, st);
        else if (ca.cg == 1 && cb.cg == 2) frc = launch_fused_pair<1, 5, 2, 5, 4>(ga, gb, done, P, E, st);
      } else if (tm == 8 && ca.stages == 3 && cb.stages == 5) {
        if (ca.cg == 2 && cb.cg == 4) frc = launch_fused_pair<2, 3, 4, 5, 8>(ga, gb, done, P, E, st);
        else if (ca.cg == 1 && cb.cg == 2) frc = launch_fused_pair<1, 3, 2, 5, 8>(ga, gb, done, P, E, st);
      }
      if (frc == B200FP4_STATUS_SUCCESS) {
        if (g_prof_events[1]) cudaEventRecord(g_prof_events[1], st);
        if (g_prof_events[2]) cudaEventRecord(g_prof_events[2], st);
        weighted_reduce_kernel<<<reduce_grid(H, M), kRedThreads, 0, st>>>(down, topk_weights, plan.mapped, out, out_dtype, (int)M, (int)topk,
                                                      (int)H, (flags & B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT) ? 1 : 0, ld_w, sc);
        return finish_launch(3);
      }
    }
  }
  rc = run_projection(w13, plan, bf ? h16 : reinterpret_cast<const __half*>(hidden), bf ? H : ld_h, (int)topk, act,
                      B200FP4_DTYPE_F16, I, P, 2 * I, H, G13, E, (int)I, ordered, st, tm);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (g_prof_events[1]) cudaEventRecord(g_prof_events[1], st);
  rc = run_projection(w2, plan, act, I, 1, down, B200FP4_DTYPE_F32, H, P, H, I, G2, E, 0, ordered, st, tm);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (g_prof_events[2]) cudaEventRecord(g_prof_events[2], st);
  launch_pdl(weighted_reduce_kernel, reduce_grid(H, M), dim3(kRedThreads), 0, st, (const float*)down, topk_weights, (const int*)plan.mapped, out,
             out_dtype, (int)M, (int)topk, (int)H, (flags & B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT) ? 1 : 0, ld_w, sc);
  return finish_launch(4);
}

extern "C" int b200fp4_fused_sparse_moe(const void* hidden, int h_dtype, const float* topk_weights,
                                        const int32_t* topk_ids, const int32_t* expert_map, int64_t global_E,
                                        const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale,
                                        const float* w13_g, int64_t G13, const uint8_t* w2_comp, const uint8_t* w2_meta,
                                        const uint8_t* w2_scale, const float* w2_g, int64_t G2, void* out, int out_dtype,
                                        int64_t M, int64_t topk, int64_t H, int64_t I, int64_t E, int flags,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  return fused_moe_impl(hidden, H, h_dtype, topk_weights, topk, topk_ids, topk, expert_map, global_E, w13_comp, w13_meta,
                        w13_scale, w13_g, G13, w2_comp, w2_meta, w2_scale, w2_g, G2, out, out_dtype, M, topk, H, I, E, flags,
                        workspace, workspace_bytes, stream);
}

// The layer for a caller whose activations, routing and result live in HOST memory (pinned memory makes the
// copies asynchronous): three copies in, the device entry point above, one copy out, one stream
// synchronisation.  The device workspace holds the staging buffers in front of the layer's own workspace.
static size_t host_stage_bytes(int64_t M, int64_t topk, int64_t H) {
  return 2 * align_up((size_t)M * H * sizeof(__half), 256) + 2 * align_up((size_t)M * topk * sizeof(float), 256);
}

extern "C" size_t b200fp4_fused_moe_host_workspace_bytes(int64_t M, int64_t topk, int64_t H, int64_t I, int64_t E) {
  if (M < 0 || topk <= 0 || H <= 0 || I <= 0 || E <= 0) return 0;
  return host_stage_bytes(M, topk, H) + b200fp4_fused_moe_workspace_bytes(M, topk, H, I, E);
}

namespace {
// Events that order a copy stream against the compute stream, one pair per workspace (the staging buffers they guard
// live in the workspace).  Created on first use, kept for the life of the process.
struct HostSlotEvents {
  const void* workspace;
  int device;
  cudaEvent_t loaded, consumed;
  bool used;
};
constexpr int kHostSlots = 32;
HostSlotEvents g_host_slots[kHostSlots];
int g_host_slot_count = 0;
std::mutex g_host_slot_mutex;

HostSlotEvents* host_slot_events(const void* workspace) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(g_host_slot_mutex);
  for (int i = 0; i < g_host_slot_count; ++i)
    if (g_host_slots[i].workspace == workspace && g_host_slots[i].device == dev) return &g_host_slots[i];
  if (g_host_slot_count == kHostSlots) return nullptr;
  HostSlotEvents& e = g_host_slots[g_host_slot_count];
  if (cudaEventCreateWithFlags(&e.loaded, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  if (cudaEventCreateWithFlags(&e.consumed, cudaEventDisableTiming) != cudaSuccess) {
    cudaEventDestroy(e.loaded);
    return nullptr;
  }
  e.workspace = workspace;
  e.device = dev;
  e.used = false;
  ++g_host_slot_count;
  return &e;
}
}  // namespace

// Enqueue-only form: copies in (on copy_stream when one is given, ordered against the layer by events), the layer, the
// copies out; no host synchronisation.
extern "C" int b200fp4_fused_sparse_moe_host_async(const void* hidden_host, int h_dtype, const float* topk_weights_host,
                                                   const int32_t* topk_ids_host, const int32_t* expert_map,
                                                   int64_t global_E, const uint8_t* w13_comp, const uint8_t* w13_meta,
                                                   const uint8_t* w13_scale, const float* w13_g, int64_t G13,
                                                   const uint8_t* w2_comp, const uint8_t* w2_meta, const uint8_t* w2_scale,
                                                   const float* w2_g, int64_t G2, void* out_host, int out_dtype,
                                                   int32_t* status_host, int64_t M, int64_t topk, int64_t H, int64_t I,
                                                   int64_t E, int flags, void* workspace, size_t workspace_bytes,
                                                   void* stream, void* copy_stream) {
  if (M < 0 || topk <= 0 || H <= 0 || I <= 0 || E <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!hidden_host || !topk_weights_host || !topk_ids_host || !out_host || !workspace)
    return B200FP4_STATUS_INVALID_VALUE;
  if (out_dtype != B200FP4_DTYPE_F16 && out_dtype != B200FP4_DTYPE_BF16) return B200FP4_STATUS_NOT_SUPPORTED;
  const size_t stage = host_stage_bytes(M, topk, H);
  if (workspace_bytes < stage) return B200FP4_STATUS_INVALID_VALUE;
  const size_t nh = (size_t)M * H * sizeof(__half), nr = (size_t)M * topk * sizeof(float);
  char* d_hidden = static_cast<char*>(workspace);
  char* d_out = d_hidden + align_up(nh, 256);
  char* d_w = d_out + align_up(nh, 256);
  char* d_ids = d_w + align_up(nr, 256);
  cudaStream_t st = (cudaStream_t)stream;
  cudaStream_t cs = copy_stream ? (cudaStream_t)copy_stream : st;
  HostSlotEvents* ev = nullptr;
  if (cs != st) {
    ev = host_slot_events(workspace);
    if (!ev) return B200FP4_STATUS_ALLOC_FAILED;
    // the staging buffers may still be read by the layer of the previous submission with this workspace
    if (ev->used && cudaStreamWaitEvent(cs, ev->consumed, 0) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
  }
  if (cudaMemcpyAsync(d_ids, topk_ids_host, nr, cudaMemcpyHostToDevice, cs) != cudaSuccess ||
      cudaMemcpyAsync(d_w, topk_weights_host, nr, cudaMemcpyHostToDevice, cs) != cudaSuccess ||
      cudaMemcpyAsync(d_hidden, hidden_host, nh, cudaMemcpyHostToDevice, cs) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  if (ev && (cudaEventRecord(ev->loaded, cs) != cudaSuccess || cudaStreamWaitEvent(st, ev->loaded, 0) != cudaSuccess)) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  // result rows and status word: into the staging buffer and copied out, or -- with B200FP4_MOE_HOST_DIRECT_OUT and
  // pinned memory the device can address -- stored by the layer's last kernel straight into the caller's buffers
  auto mapped_of = [](void* host) -> void* {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
  };
  void* out_target = d_out;
  OutScatter sc{nullptr, 1, 0};
  if (flags & B200FP4_MOE_HOST_DIRECT_OUT) {
    if (void* mapped = mapped_of(out_host)) out_target = mapped;
    if (status_host) sc.status_out = static_cast<int*>(mapped_of(status_host));
  }
  const int rc = fused_moe_impl(d_hidden, H, h_dtype, reinterpret_cast<const float*>(d_w), topk,
                                reinterpret_cast<const int32_t*>(d_ids), topk, expert_map, global_E, w13_comp, w13_meta,
                                w13_scale, w13_g, G13, w2_comp, w2_meta, w2_scale, w2_g, G2, out_target, out_dtype, M, topk, H,
                                I, E, flags & ~B200FP4_MOE_HOST_DIRECT_OUT, static_cast<char*>(workspace) + stage,
                                workspace_bytes - stage, stream, sc);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (ev) {
    if (cudaEventRecord(ev->consumed, st) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    ev->used = true;
  }
  // the layer's status word (hdr[3] of its plan) comes back with the result
  if ((out_target == d_out && cudaMemcpyAsync(out_host, d_out, nh, cudaMemcpyDeviceToHost, st) != cudaSuccess) ||
      (status_host && !sc.status_out && cudaMemcpyAsync(status_host, reinterpret_cast<const int*>(static_cast<char*>(workspace) + stage) + 3,
                                      sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess)) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  return B200FP4_STATUS_SUCCESS;
}

extern "C" int b200fp4_fused_sparse_moe_host(const void* hidden_host, int h_dtype, const float* topk_weights_host,
                                             const int32_t* topk_ids_host, const int32_t* expert_map, int64_t global_E,
                                             const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale,
                                             const float* w13_g, int64_t G13, const uint8_t* w2_comp,
                                             const uint8_t* w2_meta, const uint8_t* w2_scale, const float* w2_g,
                                             int64_t G2, void* out_host, int out_dtype, int64_t M, int64_t topk,
                                             int64_t H, int64_t I, int64_t E, int flags, void* workspace,
                                             size_t workspace_bytes, void* stream) {
  if (M == 0 && topk > 0 && H > 0 && I > 0 && E > 0) return B200FP4_STATUS_SUCCESS;
  int moe_status = 0;
  const int rc = b200fp4_fused_sparse_moe_host_async(hidden_host, h_dtype, topk_weights_host, topk_ids_host, expert_map,
                                                     global_E, w13_comp, w13_meta, w13_scale, w13_g, G13, w2_comp, w2_meta,
                                                     w2_scale, w2_g, G2, out_host, out_dtype, &moe_status, M, topk, H, I, E,
                                                     flags, workspace, workspace_bytes, stream, nullptr);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  return moe_status == 0 ? B200FP4_STATUS_SUCCESS : B200FP4_STATUS_INTERNAL_ERROR;
}

// ------------------------------------------------------------------------------------------ expert parallel

// One record per token: [H activations (16-bit) | topk expert ids (i32) | topk router weights (f32)].
extern "C" size_t b200fp4_ep_record_bytes(int64_t H, int64_t topk) {
  if (H <= 0 || topk <= 0) return 0;
  return align_up((size_t)H * 2 + (size_t)topk * 8, 16);
}

namespace b200fp4 {
namespace {
// out[g][b] = record of token b, for every destination rank g (fixed-capacity dispatch slots)
__global__ void ep_pack_kernel(const uint4* __restrict__ hidden, const int32_t* __restrict__ ids,
                               const float* __restrict__ w, int B, int H, int topk, int G, int64_t rec_chunks,
                               uint4* __restrict__ out) {
  const int b = blockIdx.x;
  const int h_chunks = H / 8;
  __shared__ uint4 s_tail[64];
  const int tail_chunks = (int)rec_chunks - h_chunks;
  if (threadIdx.x < tail_chunks * 4) {
    const int i = threadIdx.x;            // 32-bit word index inside the tail: ids first, then weights
    uint32_t v = 0;
    if (i < topk) v = (uint32_t)ids[(int64_t)b * topk + i];
    else if (i < 2 * topk) v = __float_as_uint(w[(int64_t)b * topk + i - topk]);
    reinterpret_cast<uint32_t*>(s_tail)[i] = v;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < rec_chunks; c += blockDim.x) {
    const uint4 v = c < h_chunks ? hidden[(int64_t)b * h_chunks + c] : s_tail[c - h_chunks];
    for (int g = 0; g < G; ++g) out[((int64_t)g * B + b) * rec_chunks + c] = v;
  }
}

// out[b, :] = sum over ranks g of parts[g][b, :] accumulated in fp32
template <typename T>
__global__ void ep_combine_kernel(const T* __restrict__ parts, int B, int H, int G, T* __restrict__ out) {
  const int64_t n = (int64_t)B * H;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2; i < n; i += (int64_t)gridDim.x * blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int g = 0; g < G; ++g) {
      a0 += to_f32<T>(parts[(int64_t)g * n + i]);
      a1 += to_f32<T>(parts[(int64_t)g * n + i + 1]);
    }
    out[i] = from_f32<T>(a0);
    out[i + 1] = from_f32<T>(a1);
  }
}
}  // namespace
}  // namespace b200fp4

extern "C" int b200fp4_ep_pack(const void* hidden, const int32_t* topk_ids, const float* topk_weights, int64_t B,
                               int64_t H, int64_t topk, int64_t G, void* records, void* stream) {
  if (B < 0 || H <= 0 || (H % 8) != 0 || topk <= 0 || topk > 64 || G <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (B == 0) return B200FP4_STATUS_SUCCESS;
  if (!hidden || !topk_ids || !topk_weights || !records || !aligned(hidden, 16) || !aligned(records, 16))
    return B200FP4_STATUS_INVALID_VALUE;
  const int64_t rec_chunks = (int64_t)b200fp4_ep_record_bytes(H, topk) / 16;
  ep_pack_kernel<<<(unsigned)B, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint4*>(hidden), topk_ids,
                                                               topk_weights, (int)B, (int)H, (int)topk, (int)G,
                                                               rec_chunks, reinterpret_cast<uint4*>(records));
  return finish_launch(1);
}

extern "C" int b200fp4_ep_combine(const void* parts, int dtype, int64_t B, int64_t H, int64_t G, void* out, void* stream) {
  if (B < 0 || H <= 0 || (H % 2) != 0 || G <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (dtype != B200FP4_DTYPE_BF16 && dtype != B200FP4_DTYPE_F16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (B == 0) return B200FP4_STATUS_SUCCESS;
  if (!parts || !out) return B200FP4_STATUS_INVALID_VALUE;
  int64_t blocks = (B * H / 2 + 255) / 256;
  if (blocks > 4 * (int64_t)sm_count()) blocks = 4 * (int64_t)sm_count();
  if (dtype == B200FP4_DTYPE_BF16)
    ep_combine_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(parts), (int)B, (int)H, (int)G, reinterpret_cast<__nv_bfloat16*>(out));
  else
    ep_combine_kernel<__half><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __half*>(parts), (int)B, (int)H, (int)G, reinterpret_cast<__half*>(out));
  return finish_launch(1);
}

// The fused layer over received dispatch records ([T] records of record_bytes each, as written by
// b200fp4_ep_pack on the source ranks): activations, ids and weights are read in place.
extern "C" int b200fp4_fused_sparse_moe_records(const void* records, int64_t record_bytes, int h_dtype,
                                                const int32_t* expert_map, int64_t global_E, const uint8_t* w13_comp,
                                                const uint8_t* w13_meta, const uint8_t* w13_scale, const float* w13_g,
                                                int64_t G13, const uint8_t* w2_comp, const uint8_t* w2_meta,
                                                const uint8_t* w2_scale, const float* w2_g, int64_t G2, void* out,
                                                int out_dtype, int64_t T, int64_t topk, int64_t H, int64_t I, int64_t E,
                                                int flags, void* workspace, size_t workspace_bytes, void* stream) {
  if (!records || record_bytes != (int64_t)b200fp4_ep_record_bytes(H, topk)) return B200FP4_STATUS_INVALID_VALUE;
  const unsigned char* r = reinterpret_cast<const unsigned char*>(records);
  return fused_moe_impl(r, record_bytes / 2, h_dtype, reinterpret_cast<const float*>(r + H * 2 + topk * 4),
                        record_bytes / 4, reinterpret_cast<const int32_t*>(r + H * 2), record_bytes / 4, expert_map,
                        global_E, w13_comp, w13_meta, w13_scale, w13_g, G13, w2_comp, w2_meta, w2_scale, w2_g, G2, out,
                        out_dtype, T, topk, H, I, E, flags & ~B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT, workspace, workspace_bytes,
                        stream);
}

// The same with the result scattered over several buffers: row m (token m of the T received records) goes to row
// dest_row0 + m % rows_per_dest of the buffer out_ptrs[m / rows_per_dest].  out_ptrs is a DEVICE array of T /
// rows_per_dest pointers, which may point into peer GPUs' memory (plain stores over NVLink).
extern "C" int b200fp4_fused_sparse_moe_records_scatter(
    const void* records, int64_t record_bytes, int h_dtype, const int32_t* expert_map, int64_t global_E,
    const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale, const float* w13_g, int64_t G13,
    const uint8_t* w2_comp, const uint8_t* w2_meta, const uint8_t* w2_scale, const float* w2_g, int64_t G2,
    void* const* out_ptrs, int64_t rows_per_dest, int64_t dest_row0, int out_dtype, int64_t T, int64_t topk, int64_t H, int64_t I,
    int64_t E, int flags, void* workspace, size_t workspace_bytes, void* stream) {
  if (!records || record_bytes != (int64_t)b200fp4_ep_record_bytes(H, topk) || !out_ptrs) return B200FP4_STATUS_INVALID_VALUE;
  if (rows_per_dest <= 0 || rows_per_dest > 0x7FFFFFFF || dest_row0 < 0 || dest_row0 > 0x7FFFFFFF) return B200FP4_STATUS_INVALID_VALUE;
  const unsigned char* r = reinterpret_cast<const unsigned char*>(records);
  OutScatter sc{out_ptrs, (int)rows_per_dest, (int)dest_row0};
  return fused_moe_impl(r, record_bytes / 2, h_dtype, reinterpret_cast<const float*>(r + H * 2 + topk * 4), record_bytes / 4,
                        reinterpret_cast<const int32_t*>(r + H * 2), record_bytes / 4, expert_map, global_E, w13_comp, w13_meta,
                        w13_scale, w13_g, G13, w2_comp, w2_meta, w2_scale, w2_g, G2, nullptr, out_dtype, T, topk, H, I, E,
                        flags & ~B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT, workspace, workspace_bytes, stream, sc);
}
