// Dense block-scaled NVFP4 GEMM for sm_100a: out[M,N] = alpha * (A . sfA)(B . sfB)^T
//
// Replaces the GEMM behind cuda_fp4_gemm.h / cutlass_scaled_fp4_mm in the reference (whose own
// kernels are scalar CUDA-core loops, cutlass_nvfp4/nvfp4_gemm_kernel.cuh:296-345) with a
// tcgen05 design:
//   * persistent, warp-specialised CTAs (one per SM): warp 0 issues TMA loads, warp 1 issues
//     tcgen05.cp / tcgen05.mma, warps 2-5 run the epilogue;
//   * operands are packed E2M1 bytes, K-major, staged by 2-D TMA (no multicast) into 128-byte
//     swizzled shared-memory tiles of 128 (A) / BN (B) rows x 256 k; scale factors come from the
//     128x4-tile swizzled global layout, where the 4 k-blocks x 128 rows an MMA needs are 512
//     contiguous bytes: one bulk copy per stage brings them to shared memory and four dedicated
//     warps (one per 32-lane quarter of tensor memory) move them on with tcgen05.st, which keeps
//     them off the tensor pipe (a tcgen05.cp per scale tile measured ~36 cycles there, a quarter
//     of an MMA);
//   * tcgen05.mma.kind::mxf4nvf4.block_scale (M=128, N=BN, K=64) accumulates fp32 in tensor
//     memory; the epilogue reads it with tcgen05.ld, multiplies by alpha and writes bf16/f16;
//   * BN=128 double-buffers the accumulator (epilogue of tile i overlaps the main loop of tile
//     i+1); BN=256 keeps one accumulator but drains it into packed registers and releases it before
//     the global stores, so only the ~1200-cycle drain is exposed; it moves 25 % fewer bytes per flop.
// Every mbarrier wait is bounded: on expiry the kernel records an error code in the status word
// and all roles drain out, so a protocol error cannot hang the GPU.
#include <cstring>
#include <mutex>
#include <type_traits>

#include "sm100_ptx.cuh"

namespace b200fp4 {

// CTA-pair (cta_group::2) kernel, gemm_pair.cu
int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                     void* out, int out_bf16, int M, int N, int K, int* status, cudaStream_t st);

namespace {

constexpr int kBM = 128;
constexpr int kGemmThreads = 448;         // warp 0 TMA, warp 1 MMA, warps 2-5 and 10-13 epilogue, warps 6-9 scale factors
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
  const uint8_t* sfa;   // swizzled [ceil(M/128)*128, ceil(K/64)*4]
  const uint8_t* sfb;   // swizzled [ceil(N/128)*128, ceil(K/64)*4]
  const float* alpha;
  void* out;
  int out_bf16;
  int out_f32;          // dense mode only: out is fp32 [M, N] (the accumulator times alpha, unrounded)
  int out_tma;          // dense 16-bit output through map_out: the epilogue stages tiles in shared memory and the copy
                        // engine writes whole lines (256-wide tiles only)
  int M, N, K;
  int m_tiles, n_tiles, k_stages;
  int* status;          // 0 = ok; otherwise the code of the wait that expired
  // grouped (per-expert) mode: rows of A/out are permuted by expert, B is [E, N, K/2]
  const int* g_hdr;       // [0] = number of 128-row tiles over all experts
  const int4* g_mtiles;   // per 128-row tile: {first row, end row of its expert, scale-tile row of A, expert}
  const float* g_alphas;  // [E]
  long long g_sfb_expert_bytes;
  // fused SiLU(gate)*up + NVFP4 quantization of the result (grouped gate_up projection, N = 2*q_inter):
  // `out` receives packed codes [rows, q_inter/2], q_sf the swizzled block scales, q_gs[E] the global scales
  int q_inter;
  uint8_t* q_sf;
  const float* q_gs;
};

// What the roles need to know about one output tile.
struct TileInfo {
  int a_row0;       // first row of A / out
  int row_end;      // rows >= row_end are not stored
  int sfa_tile;     // index of the 128-row scale tile of A
  int b_row0;       // first row of the (flattened) B matrix
  int sfb_tile0;    // index of the first 128-row scale tile of B inside its expert
  int sfb_tile1;    // ... of the second one (256-wide tiles)
  int b_row1;       // fused SiLU tiles: first row of the "up" half of B (the gate half starts at b_row0)
  int expert;       // -1 in dense mode
  int n0;           // first output column
};

template <int BN, bool kGrouped, bool kSiluQuant = false>
__device__ __forceinline__ TileInfo tile_info(const GemmParams& p, int tile, int m_tiles) {
  TileInfo t;
  const int mt = tile % m_tiles, nt = tile / m_tiles;
  if (kSiluQuant) {
    // tile nt pairs gate columns [128 nt, +128) with up columns q_inter + [128 nt, +128); n0 counts output columns
    const int4 r = p.g_mtiles[mt];
    t.n0 = nt * 128;
    t.sfb_tile0 = nt;
    t.sfb_tile1 = p.q_inter / 128 + nt;
    t.a_row0 = r.x;
    t.row_end = r.y;
    t.sfa_tile = r.z;
    t.expert = r.w;
    t.b_row0 = r.w * p.N + nt * 128;
    t.b_row1 = t.b_row0 + p.q_inter;
    return t;
  }
  t.n0 = nt * BN;
  t.sfb_tile0 = nt * (BN / 128);
  t.sfb_tile1 = t.sfb_tile0 + 1;
  t.b_row1 = 0;
  if (kGrouped) {
    const int4 r = p.g_mtiles[mt];
    t.a_row0 = r.x;
    t.row_end = r.y;
    t.sfa_tile = r.z;
    t.expert = r.w;
    t.b_row0 = r.w * p.N + nt * BN;
  } else {
    t.a_row0 = mt * kBM;
    t.row_end = p.M;
    t.sfa_tile = mt;
    t.expert = -1;
    t.b_row0 = nt * BN;
  }
  return t;
}

// 64 gate and 64 up values of one row (as 16-bit pairs) -> SiLU(gate)*up rounded to T -> four NVFP4 blocks:
// 8 words of codes and 4 scale bytes, with the arithmetic of the stand-alone SiLU-mul quantizer.
template <typename T>
__device__ __forceinline__ void silu_quant_row(const uint32_t* pg, const uint32_t* pu, float gs, float rcp_gs,
                                               uint32_t* codes, uint32_t& sf4) {
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    float x[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t wg = pg[b * 8 + i], wu = pu[b * 8 + i];
      float g0, g1, u0, u1;
      if (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
        g0 = __uint_as_float(wg << 16); g1 = __uint_as_float(wg & 0xFFFF0000u);
        u0 = __uint_as_float(wu << 16); u1 = __uint_as_float(wu & 0xFFFF0000u);
      } else {
        const float2 fg = __half22float2(*reinterpret_cast<const __half2*>(&wg));
        const float2 fu = __half22float2(*reinterpret_cast<const __half2*>(&wu));
        g0 = fg.x; g1 = fg.y; u0 = fu.x; u1 = fu.y;
      }
      x[2 * i] = to_f32<T>(from_f32<T>(silu_f32(g0) * u0));
      x[2 * i + 1] = to_f32<T>(from_f32<T>(silu_f32(g1) * u1));
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
    float scale = __fmul_rn(gs, __fmul_rn(amax, 0.16666667163372039794921875f));
    scale = fminf(scale, 448.f);
    const uint8_t sfb = f32_to_e4m3(scale);
    const float os = out_scale_of(sfb, rcp_gs);
    codes[b * 2] = f32x8_to_e2m1(__fmul_rn(x[0], os), __fmul_rn(x[1], os), __fmul_rn(x[2], os), __fmul_rn(x[3], os),
                                 __fmul_rn(x[4], os), __fmul_rn(x[5], os), __fmul_rn(x[6], os), __fmul_rn(x[7], os));
    codes[b * 2 + 1] = f32x8_to_e2m1(__fmul_rn(x[8], os), __fmul_rn(x[9], os), __fmul_rn(x[10], os), __fmul_rn(x[11], os),
                                     __fmul_rn(x[12], os), __fmul_rn(x[13], os), __fmul_rn(x[14], os), __fmul_rn(x[15], os));
    sf4 |= (uint32_t)sfb << (8 * b);
  }
}

// ---------------------------------------------------------------------------------------- kernel

// BN = tile width; KB = 64-wide k-blocks (MMAs) per shared-memory stage.  Smaller stages do not change
// the bytes resident in shared memory but refill in finer steps, which keeps more of them in flight.
template <int BN, int KB, bool kOutTma = false>
struct Cfg {
  static constexpr int kAcc = BN == 128 ? 2 : 1;                    // accumulator buffers in tensor memory
  static constexpr int kSfTiles = BN / 128;                         // 128-row scale tiles on the B side
  static constexpr int kRowBytes = KB * 32;                         // packed codes per row per stage
  static constexpr int kStageA = kBM * kRowBytes;
  static constexpr int kStageB = BN * kRowBytes;
  static constexpr int kStageSFA = KB * 512;
  static constexpr int kStageSFB = kSfTiles * KB * 512;
  static constexpr int kStageBytes = kStageA + kStageB + kStageSFA + kStageSFB;
  // BN = 256 gives one of its four stages to the epilogue's staging buffers (tile stores through the copy engine)
  static constexpr int kStages = (BN == 128 ? 24 : (kOutTma ? 12 : 16)) / KB;
  static constexpr int kOutStage = kOutTma ? 8 * 4096 : 0;         // 8 epilogue warps x [32 rows x 64 columns] 16-bit
  // tensor-memory column map: accumulators, then one scale-factor block per shared-memory stage
  // (4 columns per k-block for A, 4*kSfTiles for B)
  static constexpr uint32_t kSfCols = KB * (4 + 4 * kSfTiles);
  static constexpr uint32_t kSfBase = kAcc * BN;
  static_assert(kSfBase + kStages * kSfCols <= 512, "tensor memory budget");
  static constexpr int kBarBytes = 1024;
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + kOutStage + 1024 /*alignment slack*/ + kBarBytes;
  // instruction descriptor: E2M1 x E2M1, UE4M3 scales, K-major A and B, N = BN, M = 128, dense K = 64
  static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
};

template <int BN, int KB, bool kGrouped, bool kSiluQuant = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
    nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  constexpr bool kOutTma = BN == 256 && !kGrouped && !kSiluQuant;     // the dense wide-tile kernel stores tiles through the copy engine
  using C = Cfg<BN, KB, kOutTma>;
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* out_stage = smem + (size_t)C::kStages * C::kStageBytes;      // 1024-byte aligned (stages are multiples of 1 KiB)
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + C::kOutStage);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* acc_full = bars + 2 * C::kStages;
  uint64_t* acc_empty = acc_full + C::kAcc;
  uint64_t* sf_ready = acc_empty + C::kAcc;
  uint64_t* sf_full = sf_ready + C::kStages;     // scale factors of the stage have landed (before the operands)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(sf_full + C::kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // dense mode: the status word is cleared here instead of by a separate memset (a wait only writes it after its ~1 s
  // budget, long after this store); in grouped mode the tile-list kernel has cleared it
  if (!kGrouped && blockIdx.x == 0 && threadIdx.x == 0) *p.status = 0;
  const int m_tiles = kGrouped ? p.g_hdr[0] : p.m_tiles;
  const int n_tiles_total = m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_ready[s]), 4);       // one arrival per scale-factor warp
      mbar_init(smem_u32(&sf_full[s]), 1);
    }
    for (int a = 0; a < C::kAcc; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 8);      // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr_smem)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const int KT = (p.K + 63) / 64;   // 64-wide k-blocks = 512-byte scale tiles per 128 rows

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
        const TileInfo ti = tile_info<BN, kGrouped, kSiluQuant>(p, tile, m_tiles);
        const uint8_t* sfb_base = p.sfb + (kGrouped ? (size_t)ti.expert * (size_t)p.g_sfb_expert_bytes : (size_t)0);
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, 1)) { ok = false; break; }
          unsigned char* st = smem + (size_t)s * C::kStageBytes;
          const int kblocks = min(KB, KT - ks * KB);
          int sf_tiles = 0;
          for (int j = 0; j < C::kSfTiles; ++j) sf_tiles += ((j == 0 ? ti.sfb_tile0 : ti.sfb_tile1) * 128 < p.N) ? 1 : 0;
          // the small scale-factor copies go first and on their own barrier, so the scale warps can
          // move them into tensor memory while the operand tiles are still in flight
          const uint32_t sbar = smem_u32(&sf_full[s]);
          mbar_expect_tx(sbar, (uint32_t)(kblocks * 512 * (1 + sf_tiles)));
          bulk_load_1d(smem_u32(st + C::kStageA + C::kStageB), p.sfa + ((size_t)ti.sfa_tile * KT + (size_t)ks * KB) * 512,
                       (uint32_t)kblocks * 512, sbar);
          for (int j = 0; j < sf_tiles; ++j)
            bulk_load_1d(smem_u32(st + C::kStageA + C::kStageB + C::kStageSFA + j * (KB * 512)),
                         sfb_base + ((size_t)(j == 0 ? ti.sfb_tile0 : ti.sfb_tile1) * KT + (size_t)ks * KB) * 512,
                         (uint32_t)kblocks * 512, sbar);
          const uint32_t bar = smem_u32(&full_bar[s]);
          mbar_expect_tx(bar, (uint32_t)(C::kStageA + C::kStageB));
          tma_load_2d(smem_u32(st), &map_a, ks * C::kRowBytes, ti.a_row0, bar);
          if (kSiluQuant) {
            // map_b's box is 128 rows here: the gate rows and the up rows of the tile land one after the other
            tma_load_2d(smem_u32(st + C::kStageA), &map_b, ks * C::kRowBytes, ti.b_row0, bar);
            tma_load_2d(smem_u32(st + C::kStageA + 128 * C::kRowBytes), &map_b, ks * C::kRowBytes, ti.b_row1, bar);
          } else {
            tma_load_2d(smem_u32(st + C::kStageA), &map_b, ks * C::kRowBytes, ti.b_row0, bar);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount % C::kAcc, aph = (tcount / C::kAcc) & 1;
        if (!mbar_wait(smem_u32(&acc_empty[acc]), aph ^ 1, p.status, 2)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, p.status, 3)) { ok = false; break; }
          tcgen05_fence_after();
          unsigned char* st = smem + (size_t)s * C::kStageBytes;
          const int kblocks = min(KB, KT - ks * KB);
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + C::kStageA);
          const uint32_t sfa_tmem = tmem_base + C::kSfBase + s * C::kSfCols, sfb_tmem = sfa_tmem + 4 * KB;
          if (!mbar_wait(smem_u32(&sf_ready[s]), ph, p.status, 5)) { ok = false; break; }
          tcgen05_fence_after();
          for (int kb = 0; kb < kblocks; ++kb) {
            // each 64-wide k-block is 32 bytes further along the swizzled 128-byte rows
            tcgen05_mma_nvf4(d_tmem, desc_kmajor<C::kRowBytes>(a_addr + kb * 32), desc_kmajor<C::kRowBytes>(b_addr + kb * 32),
                             C::kIdesc, sfa_tmem + kb * 4, sfb_tmem + kb * (4 * C::kSfTiles), (ks > 0 || kb > 0) ? 1u : 0u);
          }
          tcgen05_commit(smem_u32(&empty_bar[s]));    // frees the stage when these MMAs have read it
        }
        if (ok) tcgen05_commit(smem_u32(&acc_full[acc]));
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ------------------------------------------------------------------ scale factors (warps 6..9)
    // Each warp owns one 32-lane quarter of tensor memory.  Lane L needs row L of every 32x16-byte
    // scale tile (the four quarters hold identical copies), so each lane moves 16 bytes from shared
    // memory to its own lane with tcgen05.st -- this keeps the scale traffic off the tensor pipe,
    // where a tcgen05.cp per tile costs about a quarter of an MMA.
    const int quarter = warp & 3;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
      for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
        const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1;
        ok = mbar_wait(smem_u32(&sf_full[s]), ph, p.status, 6);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const unsigned char* sf = smem + (size_t)s * C::kStageBytes + C::kStageA + C::kStageB;
        const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::kSfBase + s * C::kSfCols;
        const int kblocks = min(KB, KT - ks * KB);
        for (int kb = 0; kb < kblocks; ++kb) {
          tcgen05_st_32x32_x4(t0 + kb * 4, *reinterpret_cast<const uint4*>(sf + kb * 512 + lane * 16));
#pragma unroll
          for (int j = 0; j < C::kSfTiles; ++j)
            tcgen05_st_32x32_x4(t0 + 4 * KB + kb * (4 * C::kSfTiles) + j * 4,
                                *reinterpret_cast<const uint4*>(sf + C::kStageSFA + j * (KB * 512) + kb * 512 + lane * 16));
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sf_ready[s]));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 and 10..13)
    // Two warps per tensor-memory lane quarter, each draining and storing half of the tile's columns.
    // With long K the epilogue hides behind the next tile either way; with short K (the grouped down
    // projection: 8 MMAs per tile) the kernel is bound by how fast a tile can be drained and stored.
    const int quarter = warp & 3;                 // tensor-memory lanes [32*quarter, +32) belong to this warp
    constexpr int CH = BN / 64;                   // 32-column chunks per warp
    const int c_first = warp >= 10 ? CH : 0;
    const float alpha_dense = kGrouped ? 0.f : p.alpha[0];
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x, ++tcount) {
      const TileInfo ti = tile_info<BN, kGrouped, kSiluQuant>(p, tile, m_tiles);
      const float alpha = kGrouped ? p.g_alphas[ti.expert] : alpha_dense;
      const uint32_t acc = tcount % C::kAcc, aph = (tcount / C::kAcc) & 1;
      ok = mbar_wait(smem_u32(&acc_full[acc]), aph, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = ti.a_row0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      if constexpr (kSiluQuant) {
        // Tensor-memory columns [0,128) hold the gate half of this thread's row, [128,256) the up half.
        // This warp takes 64 of the 128 output columns: 4 blocks of 16 -> 32 bytes of codes + 4 scale bytes,
        // computed exactly as the separate SiLU-mul quantizer does from the 16-bit rounded GEMM output.
        const int half = warp >= 10 ? 1 : 0;
        const float gs = p.q_gs[ti.expert];
        const float rcp_gs = __frcp_rn(gs + (gs == 0.f ? 1.0e8f : 0.f));
        // drain both halves as 16-bit pairs (the rounding the separate GEMM's output has), hand the accumulator
        // back, and only then do the SiLU / quantization arithmetic, so that it overlaps the next tile's main loop
        uint32_t pg[32], pu[32];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rg[32], ru[32];
          tcgen05_ld_32x32(taddr + (half * 2 + c) * 32, rg);
          tcgen05_ld_32x32(taddr + 128 + (half * 2 + c) * 32, ru);
          tcgen05_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float g0 = __uint_as_float(rg[2 * i]) * alpha, g1 = __uint_as_float(rg[2 * i + 1]) * alpha;
            const float u0 = __uint_as_float(ru[2 * i]) * alpha, u1 = __uint_as_float(ru[2 * i + 1]) * alpha;
            if (p.out_bf16) {
              const __nv_bfloat162 vg = __floats2bfloat162_rn(g0, g1), vu = __floats2bfloat162_rn(u0, u1);
              pg[c * 16 + i] = *reinterpret_cast<const uint32_t*>(&vg);
              pu[c * 16 + i] = *reinterpret_cast<const uint32_t*>(&vu);
            } else {
              const __half2 vg = __floats2half2_rn(g0, g1), vu = __floats2half2_rn(u0, u1);
              pg[c * 16 + i] = *reinterpret_cast<const uint32_t*>(&vg);
              pu[c * 16 + i] = *reinterpret_cast<const uint32_t*>(&vu);
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
        // rows past the end of the expert are never stored: warps whose 32 rows are all past it skip the arithmetic
        if (row < ti.row_end) {
          uint32_t codes[8];
          uint32_t sf4 = 0;
          if (p.out_bf16) silu_quant_row<__nv_bfloat16>(pg, pu, gs, rcp_gs, codes, sf4);
          else silu_quant_row<__half>(pg, pu, gs, rcp_gs, codes, sf4);
          uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + (size_t)row * (size_t)(p.q_inter / 2) + (ti.n0 + half * 64) / 2;
          st_global_v8(dst, codes);
          const size_t kt2 = (size_t)(p.q_inter / 64);
          *reinterpret_cast<uint32_t*>(p.q_sf + ((size_t)ti.sfa_tile * kt2 + (size_t)(ti.n0 / 64 + half)) * 512 + lane * 16 +
                                       quarter * 4) = sf4;
        }
        continue;
      }
      if (!kGrouped && p.out_f32) {
        // fp32 output (the cudaFP4GemmEx form): each 32-column chunk goes straight from tensor memory to global
        // memory; the accumulator is handed back after the last chunk
        float* dst_row = reinterpret_cast<float*>(p.out) + (size_t)row * p.N;
#pragma unroll 1
        for (int c = 0; c < CH; ++c) {
          uint32_t r[32];
          tcgen05_ld_32x32(taddr + (c_first + c) * 32, r);
          tcgen05_wait_ld();
          const int col0 = ti.n0 + (c_first + c) * 32;
          if (row < ti.row_end && col0 < p.N) {
            if (col0 + 32 <= p.N && (p.N % 4) == 0) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(dst_row + col0)[i] =
                    make_float4(__uint_as_float(r[4 * i]) * alpha, __uint_as_float(r[4 * i + 1]) * alpha,
                                __uint_as_float(r[4 * i + 2]) * alpha, __uint_as_float(r[4 * i + 3]) * alpha);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) dst_row[col0 + i] = __uint_as_float(r[i]) * alpha;
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
        continue;
      }
      // drain this thread's row of the accumulator into packed 16-bit registers ...
      uint32_t packed[BN / 4];
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        uint32_t r[32];
        tcgen05_ld_32x32(taddr + (c_first + c) * 32, r);
        tcgen05_wait_ld();
        if (p.out_bf16) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * i]) * alpha, __uint_as_float(r[2 * i + 1]) * alpha);
            packed[c * 16 + i] = *reinterpret_cast<uint32_t*>(&v);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __half2 v = __floats2half2_rn(__uint_as_float(r[2 * i]) * alpha, __uint_as_float(r[2 * i + 1]) * alpha);
            packed[c * 16 + i] = *reinterpret_cast<uint32_t*>(&v);
          }
        }
      }
      // ... hand the accumulator back to the MMA warp, and only then write to global memory, so
      // that the stores overlap the next tile's main loop
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
      if (kOutTma && p.out_tma) {
        // This warp's 32 rows x 128 columns leave in two halves of 64 columns (128 bytes per row): rows go to a private
        // staging buffer with the 128-byte swizzle of the tensor map (16-byte chunk c of row r at c ^ (r % 8): the
        // lanes of a warp write different banks), one lane hands the box to the copy engine, which writes whole lines
        // and clips rows / columns beyond the tensor.
        const uint32_t stg = smem_u32(out_stage) + (uint32_t)((warp >= 10 ? 4 : 0) + quarter) * 4096u;
        const int row0 = ti.a_row0 + quarter * 32;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (lane == 0) bulk_wait_read0();          // the previous box has left the buffer
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            sts128(stg + (uint32_t)lane * 128u + (uint32_t)((c ^ (lane & 7)) << 4), packed[hh * 32 + 4 * c],
                   packed[hh * 32 + 4 * c + 1], packed[hh * 32 + 4 * c + 2], packed[hh * 32 + 4 * c + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          const int col0 = ti.n0 + (c_first * 32) + hh * 64;
          if (lane == 0 && col0 < p.N && row0 < p.M) {
            tma_store_2d(&map_out, col0, row0, stg);
            bulk_commit();
          }
        }
        continue;
      }
      if (row < ti.row_end) {
        uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.out) + (size_t)row * p.N;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const int col0 = ti.n0 + (c_first + c) * 32;
          if (col0 < p.N) {
            uint16_t* dst = dst_row + col0;
            if (col0 + 32 <= p.N && (p.N % 16) == 0 && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
              // 32-byte stores: whole sectors, half as many store instructions as 16-byte ones
#pragma unroll
              for (int i = 0; i < 2; ++i)
                st_global_v8(dst + 16 * i, &packed[c * 16 + 8 * i]);
            } else if (col0 + 32 <= p.N && (p.N % 8) == 0) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(packed[c * 16 + 4 * i], packed[c * 16 + 4 * i + 1],
                                                              packed[c * 16 + 4 * i + 2], packed[c * 16 + 4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N)
                  dst[i] = (uint16_t)((i & 1) ? (packed[c * 16 + (i >> 1)] >> 16) : (packed[c * 16 + (i >> 1)] & 0xFFFFu));
            }
          }
        }
      }
    }
  }
  // all roles fall through to here (also after a timed-out wait), so tensor memory is always freed
  if (kOutTma && p.out_tma && lane == 0 && (warp >= 2 && (warp < 6 || warp >= 10))) bulk_wait0();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------- grouped helpers

constexpr int kGroupMaxExperts = 4096;
constexpr int kPermuteGridMinPairs = 8192;   // below this one block does the whole routing pass

// One block: cuts every expert's row range into 128-row tiles.
//   hdr[0] = number of tiles; mtiles[t] = {first row, end row of the expert, A scale-tile row, expert}
__global__ void __launch_bounds__(1024)
    grouped_tiles_kernel(const int* __restrict__ expert_offsets, const int* __restrict__ sf_offsets, int E, int* hdr,
                         int4* mtiles, int max_tiles) {
  __shared__ int s_scan[1024];
  __shared__ int s_base;
  const int tid = threadIdx.x;
  if (tid == 0) s_base = 0;
  // the four ints in front of hdr are the GEMM's status word (0 = ok) and its padding: cleared here with hdr, so the
  // call needs no separate memset
  if (tid < 8) hdr[tid - 4] = 0;
  __syncthreads();
  for (int e0 = 0; e0 < E; e0 += 1024) {
    const int e = e0 + tid;
    int rows = 0, first = 0;
    if (e < E) {
      first = expert_offsets[e];
      rows = expert_offsets[e + 1] - first;
    }
    const int nt = (rows + kBM - 1) / kBM;
    s_scan[tid] = nt;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {          // inclusive Hillis-Steele scan
      const int v = tid >= d ? s_scan[tid - d] : 0;
      __syncthreads();
      s_scan[tid] += v;
      __syncthreads();
    }
    const int start = s_base + s_scan[tid] - nt;
    if (e < E) {
      const int sf_row_tile = sf_offsets[e] / 128;
      for (int i = 0; i < nt; ++i)
        if (start + i < max_tiles) mtiles[start + i] = make_int4(first + i * kBM, first + rows, sf_row_tile + i, e);
    }
    __syncthreads();
    if (tid == 1023) s_base += s_scan[1023];
    __syncthreads();
  }
  if (tid == 0) hdr[0] = min(s_base, max_tiles);
}

// Routing metadata for the grouped path (one block): counts pairs per local expert and writes
//   expert_offsets[E+1]      first permuted row of every expert
//   blockscale_offsets[E+1]  the same with every expert padded to a multiple of 128 rows
//   dst2src[P]               permuted row -> pair index (token*topk + slot); -1 past the last valid row
//   src2dst[P]               pair index -> permuted row, or -1 if the pair's expert is not local
__global__ void __launch_bounds__(1024)
    moe_permute_kernel(const int32_t* __restrict__ topk_ids, int P, const int32_t* __restrict__ expert_map, int global_E,
                       int E, int* expert_offsets, int* blockscale_offsets, int* dst2src, int* src2dst) {
  __shared__ int s_count[kGroupMaxExperts];
  __shared__ int s_scan[1024], s_scan2[1024];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += 1024) s_count[e] = 0;
  __syncthreads();
  for (int p = tid; p < P; p += 1024) {
    int e = topk_ids[p];
    if (expert_map != nullptr) e = (e >= 0 && e < global_E) ? expert_map[e] : -1;
    if (e < 0 || e >= E) e = -1;
    src2dst[p] = e;                      // holds the local expert id until the scatter below
    dst2src[p] = -1;
    if (e >= 0) atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  const int per = (E + 1023) / 1024;
  int sum = 0, sum_pad = 0;
  for (int i = 0; i < per; ++i) {
    const int e = tid * per + i;
    if (e < E) {
      sum += s_count[e];
      sum_pad += (s_count[e] + 127) / 128 * 128;
    }
  }
  s_scan[tid] = sum;
  s_scan2[tid] = sum_pad;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    const int v = tid >= d ? s_scan[tid - d] : 0, v2 = tid >= d ? s_scan2[tid - d] : 0;
    __syncthreads();
    s_scan[tid] += v;
    s_scan2[tid] += v2;
    __syncthreads();
  }
  int base = s_scan[tid] - sum, base_pad = s_scan2[tid] - sum_pad;
  for (int i = 0; i < per; ++i) {
    const int e = tid * per + i;
    if (e < E) {
      const int c = s_count[e];
      expert_offsets[e] = base;
      blockscale_offsets[e] = base_pad;
      s_count[e] = base;                 // scatter cursor
      base += c;
      base_pad += (c + 127) / 128 * 128;
    }
  }
  if (tid == 1023) {
    expert_offsets[E] = s_scan[1023];
    blockscale_offsets[E] = s_scan2[1023];
  }
  __syncthreads();
  for (int p = tid; p < P; p += 1024) {
    const int e = src2dst[p];
    if (e >= 0) {
      const int pos = atomicAdd(&s_count[e], 1);
      src2dst[p] = pos;
      dst2src[pos] = p;
    }
  }
}

// The same routing metadata for large batches, as three grid-wide steps around global counters kept in
// expert_offsets itself (no scratch): count pairs per expert, scan, scatter with expert_offsets[e] as
// the running cursor, then shift the cursors (now each expert's end) back into start offsets.
// Both grid-wide passes aggregate per block in shared memory first: with skewed routing a popular expert would
// otherwise take one global atomic per pair on a single address.
constexpr int kPermuteBlock = 1024;

__global__ void __launch_bounds__(kPermuteBlock)
    moe_permute_count_kernel(const int32_t* __restrict__ topk_ids, int P, const int32_t* __restrict__ expert_map,
                             int global_E, int E, int* expert_offsets, int* dst2src, int* src2dst) {
  __shared__ int s_count[kGroupMaxExperts];
  for (int e = threadIdx.x; e < E; e += kPermuteBlock) s_count[e] = 0;
  __syncthreads();
  const int p = blockIdx.x * kPermuteBlock + threadIdx.x;
  if (p < P) {
    int e = topk_ids[p];
    if (expert_map != nullptr) e = (e >= 0 && e < global_E) ? expert_map[e] : -1;
    if (e < 0 || e >= E) e = -1;
    src2dst[p] = e;
    dst2src[p] = -1;
    if (e >= 0) atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kPermuteBlock) {
    const int c = s_count[e];
    if (c > 0) atomicAdd(&expert_offsets[e], c);
  }
}

__global__ void __launch_bounds__(1024)
    moe_permute_scan_kernel(int E, int* expert_offsets, int* blockscale_offsets) {
  __shared__ int s_scan[1024], s_scan2[1024];
  const int tid = threadIdx.x;
  const int per = (E + 1023) / 1024;
  int sum = 0, sum_pad = 0;
  for (int i = 0; i < per; ++i) {
    const int e = tid * per + i;
    if (e < E) {
      const int c = expert_offsets[e];
      sum += c;
      sum_pad += (c + 127) / 128 * 128;
    }
  }
  s_scan[tid] = sum;
  s_scan2[tid] = sum_pad;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    const int v = tid >= d ? s_scan[tid - d] : 0, v2 = tid >= d ? s_scan2[tid - d] : 0;
    __syncthreads();
    s_scan[tid] += v;
    s_scan2[tid] += v2;
    __syncthreads();
  }
  int base = s_scan[tid] - sum, base_pad = s_scan2[tid] - sum_pad;
  for (int i = 0; i < per; ++i) {
    const int e = tid * per + i;
    if (e < E) {
      const int c = expert_offsets[e];
      expert_offsets[e] = base;
      blockscale_offsets[e] = base_pad;
      base += c;
      base_pad += (c + 127) / 128 * 128;
    }
  }
  if (tid == 1023) {
    expert_offsets[E] = s_scan[1023];
    blockscale_offsets[E] = s_scan2[1023];
  }
}

__global__ void __launch_bounds__(kPermuteBlock)
    moe_permute_scatter_kernel(int P, int E, int* expert_offsets, int* dst2src, int* src2dst) {
  __shared__ int s_count[kGroupMaxExperts];     // pairs of this block per expert, then the block's first row
  for (int e = threadIdx.x; e < E; e += kPermuteBlock) s_count[e] = 0;
  __syncthreads();
  const int p = blockIdx.x * kPermuteBlock + threadIdx.x;
  int e = -1, rank = 0;
  if (p < P) {
    e = src2dst[p];
    if (e >= 0) rank = atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += kPermuteBlock) {
    const int c = s_count[i];
    if (c > 0) s_count[i] = atomicAdd(&expert_offsets[i], c);
  }
  __syncthreads();
  if (e >= 0) {
    const int pos = s_count[e] + rank;
    src2dst[p] = pos;
    dst2src[pos] = p;
  }
}

__global__ void __launch_bounds__(1024) moe_permute_shift_kernel(int E, int* expert_offsets) {
  __shared__ int s_end[kGroupMaxExperts];
  for (int e = threadIdx.x; e < E; e += 1024) s_end[e] = expert_offsets[e];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += 1024) expert_offsets[e + 1] = s_end[e];
  if (threadIdx.x == 0) expert_offsets[0] = 0;
}

// out[i, :] = in[dst2src[i] / src_div, :] for 16-byte chunks; rows whose map entry is < 0 become zero.
__global__ void shuffle_rows_kernel(const uint4* __restrict__ in, const int* __restrict__ dst2src, int src_div,
                                    int64_t chunks_per_row, int64_t n_dst, uint4* __restrict__ out) {
  const int64_t total = n_dst * chunks_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks_per_row, c = i - r * chunks_per_row;
    const int src = dst2src[r];
    out[i] = src >= 0 ? in[(int64_t)(src / src_div) * chunks_per_row + c] : make_uint4(0, 0, 0, 0);
  }
}

// out[m, h] = sum over the token's slots of weight * expert_out[src2dst[m*topk + t], h] (local pairs only).
template <typename T>
__global__ void unpermute_reduce_kernel(const T* __restrict__ expert_out, const int* __restrict__ src2dst,
                                        const float* __restrict__ topk_w, int M, int topk, int H, T* __restrict__ out) {
  const int m = blockIdx.y;
  for (int h = (blockIdx.x * blockDim.x + threadIdx.x) * 2; h < H; h += gridDim.x * blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int t = 0; t < topk; ++t) {
      const int r = src2dst[m * topk + t];
      if (r < 0) continue;
      const float w = topk_w[m * topk + t];
      a0 = fmaf(w, to_f32<T>(expert_out[(int64_t)r * H + h]), a0);
      a1 = fmaf(w, to_f32<T>(expert_out[(int64_t)r * H + h + 1]), a1);
    }
    out[(int64_t)m * H + h] = from_f32<T>(a0);
    out[(int64_t)m * H + h + 1] = from_f32<T>(a1);
  }
}

// The same for H % 8 == 0 and 16-byte aligned rows: eight columns per thread, 16-byte loads and stores,
// same order of additions per output element.
template <typename T>
__global__ void unpermute_reduce_vec8_kernel(const T* __restrict__ expert_out, const int* __restrict__ src2dst,
                                             const float* __restrict__ topk_w, int M, int topk, int H, T* __restrict__ out) {
  const int m = blockIdx.y;
  const int h = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (h >= H) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int t = 0; t < topk; ++t) {
    const int r = src2dst[m * topk + t];
    if (r < 0) continue;
    const float w = topk_w[m * topk + t];
    const uint4 raw = *reinterpret_cast<const uint4*>(expert_out + (int64_t)r * H + h);
    const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, to_f32<T>(v[i]), acc[i]);
  }
  uint4 o;
  T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
  for (int i = 0; i < 8; ++i) ov[i] = from_f32<T>(acc[i]);
  *reinterpret_cast<uint4*>(out + (int64_t)m * H + h) = o;
}

// ---------------------------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Encoded maps are remembered by their arguments (a weight is encoded once, not once per call).
struct MapKey {
  const void* base;
  uint64_t rows, row_bytes;
  uint32_t box_rows;
  int box_bytes;
};
struct MapCache {
  static constexpr int kSlots = 64;
  MapKey key[kSlots];
  CUtensorMap map[kSlots];
  bool used[kSlots] = {false};
  std::mutex mu;
};
MapCache g_map_cache;

bool make_map_uncached(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, int box_bytes);

// [rows, row_bytes] u8 row-major; box = box_bytes (128/64/32) x box_rows with the matching swizzle, zero fill out of bounds
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, int box_bytes) {
  const MapKey k{base, rows, row_bytes, box_rows, box_bytes};
  const size_t h = (reinterpret_cast<uintptr_t>(base) >> 8) * 0x9E3779B97F4A7C15ull + rows * 31 + box_rows;
  const int slot = (int)(h % MapCache::kSlots);
  std::lock_guard<std::mutex> lock(g_map_cache.mu);
  if (g_map_cache.used[slot] && memcmp(&g_map_cache.key[slot], &k, sizeof(MapKey)) == 0) {
    *map = g_map_cache.map[slot];
    return true;
  }
  if (!make_map_uncached(map, base, rows, row_bytes, box_rows, box_bytes)) return false;
  memset(&g_map_cache.key[slot], 0, sizeof(MapKey));
  g_map_cache.key[slot] = k;
  g_map_cache.map[slot] = *map;
  g_map_cache.used[slot] = true;
  return true;
}

bool make_map_uncached(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, int box_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, box_rows};
  const CUtensorMapSwizzle sw = box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : (box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [rows, cols] 16-bit row-major output; box = 64 columns (128 bytes) x 32 rows, 128-byte swizzle
bool make_out_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int KB, bool kGrouped, bool kSiluQuant = false>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p, int max_m_tiles, cudaStream_t st,
                const CUtensorMap* mo = nullptr) {
  using C = Cfg<BN, KB, BN == 256 && !kGrouped && !kSiluQuant>;
  CUtensorMap dummy = {};
  if (mo == nullptr) {
    mo = &dummy;
    p.out_tma = 0;
  }
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(nvfp4_gemm_kernel<BN, KB, kGrouped, kSiluQuant>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)C::kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  p.n_tiles = kSiluQuant ? p.q_inter / 128 : (p.N + BN - 1) / BN;
  long long grid = (long long)max_m_tiles * p.n_tiles;
  if (grid > sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  p.k_stages = (p.K + KB * 64 - 1) / (KB * 64);
  nvfp4_gemm_kernel<BN, KB, kGrouped, kSiluQuant><<<(unsigned)grid, kGemmThreads, C::kSmemBytes, st>>>(ma, mb, *mo, p);
  return B200FP4_STATUS_SUCCESS;
}

// 64-wide k-blocks per shared-memory stage.  The kernel template also builds with 2 or 1 (64- and
// 32-byte swizzled rows, 8 or 16 stages); on B200 those measured 190 and 317 us against 150 us at
// M=4096 (TMA issues one request per box row, so narrower rows double and quadruple the requests).
int stage_kblocks() { return 4; }

template <bool kGrouped>
int dispatch_gemm(int bn, int kb, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int max_m_tiles,
                  cudaStream_t st, const CUtensorMap* mo = nullptr) {
  (void)kb;
  if (bn == 256) return launch_gemm<256, 4, kGrouped>(ma, mb, p, max_m_tiles, st, mo);
  return launch_gemm<128, 4, kGrouped>(ma, mb, p, max_m_tiles, st);
}

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" size_t b200fp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  (void)M; (void)N; (void)K;
  return 256;
}

extern "C" int b200fp4_gemm_nvfp4(const void* a_codes, const void* b_codes, const void* sfa, const void* sfb,
                                  const float* alpha, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                                  int tile_n, void* workspace, size_t workspace_bytes, void* stream) {
  if (M < 0 || N <= 0 || K <= 0 || (K % 64) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (out_dtype != B200FP4_DTYPE_BF16 && out_dtype != B200FP4_DTYPE_F16 && out_dtype != B200FP4_DTYPE_F32)
    return B200FP4_STATUS_NOT_SUPPORTED;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!a_codes || !b_codes || !sfa || !sfb || !alpha || !out) return B200FP4_STATUS_INVALID_VALUE;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(sfa, 16) || !aligned(sfb, 16) || !aligned(out, 16) ||
      ((K / 2) % 16) != 0)
    return B200FP4_STATUS_INVALID_VALUE;
  if (!workspace || workspace_bytes < 256 || !aligned(workspace, 16)) return B200FP4_STATUS_ALLOC_FAILED;
  if (tile_n != 0 && tile_n != 128 && tile_n != 256 && tile_n != 512) return B200FP4_STATUS_INVALID_VALUE;
  if (tile_n == 512 && out_dtype == B200FP4_DTYPE_F32) return B200FP4_STATUS_NOT_SUPPORTED;
  if (M > (1 << 24) || N > (1 << 24) || K > (1 << 24)) return B200FP4_STATUS_NOT_SUPPORTED;
  if (b200fp4_has_hardware_acceleration() != 1) return B200FP4_STATUS_ARCH_MISMATCH;
  cudaStream_t st = (cudaStream_t)stream;
  GemmParams p;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa);
  p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.alpha = alpha;
  p.out = out;
  p.out_bf16 = out_dtype == B200FP4_DTYPE_BF16;
  p.out_f32 = out_dtype == B200FP4_DTYPE_F32;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.m_tiles = (int)((M + kBM - 1) / kBM);
  p.status = reinterpret_cast<int*>(workspace);
  // Wide tiles once there are enough of them to fill the GPU; narrow tiles (double-buffered
  // accumulator, twice the CTAs) for small problems.
  // ... and 256 x 256 tiles on pairs of CTAs (gemm_pair.cu) once there are two rounds of those for every pair of SMs
  // (measured at N=14336, K=4096: M=1024 46 us against 48 us, M=4096 123 us against 129 us; M=128 stays with 128-wide tiles).
  int bn = tile_n;
  if (bn == 0) {
    bn = (p.m_tiles * ((N + 255) / 256) >= sm_count()) ? 256 : 128;
    if (bn == 256 && !p.out_f32 && ((M + 255) / 256) * ((N + 255) / 256) >= sm_count()) bn = 512;
  }
  const int kb = stage_kblocks();
  if (bn == 512) {
    // 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2)
    CUtensorMap pa, pb;
    if (!make_map(&pa, a_codes, (uint64_t)M, (uint64_t)K / 2, 128, 128) ||
        !make_map(&pb, b_codes, (uint64_t)N, (uint64_t)K / 2, 128, 128))
      return B200FP4_STATUS_INTERNAL_ERROR;
    const int rc2 = launch_gemm_pair(pa, pb, p.sfa, p.sfb, alpha, out, p.out_bf16, (int)M, (int)N, (int)K, p.status, st);
    if (rc2 != B200FP4_STATUS_SUCCESS) return rc2;
    return finish_launch(1);
  }
  CUtensorMap ma, mb;
  if (!make_map(&ma, a_codes, (uint64_t)M, (uint64_t)K / 2, kBM, kb * 32) ||
      !make_map(&mb, b_codes, (uint64_t)N, (uint64_t)K / 2, (uint32_t)bn, kb * 32))
    return B200FP4_STATUS_INTERNAL_ERROR;
  p.g_hdr = nullptr;
  p.g_mtiles = nullptr;
  p.g_alphas = nullptr;
  p.g_sfb_expert_bytes = 0;
  // wide tiles, 16-bit output with 16-byte aligned rows: tiles leave through the copy engine
  CUtensorMap mo;
  const bool tma_out = bn == 256 && !p.out_f32 && (N % 8) == 0 && make_out_map(&mo, out, (uint64_t)M, (uint64_t)N);
  p.out_tma = tma_out ? 1 : 0;
  int rc = dispatch_gemm<false>(bn, kb, ma, mb, p, p.m_tiles, st, tma_out ? &mo : nullptr);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  return finish_launch(1);
}

// ---------------------------------------------------------------------------------------- linear layer in one call

// y = NVFP4(x) @ W^T: the activation quantizer and the GEMM queued by one call (two launches a few microseconds apart;
// through two Python calls the GPU idles between them for longer than either kernel runs at prefill sizes).
// workspace: [codes M*K/2 | swizzled block scales | GEMM workspace], each part 256-byte aligned.
static size_t linear_part(size_t v) { return (v + 255) / 256 * 256; }

extern "C" size_t b200fp4_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M < 0 || N <= 0 || K <= 0 || (K % 16) != 0) return 0;
  return linear_part((size_t)M * (size_t)K / 2) + linear_part(b200fp4_sf_swizzled_bytes(M, K / 16)) +
         linear_part(b200fp4_gemm_workspace_bytes(M, N, K));
}

extern "C" int b200fp4_linear_nvfp4(const void* x, int x_dtype, int64_t ldx, const float* x_global_scale, const void* w_codes,
                                    const void* w_sf, const float* alpha, void* out, int out_dtype, int64_t M, int64_t N,
                                    int64_t K, int tile_n, void* workspace, size_t workspace_bytes, void* stream) {
  if (M < 0 || N <= 0 || K <= 0 || (K % 64) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!workspace || !aligned(workspace, 256) || workspace_bytes < b200fp4_linear_workspace_bytes(M, N, K))
    return B200FP4_STATUS_ALLOC_FAILED;
  unsigned char* codes = static_cast<unsigned char*>(workspace);
  unsigned char* sf = codes + linear_part((size_t)M * (size_t)K / 2);
  unsigned char* gemm_ws = sf + linear_part(b200fp4_sf_swizzled_bytes(M, K / 16));
  int rc = b200fp4_quantize(x, x_dtype, M, K, ldx, x_global_scale, codes, sf, 1, stream);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  return b200fp4_gemm_nvfp4(codes, w_codes, sf, w_sf, alpha, out, out_dtype, M, N, K, tile_n, gemm_ws,
                            b200fp4_gemm_workspace_bytes(M, N, K), stream);
}

// ---------------------------------------------------------------------------------------- grouped entry points

extern "C" size_t b200fp4_grouped_gemm_workspace_bytes(int64_t rows_capacity, int64_t E) {
  if (rows_capacity < 0 || E < 0) return 0;
  return 256 + (size_t)(rows_capacity / kBM + E + 1) * sizeof(int4);
}

// q_sf / q_gs non-null: the gate_up projection with SiLU(gate)*up and the NVFP4 quantization of the result in the
// epilogue (out = packed codes [rows_capacity, N/4]).
static int grouped_gemm_impl(const void* a_codes, const void* b_codes, const void* a_sf, const void* b_sf,
                             const float* alphas, const int32_t* expert_offsets, const int32_t* sf_offsets, void* out,
                             int out_dtype, int64_t rows_capacity, int64_t N, int64_t K, int64_t E, int tile_n,
                             void* workspace, size_t workspace_bytes, void* stream, void* q_sf, const float* q_gs) {
  const bool fused = q_sf != nullptr;
  if (fused && (!q_gs || (N % 256) != 0 || !aligned(out, 32) || !aligned(q_sf, 4))) return B200FP4_STATUS_INVALID_VALUE;
  if (rows_capacity < 0 || N <= 0 || K <= 0 || E <= 0 || (K % 64) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (out_dtype != B200FP4_DTYPE_BF16 && out_dtype != B200FP4_DTYPE_F16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (rows_capacity == 0) return B200FP4_STATUS_SUCCESS;
  if (!a_codes || !b_codes || !a_sf || !b_sf || !alphas || !expert_offsets || !sf_offsets || !out)
    return B200FP4_STATUS_INVALID_VALUE;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(a_sf, 16) || !aligned(b_sf, 16) || !aligned(out, 16) ||
      ((K / 2) % 16) != 0)
    return B200FP4_STATUS_INVALID_VALUE;
  if (E > kGroupMaxExperts || rows_capacity > (1 << 24) || N > (1 << 20) || K > (1 << 24) || E * N > (int64_t)1 << 30)
    return B200FP4_STATUS_NOT_SUPPORTED;
  if (tile_n != 0 && tile_n != 128 && tile_n != 256 && tile_n != 512) return B200FP4_STATUS_INVALID_VALUE;
  if (tile_n == 512 && out_dtype == B200FP4_DTYPE_F32) return B200FP4_STATUS_NOT_SUPPORTED;
  if (fused && tile_n == 128) return B200FP4_STATUS_INVALID_VALUE;
  if (!workspace || !aligned(workspace, 16) || workspace_bytes < b200fp4_grouped_gemm_workspace_bytes(rows_capacity, E))
    return B200FP4_STATUS_ALLOC_FAILED;
  if (b200fp4_has_hardware_acceleration() != 1) return B200FP4_STATUS_ARCH_MISMATCH;
  cudaStream_t st = (cudaStream_t)stream;
  const int max_tiles = (int)(rows_capacity / kBM + E + 1);
  GemmParams p;
  p.sfa = reinterpret_cast<const uint8_t*>(a_sf);
  p.sfb = reinterpret_cast<const uint8_t*>(b_sf);
  p.alpha = nullptr;
  p.out = out;
  p.out_bf16 = out_dtype == B200FP4_DTYPE_BF16;
  p.out_f32 = 0;
  p.out_tma = 0;
  p.M = (int)rows_capacity; p.N = (int)N; p.K = (int)K;
  p.m_tiles = max_tiles;
  p.status = reinterpret_cast<int*>(workspace);
  p.g_hdr = reinterpret_cast<int*>(workspace) + 4;
  p.g_mtiles = reinterpret_cast<const int4*>(reinterpret_cast<unsigned char*>(workspace) + 256);
  p.g_alphas = alphas;
  p.g_sfb_expert_bytes = (long long)b200fp4_sf_swizzled_bytes(N, K / 16);
  p.q_inter = fused ? (int)(N / 2) : 0;
  p.q_sf = reinterpret_cast<uint8_t*>(q_sf);
  p.q_gs = q_gs;
  // short K means short main loops: prefer the double-buffered narrow tile there, unless there are several
  // waves of wide tiles anyway (then halving the A re-reads and the tile count wins: 171 vs 183 us on
  // 81,920 rows x 2048 columns, K = 512)
  int bn = tile_n;
  if (bn == 0) {
    const long long wide_tiles = (long long)max_tiles * (N / 256);
    bn = (N % 256 == 0 && (K >= 2048 || wide_tiles >= 4LL * sm_count())) ? 256 : 128;
  }
  if (fused) bn = 256;
  const int kb = stage_kblocks();
  CUtensorMap ma, mb;
  if (!make_map(&ma, a_codes, (uint64_t)rows_capacity, (uint64_t)K / 2, kBM, kb * 32) ||
      !make_map(&mb, b_codes, (uint64_t)(E * N), (uint64_t)K / 2, fused ? 128u : (uint32_t)bn, kb * 32))
    return B200FP4_STATUS_INTERNAL_ERROR;
  grouped_tiles_kernel<<<1, 1024, 0, st>>>(expert_offsets, sf_offsets, (int)E, const_cast<int*>(p.g_hdr),
                                           const_cast<int4*>(p.g_mtiles), max_tiles);
  int rc = fused ? launch_gemm<256, 4, true, true>(ma, mb, p, max_tiles, st) : dispatch_gemm<true>(bn, kb, ma, mb, p, max_tiles, st);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  return finish_launch(2);
}

extern "C" int b200fp4_grouped_gemm_nvfp4(const void* a_codes, const void* b_codes, const void* a_sf, const void* b_sf,
                                          const float* alphas, const int32_t* expert_offsets, const int32_t* sf_offsets,
                                          void* out, int out_dtype, int64_t rows_capacity, int64_t N, int64_t K, int64_t E,
                                          int tile_n, void* workspace, size_t workspace_bytes, void* stream) {
  return grouped_gemm_impl(a_codes, b_codes, a_sf, b_sf, alphas, expert_offsets, sf_offsets, out, out_dtype, rows_capacity,
                           N, K, E, tile_n, workspace, workspace_bytes, stream, nullptr, nullptr);
}

extern "C" int b200fp4_grouped_gemm_nvfp4_silu_quant(const void* a_codes, const void* b_codes, const void* a_sf,
                                                     const void* b_sf, const float* alphas, const int32_t* expert_offsets,
                                                     const int32_t* sf_offsets, const float* out_global_scales,
                                                     int mid_dtype, void* out_codes, void* out_sf, int64_t rows_capacity,
                                                     int64_t N, int64_t K, int64_t E, void* workspace,
                                                     size_t workspace_bytes, void* stream) {
  if (!out_sf || !out_global_scales) return B200FP4_STATUS_INVALID_VALUE;
  return grouped_gemm_impl(a_codes, b_codes, a_sf, b_sf, alphas, expert_offsets, sf_offsets, out_codes, mid_dtype,
                           rows_capacity, N, K, E, 0, workspace, workspace_bytes, stream, out_sf, out_global_scales);
}

extern "C" int b200fp4_moe_permute(const int32_t* topk_ids, const int32_t* expert_map, int64_t global_E, int64_t M,
                                   int64_t topk, int64_t E, int32_t* expert_offsets, int32_t* blockscale_offsets,
                                   int32_t* dst2src, int32_t* src2dst, void* stream) {
  if (M < 0 || topk <= 0 || E <= 0 || E > kGroupMaxExperts || M * topk > (1 << 24)) return B200FP4_STATUS_INVALID_VALUE;
  if (!expert_offsets || !blockscale_offsets) return B200FP4_STATUS_INVALID_VALUE;
  if (M > 0 && (!topk_ids || !dst2src || !src2dst)) return B200FP4_STATUS_INVALID_VALUE;
  if (expert_map && global_E <= 0) return B200FP4_STATUS_INVALID_VALUE;
  const int P = (int)(M * topk);
  cudaStream_t st = (cudaStream_t)stream;
  if (P < kPermuteGridMinPairs) {
    moe_permute_kernel<<<1, 1024, 0, st>>>(topk_ids, P, expert_map, (int)global_E, (int)E, expert_offsets,
                                           blockscale_offsets, dst2src, src2dst);
    return finish_launch(1);
  }
  if (cudaMemsetAsync(expert_offsets, 0, (size_t)(E + 1) * sizeof(int32_t), st) != cudaSuccess)
    return B200FP4_STATUS_EXECUTION_FAILED;
  const int blocks = (P + kPermuteBlock - 1) / kPermuteBlock;
  moe_permute_count_kernel<<<blocks, kPermuteBlock, 0, st>>>(topk_ids, P, expert_map, (int)global_E, (int)E,
                                                             expert_offsets, dst2src, src2dst);
  moe_permute_scan_kernel<<<1, 1024, 0, st>>>((int)E, expert_offsets, blockscale_offsets);
  moe_permute_scatter_kernel<<<blocks, kPermuteBlock, 0, st>>>(P, (int)E, expert_offsets, dst2src, src2dst);
  moe_permute_shift_kernel<<<1, 1024, 0, st>>>((int)E, expert_offsets);
  return finish_launch(4);
}

extern "C" int b200fp4_shuffle_rows(const void* in, int64_t row_bytes, const int32_t* dst2src, int64_t n_dst,
                                    int64_t src_div, void* out, void* stream) {
  if (n_dst < 0 || row_bytes <= 0 || (row_bytes % 16) != 0 || src_div <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (n_dst == 0) return B200FP4_STATUS_SUCCESS;
  if (!in || !dst2src || !out || !aligned(in, 16) || !aligned(out, 16)) return B200FP4_STATUS_INVALID_VALUE;
  const int64_t total = n_dst * (row_bytes / 16);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 16 * (int64_t)sm_count()) blocks = 16 * (int64_t)sm_count();
  shuffle_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(in), dst2src, (int)src_div, row_bytes / 16, n_dst, reinterpret_cast<uint4*>(out));
  return finish_launch(1);
}

extern "C" int b200fp4_moe_unpermute_reduce(const void* expert_out, int dtype, const int32_t* src2dst,
                                            const float* topk_weights, int64_t M, int64_t topk, int64_t H, void* out,
                                            void* stream) {
  if (M < 0 || topk <= 0 || H <= 0 || (H % 2) != 0 || M > 65535) return B200FP4_STATUS_INVALID_VALUE;
  if (dtype != B200FP4_DTYPE_BF16 && dtype != B200FP4_DTYPE_F16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!expert_out || !src2dst || !topk_weights || !out) return B200FP4_STATUS_INVALID_VALUE;
  if ((H % 8) == 0 && aligned(expert_out, 16) && aligned(out, 16)) {
    dim3 grid8((unsigned)((H / 8 + 127) / 128), (unsigned)M);
    if (dtype == B200FP4_DTYPE_BF16)
      unpermute_reduce_vec8_kernel<__nv_bfloat16><<<grid8, 128, 0, (cudaStream_t)stream>>>(
          reinterpret_cast<const __nv_bfloat16*>(expert_out), src2dst, topk_weights, (int)M, (int)topk, (int)H,
          reinterpret_cast<__nv_bfloat16*>(out));
    else
      unpermute_reduce_vec8_kernel<__half><<<grid8, 128, 0, (cudaStream_t)stream>>>(
          reinterpret_cast<const __half*>(expert_out), src2dst, topk_weights, (int)M, (int)topk, (int)H,
          reinterpret_cast<__half*>(out));
    return finish_launch(1);
  }
  dim3 grid((unsigned)((H / 2 + 127) / 128), (unsigned)M);
  if (dtype == B200FP4_DTYPE_BF16)
    unpermute_reduce_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(expert_out), src2dst, topk_weights, (int)M, (int)topk, (int)H,
        reinterpret_cast<__nv_bfloat16*>(out));
  else
    unpermute_reduce_kernel<__half><<<grid, 128, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __half*>(expert_out), src2dst, topk_weights, (int)M, (int)topk, (int)H,
        reinterpret_cast<__half*>(out));
  return finish_launch(1);
}
