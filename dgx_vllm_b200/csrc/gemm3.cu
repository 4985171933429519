// Dense block-scaled NVFP4 GEMM for large M: one CTA computes a 256 x 224 output tile.
//
// Idea tested.  With 128 x 256 tiles (gemm.cu) every 128x256x64 MMA needs 12 KB of operands from L2.
// Here the CTA holds two 128-row halves of A and issues two MMAs per k-block against the same B
// tile: 15 KB of operands per two 128x224x64 MMAs, i.e. a third less L2 -> SM traffic per flop.  224
// (not 256) columns because the two accumulators take 2*BN of the 512 tensor-memory columns and the
// scale factors need the rest; 14336 / 224 = 64 also makes 1024 tiles = 6.9 waves of 148 SMs at
// M = 4096.  (Timing gemm.cu with its loads switched off later showed that operand traffic is not
// what limits it -- 144 us without loads against 154 us with them -- so the premise does not hold on
// B200; see the status note below.)
//
// Roles (14 warps): warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 epilogue (two per tensor-memory
// lane quarter: one per accumulator half), warps 10-13 scale factors.
//
// Scale factors.  Tensor memory has room for four k-blocks of scale factors (16 columns each: two
// 128-row tiles of A, two of B), one shared-memory stage's worth, so the slots are recycled per
// k-block: the MMA issuer commits after each k-block's pair of MMAs and the scale warps refill that
// slot for the next stage while the other three k-blocks run.  A tile's first B row, 224*nt, is a
// multiple of 32 but not of 128, so its rows straddle the 128-row tiles of the swizzled scale layout:
// three tiles are staged and every lane picks its four 4-byte groups (rows L, L+32, L+64, L+96 of the
// MMA's N index) out of two of them.
//
// Every wait is bounded and reports through the status word, as in gemm.cu.
//
// Status: correct on every tested shape (tile_n = 224), but slower on B200 as written: 175 us against
// 152 us at M=4096, N=14336, K=4096.  With only four scale slots a slot's refill (commit -> scale warps
// -> tcgen05.st -> barrier -> MMA issuer, ~3-4 k cycles measured) has to fit into three k-blocks of
// MMAs (~700 cycles), so the tensor pipe waits for scale factors.  Opt-in, never chosen automatically.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/b200_nvfp4.h"
#include "sm100_ptx.cuh"

namespace b200fp4 {
namespace {

constexpr int kTallBM = 256;
constexpr int kTallBN = 224;
constexpr int kTallKB = 4;                      // 64-wide k-blocks per stage (128-byte rows)
constexpr int kTallThreads = 448;
constexpr int kTallStages = 3;
constexpr int kTallStageA = kTallBM * 128;      // 32 KiB
constexpr int kTallStageB = kTallBN * 128;      // 28 KiB
constexpr int kTallStageSFA = 2 * kTallKB * 512;
constexpr int kTallStageSFB = 3 * kTallKB * 512;
constexpr int kTallStageBytes = kTallStageA + kTallStageB + kTallStageSFA + kTallStageSFB;   // 70 KiB
constexpr int kTallSmemBytes = kTallStages * kTallStageBytes + 1024 + 1024;
constexpr uint32_t kTallSfBase = 2 * kTallBN;   // tensor-memory column of the first scale slot
constexpr int kTallSlots = 4;                   // scale slots of 16 columns: A lo, A hi, B tile 0, B tile 1
constexpr uint32_t kTallIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(kTallBN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
static_assert(kTallSfBase + kTallSlots * 16 <= 512, "tensor memory budget");
static_assert(kTallStageBytes % 1024 == 0, "stages keep the 1024-byte alignment of the swizzle atoms");

struct TallParams {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha;
  void* out;
  int out_bf16;
  int M, N, K;
  int m_tiles, n_tiles, k_stages;
  int* status;
};

__global__ void __launch_bounds__(kTallThreads, 1)
    nvfp4_gemm_tall_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const TallParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kTallStages * kTallStageBytes);
  uint64_t* full_bar = bars;                         // operands of the stage have landed
  uint64_t* empty_bar = full_bar + kTallStages;      // the stage's MMAs have read it
  uint64_t* sf_full = empty_bar + kTallStages;       // scale factors of the stage have landed
  uint64_t* sf_ready = sf_full + kTallStages;        // [slot] scale factors are in tensor memory
  uint64_t* sf_free = sf_ready + kTallSlots;         // [slot] the MMAs that used the slot are done
  uint64_t* acc_full = sf_free + kTallSlots;         // both accumulators hold a finished tile
  uint64_t* acc_empty = acc_full + 1;                // [half] drained by its four epilogue warps
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles_total = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTallStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_full[s]), 1);
    }
    for (int s = 0; s < kTallSlots; ++s) {
      mbar_init(smem_u32(&sf_ready[s]), 4);
      mbar_init(smem_u32(&sf_free[s]), 1);
    }
    mbar_init(smem_u32(&acc_full[0]), 1);
    mbar_init(smem_u32(&acc_empty[0]), 4);
    mbar_init(smem_u32(&acc_empty[1]), 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr_smem)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const int KT = (p.K + 63) / 64;
  const int sfa_tiles_total = (p.M + 127) / 128, sfb_tiles_total = (p.N + 127) / 128;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
        const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
        const int n0 = nt * kTallBN, sfb_t0 = n0 / 128;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kTallStages, ph = (it / kTallStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, 1)) { ok = false; break; }
          unsigned char* st = smem + (size_t)s * kTallStageBytes;
          const int kblocks = min(kTallKB, KT - ks * kTallKB);
          int n_sf = 0;
          for (int j = 0; j < 2; ++j) n_sf += (2 * mt + j < sfa_tiles_total) ? 1 : 0;
          for (int j = 0; j < 3; ++j) n_sf += (sfb_t0 + j < sfb_tiles_total) ? 1 : 0;
          const uint32_t sbar = smem_u32(&sf_full[s]);
          mbar_expect_tx(sbar, (uint32_t)(kblocks * 512 * n_sf));
          unsigned char* sf = st + kTallStageA + kTallStageB;
          for (int j = 0; j < 2; ++j)
            if (2 * mt + j < sfa_tiles_total)
              bulk_load_1d(smem_u32(sf + j * (kTallKB * 512)), p.sfa + ((size_t)(2 * mt + j) * KT + (size_t)ks * kTallKB) * 512,
                           (uint32_t)kblocks * 512, sbar);
          for (int j = 0; j < 3; ++j)
            if (sfb_t0 + j < sfb_tiles_total)
              bulk_load_1d(smem_u32(sf + kTallStageSFA + j * (kTallKB * 512)),
                           p.sfb + ((size_t)(sfb_t0 + j) * KT + (size_t)ks * kTallKB) * 512, (uint32_t)kblocks * 512, sbar);
          const uint32_t bar = smem_u32(&full_bar[s]);
          mbar_expect_tx(bar, (uint32_t)(kTallStageA + kTallStageB));
          tma_load_2d(smem_u32(st), &map_a, ks * 128, mt * kTallBM, bar);
          tma_load_2d(smem_u32(st + kTallStageA), &map_b, ks * 128, n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, g = 0, tcount = 0;   // stage counter, k-block (scale slot) counter, tile counter
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x, ++tcount) {
        const uint32_t aph = tcount & 1;
        if (!mbar_wait(smem_u32(&acc_empty[0]), aph ^ 1, p.status, 2)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&acc_empty[1]), aph ^ 1, p.status, 2)) { ok = false; break; }
        tcgen05_fence_after();
        for (int ks = 0; ok && ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kTallStages, ph = (it / kTallStages) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, p.status, 3)) { ok = false; break; }
          tcgen05_fence_after();
          unsigned char* st = smem + (size_t)s * kTallStageBytes;
          const int kblocks = min(kTallKB, KT - ks * kTallKB);
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + kTallStageA);
          for (int kb = 0; kb < kblocks; ++kb, ++g) {
            const uint32_t slot = g % kTallSlots, sph = (g / kTallSlots) & 1;
            if (!mbar_wait(smem_u32(&sf_ready[slot]), sph, p.status, 5)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t sf_t = tmem_base + kTallSfBase + slot * 16;
            const uint64_t b_desc = desc_kmajor<128>(b_addr + kb * 32);
            const uint32_t accum = (ks > 0 || kb > 0) ? 1u : 0u;
            tcgen05_mma_nvf4(tmem_base, desc_kmajor<128>(a_addr + kb * 32), b_desc, kTallIdesc, sf_t, sf_t + 8, accum);
            tcgen05_mma_nvf4(tmem_base + kTallBN, desc_kmajor<128>(a_addr + 128 * 128 + kb * 32), b_desc, kTallIdesc, sf_t + 4,
                             sf_t + 8, accum);
            tcgen05_commit(smem_u32(&sf_free[slot]));
          }
          if (ok) tcgen05_commit(smem_u32(&empty_bar[s]));
        }
        if (ok) tcgen05_commit(smem_u32(&acc_full[0]));
      }
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------------ scale factors (warps 10..13)
    const int quarter = warp & 3;
    uint32_t it = 0, g = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
      const int nt = tile / p.m_tiles;
      const int rot = ((nt * kTallBN) >> 5) & 3;     // first B row of the tile, in 32-row groups, inside its 128-row scale tile
      for (int ks = 0; ok && ks < p.k_stages; ++ks, ++it) {
        const uint32_t s = it % kTallStages, ph = (it / kTallStages) & 1;
        ok = mbar_wait(smem_u32(&sf_full[s]), ph, p.status, 6);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const unsigned char* sf = smem + (size_t)s * kTallStageBytes + kTallStageA + kTallStageB;
        const int kblocks = min(kTallKB, KT - ks * kTallKB);
        for (int kb = 0; kb < kblocks; ++kb, ++g) {
          const uint32_t slot = g % kTallSlots, sph = (g / kTallSlots) & 1;
          // operand bytes first, so that the loads overlap the wait for the slot
          const uint4 a_lo = *reinterpret_cast<const uint4*>(sf + kb * 512 + lane * 16);
          const uint4 a_hi = *reinterpret_cast<const uint4*>(sf + (kTallKB + kb) * 512 + lane * 16);
          uint32_t w[12];
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            const uint4 v = *reinterpret_cast<const uint4*>(sf + kTallStageSFA + (j * kTallKB + kb) * 512 + lane * 16);
            w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
          }
          // lane L holds rows L, L+32, L+64, L+96 of every 128-row tile as words 0..3; the MMA's N rows
          // 128*j + L + 32*i are words rot + 4*j + i of the staged run of three tiles
          uint4 b0, b1;
          if (rot == 0) { b0 = make_uint4(w[0], w[1], w[2], w[3]); b1 = make_uint4(w[4], w[5], w[6], w[7]); }
          else if (rot == 1) { b0 = make_uint4(w[1], w[2], w[3], w[4]); b1 = make_uint4(w[5], w[6], w[7], w[8]); }
          else if (rot == 2) { b0 = make_uint4(w[2], w[3], w[4], w[5]); b1 = make_uint4(w[6], w[7], w[8], w[9]); }
          else { b0 = make_uint4(w[3], w[4], w[5], w[6]); b1 = make_uint4(w[7], w[8], w[9], w[10]); }
          ok = mbar_wait(smem_u32(&sf_free[slot]), sph ^ 1, p.status, 7);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + kTallSfBase + slot * 16;
          tcgen05_st_32x32_x4(t0, a_lo);
          tcgen05_st_32x32_x4(t0 + 4, a_hi);
          tcgen05_st_32x32_x4(t0 + 8, b0);
          tcgen05_st_32x32_x4(t0 + 12, b1);
          tcgen05_wait_st();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sf_ready[slot]));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;                 // tensor-memory lanes [32*quarter, +32) belong to this warp
    const int half = (warp - 2) >> 2;             // which accumulator (128-row half of the tile)
    const float alpha = p.alpha[0];
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x, ++tcount) {
      const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
      const int n0 = nt * kTallBN;
      ok = mbar_wait(smem_u32(&acc_full[0]), tcount & 1, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = mt * kTallBM + half * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * kTallBN;
      uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.out) + (size_t)row * p.N;
#pragma unroll 1
      for (int c = 0; c < kTallBN / 32; ++c) {
        uint32_t r[32];
        tcgen05_ld_32x32(taddr + c * 32, r);
        tcgen05_wait_ld();
        if (c == kTallBN / 32 - 1) {
          // the accumulator half is in registers: hand it back before the last stores
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&acc_empty[half]));
        }
        uint32_t packed[16];
        if (p.out_bf16) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * i]) * alpha, __uint_as_float(r[2 * i + 1]) * alpha);
            packed[i] = *reinterpret_cast<uint32_t*>(&v);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __half2 v = __floats2half2_rn(__uint_as_float(r[2 * i]) * alpha, __uint_as_float(r[2 * i + 1]) * alpha);
            packed[i] = *reinterpret_cast<uint32_t*>(&v);
          }
        }
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          uint16_t* dst = dst_row + col0;
          if (col0 + 32 <= p.N && (p.N % 8) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4*>(dst)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) dst[i] = (uint16_t)((i & 1) ? (packed[i >> 1] >> 16) : (packed[i >> 1] & 0xFFFFu));
          }
        }
      }
    }
  }
  // all roles fall through to here (also after a timed-out wait), so tensor memory is always freed
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

int launch_gemm_tall(const CUtensorMap& ma, const CUtensorMap& mb, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                     void* out, int out_bf16, int M, int N, int K, int* status, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(nvfp4_gemm_tall_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTallSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  TallParams p;
  p.sfa = sfa;
  p.sfb = sfb;
  p.alpha = alpha;
  p.out = out;
  p.out_bf16 = out_bf16;
  p.M = M;
  p.N = N;
  p.K = K;
  p.m_tiles = (M + kTallBM - 1) / kTallBM;
  p.n_tiles = (N + kTallBN - 1) / kTallBN;
  p.k_stages = (K + kTallKB * 64 - 1) / (kTallKB * 64);
  p.status = status;
  long long grid = (long long)p.m_tiles * p.n_tiles;
  if (grid > sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  nvfp4_gemm_tall_kernel<<<(unsigned)grid, kTallThreads, kTallSmemBytes, st>>>(ma, mb, p);
  return B200FP4_STATUS_SUCCESS;
}

}  // namespace b200fp4
