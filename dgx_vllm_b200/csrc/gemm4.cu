// Dense block-scaled NVFP4 GEMM with the epilogue hidden behind the next tile: 128 x 192 output
// tiles and two accumulators in tensor memory.
//
// Why this shape.  Timing the 128 x 256 kernel of gemm.cu with its loads switched off gave
// time = tiles * (4.1 us + 0.109 us per 128x256x64 MMA) on B200: the tensor pipe runs close to what
// the power-limited clock allows, but every tile pays ~4 us during which the pipe idles while the
// single 256-column accumulator is drained (two of them would fill all 512 tensor-memory columns
// and leave none for the scale factors).  With 192 columns two accumulators take 384 columns, the
// MMAs of tile i+1 run while tile i is drained, and 128 columns remain for scale factors.
//
// Roles (10 warps): warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue, warps 6-9 scale
// factors.
//
// Scale factors.  The 128 spare tensor-memory columns hold eight k-blocks of scale factors (12
// columns each: one 128-row tile of A, two of B), i.e. two of the four shared-memory stages, so the
// slots are recycled per k-block: the MMA issuer commits after every MMA and the scale warps refill
// a slot as soon as the MMA that used it has finished.  A tile's first B row, 192*nt, is a multiple
// of 64 but not of 128, so its rows straddle the 128-row tiles of the swizzled scale layout: three
// tiles are staged and every lane picks its four 4-byte groups (rows L, L+32, L+64, L+96 of the
// MMA's N index) out of two of them.
//
// Every wait is bounded and reports through the status word, as in gemm.cu.
//
// Status: correct on every tested shape (tile_n = 192), but slower on B200 as written: 274 us against
// 152 us at M=4096, N=14336, K=4096.  Recycling a scale slot takes ~3-4 k cycles (commit -> scale warps
// -> tcgen05.st -> barrier -> MMA issuer) and eight slots cover only ~800 cycles of MMAs, so the
// tensor pipe waits for scale factors.  Opt-in, never chosen automatically.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/b200_nvfp4.h"
#include "sm100_ptx.cuh"

namespace b200fp4 {
namespace {

constexpr int kOvBM = 128;
constexpr int kOvBN = 192;
constexpr int kOvKB = 4;                      // 64-wide k-blocks per stage (128-byte rows)
constexpr int kOvThreads = 320;
constexpr int kOvStages = 4;
constexpr int kOvStageA = kOvBM * 128;      // 16 KiB
constexpr int kOvStageB = kOvBN * 128;      // 24 KiB
constexpr int kOvStageSFA = 1 * kOvKB * 512;
constexpr int kOvStageSFB = 3 * kOvKB * 512;
constexpr int kOvStageBytes = kOvStageA + kOvStageB + kOvStageSFA + kOvStageSFB;   // 48 KiB
constexpr int kOvSmemBytes = kOvStages * kOvStageBytes + 1024 + 1024;
constexpr uint32_t kOvSfBase = 2 * kOvBN;   // tensor-memory column of the first scale slot
constexpr int kOvSlots = 8;                   // scale slots of 12 columns: A, B tile 0, B tile 1
constexpr int kOvSlotCols = 12;
constexpr uint32_t kOvIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(kOvBN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
static_assert(kOvSfBase + kOvSlots * kOvSlotCols <= 512, "tensor memory budget");
static_assert(kOvStageBytes % 1024 == 0, "stages keep the 1024-byte alignment of the swizzle atoms");

struct OvParams {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha;
  void* out;
  int out_bf16;
  int M, N, K;
  int m_tiles, n_tiles, k_stages;
  int* status;
};

__global__ void __launch_bounds__(kOvThreads, 1)
    nvfp4_gemm_overlap_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const OvParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kOvStages * kOvStageBytes);
  uint64_t* full_bar = bars;                         // operands of the stage have landed
  uint64_t* empty_bar = full_bar + kOvStages;      // the stage's MMAs have read it
  uint64_t* sf_full = empty_bar + kOvStages;       // scale factors of the stage have landed
  uint64_t* sf_ready = sf_full + kOvStages;        // [slot] scale factors are in tensor memory
  uint64_t* sf_free = sf_ready + kOvSlots;         // [slot] the MMAs that used the slot are done
  uint64_t* acc_full = sf_free + kOvSlots;         // [acc] the accumulator holds a finished tile
  uint64_t* acc_empty = acc_full + 2;                // [acc] drained by the four epilogue warps
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles_total = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kOvStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_full[s]), 1);
    }
    for (int s = 0; s < kOvSlots; ++s) {
      mbar_init(smem_u32(&sf_ready[s]), 4);
      mbar_init(smem_u32(&sf_free[s]), 1);
    }
    mbar_init(smem_u32(&acc_full[0]), 1);
    mbar_init(smem_u32(&acc_full[1]), 1);
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
        const int n0 = nt * kOvBN, sfb_t0 = n0 / 128;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kOvStages, ph = (it / kOvStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, 1)) { ok = false; break; }
          unsigned char* st = smem + (size_t)s * kOvStageBytes;
          const int kblocks = min(kOvKB, KT - ks * kOvKB);
          int n_sf = 0;
          n_sf += (mt < sfa_tiles_total) ? 1 : 0;
          for (int j = 0; j < 3; ++j) n_sf += (sfb_t0 + j < sfb_tiles_total) ? 1 : 0;
          const uint32_t sbar = smem_u32(&sf_full[s]);
          mbar_expect_tx(sbar, (uint32_t)(kblocks * 512 * n_sf));
          unsigned char* sf = st + kOvStageA + kOvStageB;
          if (mt < sfa_tiles_total)
            bulk_load_1d(smem_u32(sf), p.sfa + ((size_t)mt * KT + (size_t)ks * kOvKB) * 512, (uint32_t)kblocks * 512, sbar);
          for (int j = 0; j < 3; ++j)
            if (sfb_t0 + j < sfb_tiles_total)
              bulk_load_1d(smem_u32(sf + kOvStageSFA + j * (kOvKB * 512)),
                           p.sfb + ((size_t)(sfb_t0 + j) * KT + (size_t)ks * kOvKB) * 512, (uint32_t)kblocks * 512, sbar);
          const uint32_t bar = smem_u32(&full_bar[s]);
          mbar_expect_tx(bar, (uint32_t)(kOvStageA + kOvStageB));
          tma_load_2d(smem_u32(st), &map_a, ks * 128, mt * kOvBM, bar);
          tma_load_2d(smem_u32(st + kOvStageA), &map_b, ks * 128, n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, g = 0, tcount = 0;   // stage counter, k-block (scale slot) counter, tile counter
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        if (!mbar_wait(smem_u32(&acc_empty[acc]), aph ^ 1, p.status, 2)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kOvBN;
        for (int ks = 0; ok && ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kOvStages, ph = (it / kOvStages) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, p.status, 3)) { ok = false; break; }
          tcgen05_fence_after();
          unsigned char* st = smem + (size_t)s * kOvStageBytes;
          const int kblocks = min(kOvKB, KT - ks * kOvKB);
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + kOvStageA);
          for (int kb = 0; kb < kblocks; ++kb, ++g) {
            const uint32_t slot = g % kOvSlots, sph = (g / kOvSlots) & 1;
            if (!mbar_wait(smem_u32(&sf_ready[slot]), sph, p.status, 5)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t sf_t = tmem_base + kOvSfBase + slot * kOvSlotCols;
            tcgen05_mma_nvf4(d_tmem, desc_kmajor<128>(a_addr + kb * 32), desc_kmajor<128>(b_addr + kb * 32), kOvIdesc, sf_t,
                             sf_t + 4, (ks > 0 || kb > 0) ? 1u : 0u);
            tcgen05_commit(smem_u32(&sf_free[slot]));
          }
          if (ok) tcgen05_commit(smem_u32(&empty_bar[s]));
        }
        if (ok) tcgen05_commit(smem_u32(&acc_full[acc]));
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ scale factors (warps 6..9)
    const int quarter = warp & 3;
    uint32_t it = 0, g = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
      const int nt = tile / p.m_tiles;
      const int rot = ((nt * kOvBN) >> 5) & 3;     // first B row of the tile, in 32-row groups, inside its 128-row scale tile
      for (int ks = 0; ok && ks < p.k_stages; ++ks, ++it) {
        const uint32_t s = it % kOvStages, ph = (it / kOvStages) & 1;
        ok = mbar_wait(smem_u32(&sf_full[s]), ph, p.status, 6);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const unsigned char* sf = smem + (size_t)s * kOvStageBytes + kOvStageA + kOvStageB;
        const int kblocks = min(kOvKB, KT - ks * kOvKB);
        for (int kb = 0; kb < kblocks; ++kb, ++g) {
          const uint32_t slot = g % kOvSlots, sph = (g / kOvSlots) & 1;
          // operand bytes first, so that the loads overlap the wait for the slot
          const uint4 a_lo = *reinterpret_cast<const uint4*>(sf + kb * 512 + lane * 16);
          uint32_t w[12];
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            const uint4 v = *reinterpret_cast<const uint4*>(sf + kOvStageSFA + (j * kOvKB + kb) * 512 + lane * 16);
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
          const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + kOvSfBase + slot * kOvSlotCols;
          tcgen05_st_32x32_x4(t0, a_lo);
          tcgen05_st_32x32_x4(t0 + 4, b0);
          tcgen05_st_32x32_x4(t0 + 8, b1);
          tcgen05_wait_st();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sf_ready[slot]));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;                 // tensor-memory lanes [32*quarter, +32) belong to this warp
    const float alpha = p.alpha[0];
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x, ++tcount) {
      const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
      const int n0 = nt * kOvBN;
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      ok = mbar_wait(smem_u32(&acc_full[acc]), aph, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = mt * kOvBM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kOvBN;
      uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.out) + (size_t)row * p.N;
#pragma unroll 1
      for (int c = 0; c < kOvBN / 32; ++c) {
        uint32_t r[32];
        tcgen05_ld_32x32(taddr + c * 32, r);
        tcgen05_wait_ld();
        if (c == kOvBN / 32 - 1) {
          // the whole accumulator has been read: hand it back before the last stores
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
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

int launch_gemm_overlap(const CUtensorMap& ma, const CUtensorMap& mb, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                     void* out, int out_bf16, int M, int N, int K, int* status, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(nvfp4_gemm_overlap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kOvSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  OvParams p;
  p.sfa = sfa;
  p.sfb = sfb;
  p.alpha = alpha;
  p.out = out;
  p.out_bf16 = out_bf16;
  p.M = M;
  p.N = N;
  p.K = K;
  p.m_tiles = (M + kOvBM - 1) / kOvBM;
  p.n_tiles = (N + kOvBN - 1) / kOvBN;
  p.k_stages = (K + kOvKB * 64 - 1) / (kOvKB * 64);
  p.status = status;
  long long grid = (long long)p.m_tiles * p.n_tiles;
  if (grid > sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  nvfp4_gemm_overlap_kernel<<<(unsigned)grid, kOvThreads, kOvSmemBytes, st>>>(ma, mb, p);
  return B200FP4_STATUS_SUCCESS;
}

}  // namespace b200fp4
