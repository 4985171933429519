// Dense block-scaled NVFP4 GEMM on CTA pairs: tcgen05.mma.cta_group::2, tile 256 (M) x 256 (N) per pair.
//
// Same roles and data formats as the single-CTA kernel (gemm.cu).  Two CTAs of a cluster share
// one MMA: each stages its own 128 rows of A and HALF of the B tile (128 of the 256 rows), so a CTA
// moves 32 KiB of operands per 256-k stage instead of 48 KiB.  The single-CTA main loop is bound by
// bytes in flight x L2 latency; cutting the bytes per MMA by a third is what this kernel is for.
//   * every CTA's TMA loads (its operands and the scale factors of its own A rows and of all 256 B
//     rows; no multicast) complete on its own `full` barrier; its four scale warps then copy the scales
//     into its own tensor memory with tcgen05.st and arrive once per warp -- remotely, for the peer --
//     on the leader's `sf_ready` barrier, which therefore also tells the leader that the peer's
//     operands have landed;
//   * the leader's MMA thread issues the MMAs for both CTAs; tcgen05.commit with a CTA mask releases
//     the stage (`empty`) and publishes the accumulator (`acc_full`) in both CTAs at once;
//   * each CTA's epilogue drains its own 128 accumulator rows and arrives on the leader's `acc_empty`.
// All waits are bounded and report through the status word; the pair leaves through a cluster barrier
// so neither CTA frees tensor memory or exits while the other may still touch it.
//
// Status: correct on every shape the single-CTA kernel is tested on, but slower on B200 as written
// (M=4096, N=14336, K=4096: 260 us against 150 us).  With the MMAs removed it still takes 250 us, i.e.
// the stage loop itself is latency-bound: remote barrier arrivals and the commit that releases both
// CTAs lengthen the empty -> load -> scales -> MMA -> commit chain while only five stages fit.  It is
// therefore opt-in (tile_n = 512) and not chosen automatically.
#include "sm100_ptx.cuh"

namespace b200fp4 {
namespace {

constexpr int kThreads2 = 320;          // warp 0 TMA, warp 1 MMA/alloc, warps 2-5 epilogue, warps 6-9 scale factors
constexpr int kStages2 = 5;
constexpr int kStageA2 = 128 * 128;     // 128 rows x 128 bytes (256 k)
constexpr int kStageB2 = 128 * 128;     // this CTA's half of the 256-row B tile
constexpr int kStageSFA2 = 4 * 512;
constexpr int kStageSFB2 = 2 * 4 * 512;
constexpr int kStageBytes2 = kStageA2 + kStageB2 + kStageSFA2 + kStageSFB2;   // 38 KiB
constexpr uint32_t kSfCols2 = 16 + 32;
constexpr uint32_t kSfBase2 = 256;      // accumulator: columns [0, 256)
static_assert(kSfBase2 + kStages2 * kSfCols2 <= 512, "tensor memory budget");
constexpr int kBarBytes2 = 1024;
constexpr size_t kSmemBytes2 = (size_t)kStages2 * kStageBytes2 + 1024 + kBarBytes2;
// E2M1 x E2M1, UE4M3 scales, K-major, N = 256, M = 256 (pair), dense K = 64
constexpr uint32_t kIdesc2 = (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

struct Gemm2Params {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha;
  void* out;
  int out_bf16;
  int M, N, K;
  int m_pairs, n_tiles, k_stages;
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(cta_mask)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                      uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
    nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const Gemm2Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStages2 * kStageBytes2);
  uint64_t* full_bar = bars;                     // local: this CTA's operands and scale factors have landed
  uint64_t* empty_bar = bars + 2 * kStages2;     // local: stage may be refilled (MMAs done)
  uint64_t* sf_ready = bars + 3 * kStages2;      // leader's: both CTAs' scales are in tensor memory
  uint64_t* acc_full = bars + 4 * kStages2;      // local: accumulator complete
  uint64_t* acc_empty = acc_full + 1;            // leader's: both epilogues have drained
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_empty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int n_pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
  const int n_tiles_total = p.m_pairs * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_ready[s]), 8);       // one arrival per scale warp of both CTAs
    }
    mbar_init(smem_u32(acc_full), 1);
    mbar_init(smem_u32(acc_empty), 8);            // one arrival per epilogue warp of both CTAs
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr_smem)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  cluster_sync_all();          // barriers of both CTAs are initialised before anyone signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const int KT = (p.K + 63) / 64;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs) {
        const int mp = tile % p.m_pairs, nt = tile / p.m_pairs;
        const int a_row0 = mp * 256 + (int)rank * 128, b_row0 = nt * 256 + (int)rank * 128;
        const int sfa_tile = mp * 2 + (int)rank;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kStages2, ph = (it / kStages2) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, 11)) { ok = false; break; }
          unsigned char* st = smem + (size_t)s * kStageBytes2;
          const int kblocks = min(4, KT - ks * 4);
          int sf_tiles = 0;
          for (int j = 0; j < 2; ++j) sf_tiles += ((nt * 2 + j) * 128 < p.N) ? 1 : 0;
          // everything this CTA stages for the stage lands on its own barrier
          const uint32_t sfbar = smem_u32(&full_bar[s]);
          const bool sfa_ok = sfa_tile * 128 < p.M;      // the peer's A rows may lie entirely past M
          mbar_expect_tx(sfbar, (uint32_t)(kStageA2 + kStageB2 + kblocks * 512 * ((sfa_ok ? 1 : 0) + sf_tiles)));
          tma_load_2d(smem_u32(st), &map_a, ks * 128, a_row0, sfbar);
          tma_load_2d(smem_u32(st + kStageA2), &map_b, ks * 128, b_row0, sfbar);
          if (sfa_ok)
            bulk_load_1d(smem_u32(st + kStageA2 + kStageB2), p.sfa + ((size_t)sfa_tile * KT + (size_t)ks * 4) * 512,
                         (uint32_t)kblocks * 512, sfbar);
          for (int j = 0; j < sf_tiles; ++j)
            bulk_load_1d(smem_u32(st + kStageA2 + kStageB2 + kStageSFA2 + j * 2048),
                         p.sfb + ((size_t)(nt * 2 + j) * KT + (size_t)ks * 4) * 512, (uint32_t)kblocks * 512, sfbar);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs, ++tcount) {
        if (!mbar_wait(smem_u32(acc_empty), (tcount & 1) ^ 1, p.status, 12)) { ok = false; break; }
        tcgen05_fence_after();
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kStages2, ph = (it / kStages2) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, p.status, 13)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&sf_ready[s]), ph, p.status, 15)) { ok = false; break; }
          tcgen05_fence_after();
          unsigned char* st = smem + (size_t)s * kStageBytes2;
          const int kblocks = min(4, KT - ks * 4);
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + kStageA2);
          const uint32_t sfa_tmem = tmem_base + kSfBase2 + s * kSfCols2, sfb_tmem = sfa_tmem + 16;
          for (int kb = 0; kb < kblocks; ++kb)
            tcgen05_mma_nvf4_pair(tmem_base, desc_kmajor<128>(a_addr + kb * 32), desc_kmajor<128>(b_addr + kb * 32), kIdesc2,
                                  sfa_tmem + kb * 4, sfb_tmem + kb * 8, (ks > 0 || kb > 0) ? 1u : 0u);
          tcgen05_commit_pair(smem_u32(&empty_bar[s]), 3);     // both CTAs may refill this stage
        }
        if (ok) tcgen05_commit_pair(smem_u32(acc_full), 3);     // both epilogues may start
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ scale factors (both CTAs)
    const int quarter = warp & 3;
    const uint32_t ready_leader_base = map_to_cta(smem_u32(&sf_ready[0]), 0);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs) {
      for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
        const uint32_t s = it % kStages2, ph = (it / kStages2) & 1;
        ok = mbar_wait(smem_u32(&full_bar[s]), ph, p.status, 16);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const unsigned char* sf = smem + (size_t)s * kStageBytes2 + kStageA2 + kStageB2;
        const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + kSfBase2 + s * kSfCols2;
        const int kblocks = min(4, KT - ks * 4);
        for (int kb = 0; kb < kblocks; ++kb) {
          tcgen05_st_32x32_x4(t0 + kb * 4, *reinterpret_cast<const uint4*>(sf + kb * 512 + lane * 16));
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tcgen05_st_32x32_x4(t0 + 16 + kb * 8 + j * 4,
                                *reinterpret_cast<const uint4*>(sf + kStageSFA2 + j * 2048 + kb * 512 + lane * 16));
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(ready_leader_base + s * 8);   // remote arrivals are costly: one per warp
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, warps 2..5)
    const int quarter = warp & 3;
    const float alpha = p.alpha[0];
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(acc_empty), 0);
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs, ++tcount) {
      const int mp = tile % p.m_pairs, nt = tile / p.m_pairs;
      ok = mbar_wait(smem_u32(acc_full), tcount & 1, p.status, 14);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = mp * 256 + (int)rank * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      uint32_t packed[128];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t r[32];
        tcgen05_ld_32x32(taddr + c * 32, r);
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
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      if (row < p.M) {
        uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.out) + (size_t)row * p.N;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int col0 = nt * 256 + c * 32;
          if (col0 < p.N) {
            uint16_t* dst = dst_row + col0;
            if (col0 + 32 <= p.N && (p.N % 8) == 0) {
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
  // every role of both CTAs ends here, also after an expired wait
  tcgen05_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

// Launches the CTA-pair kernel.  Tensor maps: A box = 128 rows, B box = 128 rows, 128-byte rows.
int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                     void* out, int out_bf16, int M, int N, int K, int* status, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(nvfp4_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes2) !=
        cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  Gemm2Params p;
  p.sfa = sfa; p.sfb = sfb; p.alpha = alpha; p.out = out; p.out_bf16 = out_bf16;
  p.M = M; p.N = N; p.K = K;
  p.m_pairs = (M + 255) / 256;
  p.n_tiles = (N + 255) / 256;
  p.k_stages = (K + 255) / 256;
  p.status = status;
  long long pairs = (long long)p.m_pairs * p.n_tiles;
  const int max_pairs = sm_count() / 2;
  if (pairs > max_pairs) pairs = max_pairs;
  if (pairs < 1) pairs = 1;
  nvfp4_gemm_pair_kernel<<<(unsigned)(2 * pairs), kThreads2, kSmemBytes2, st>>>(ma, mb, p);
  return B200FP4_STATUS_SUCCESS;
}

}  // namespace b200fp4
