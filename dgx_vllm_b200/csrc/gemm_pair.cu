// Dense block-scaled NVFP4 GEMM on CTA pairs: tcgen05.mma.cta_group::2, one 256 (M) x 256 (N) tile per pair of SMs.
//
// Why pairs: a single CTA's MMA (128 x 256 x 64) reads 4 KiB of A and 8 KiB of B from shared memory and issues at about
// 206 cycles per MMA.  In a pair each CTA holds its own 128 rows of A and HALF of the B tile (128 of the 256 rows): 8 KiB
// per CTA per MMA for the same work per SM, and a third fewer operand bytes from L2.  Measured: a 256 x 256 x 64 MMA of
// the pair issues every 176 cycles; M=4096, N=14336, K=4096 takes about 200 k cycles against 223 k for the single-CTA
// kernel (123 us against 129 us: the SM clock settles near 1.6-1.7 GHz under either).
//
// Roles per CTA (23 warps): warp 0 loads operands, warp 1 issues the MMAs (leader CTA only) and owns tensor memory,
// warps 2-5, 10-13 and 15-22 drain and store the CTA's 128 accumulator rows (four warps per tensor-memory lane quarter, 64
// columns each: the one accumulator is handed back after two tcgen05.ld per warp), warps 6-9 move scale factors from
// shared memory into tensor memory, warp 14 loads scale factors.
//
// What keeps the stage loop short (a stage = 256 k = 4 MMAs = about 700 cycles, less than the latency of a load, so
// every hop between "stage free" and "stage ready" counts):
//   * the operand loads of BOTH CTAs complete on the LEADER's `full` barrier (the cta_group::2 form of the tensor copy
//     takes a barrier of the peer CTA), so the MMA thread learns that the peer's half has landed without a software hop;
//   * tcgen05.commit with a CTA mask frees the stage (`empty`) and publishes the accumulator (`acc_full`) in both CTAs;
//   * scale factors have their own, deeper ring in shared memory (10 stages of 6 KiB, loaded well ahead of the operands),
//     so that when a scale slot of tensor memory frees up its data is already on chip: the scale warps copy it with
//     three 16-column tcgen05.st and arrive on the leader's `sf_ready` (remotely from the peer);
//   * arrivals on a barrier of the other CTA are RELAXED at cluster scope: with release semantics each one stalled the
//     arriving warp for about 1100 cycles and the whole kernel ran at one stage per 2000 cycles (242 us).
// Where the cycles of the MMA thread go (M=4096, per pair): issuing 75 %, waiting for scales 10 %, for operands 7 %, for
// the single accumulator to be drained 8 %.
// No copy uses cluster multicast.  Every wait is bounded and reports through the status word; the pair leaves through a
// cluster barrier so neither CTA frees tensor memory or exits while the other may still signal it.
#include "sm100_ptx.cuh"

namespace b200fp4 {
namespace {

constexpr int kPairThreads = 736;
constexpr int kPStages = 5;                        // operand ring
constexpr int kPSfStages = 10;                     // scale-factor ring (shared memory)
constexpr int kPStageA = 128 * 128;                // 128 rows x 128 bytes (256 k)
constexpr int kPStageB = 128 * 128;                // this CTA's half of the 256-row B tile
constexpr int kPStageOp = kPStageA + kPStageB;     // 32 KiB
constexpr int kPSfA = 4 * 512;
constexpr int kPSfB = 2 * 4 * 512;
constexpr int kPSfStage = kPSfA + kPSfB;           // 6 KiB
constexpr uint32_t kPSfCols = 16 + 32;             // tensor-memory columns of one stage's scales (A: 4 per k-block, B: 8)
constexpr uint32_t kPSfBase = 256;                 // accumulator: columns [0, 256)
static_assert(kPSfBase + kPStages * kPSfCols <= 512, "tensor memory budget");
constexpr int kPBarBytes = 512;
constexpr size_t kPairSmemBytes = (size_t)kPStages * kPStageOp + (size_t)kPSfStages * kPSfStage + 1024 + kPBarBytes;
// E2M1 x E2M1, UE4M3 scales, K-major, N = 256, M = 256 (pair), dense K = 64
constexpr uint32_t kPIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

struct PairParams {
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
// Arrival on a barrier of any CTA of the cluster.  Relaxed: what it publishes are tensor-memory accesses, which the
// tcgen05 wait and fence before it have completed and ordered; a release at cluster scope costs the arriving thread
// about 1100 cycles here, more than a whole stage of MMAs.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 16 consecutive columns of this thread's tensor-memory lane
__device__ __forceinline__ void tcgen05_st_32x32_x16(uint32_t taddr, const uint4& a, const uint4& b, const uint4& c,
                                                     const uint4& d) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w), "r"(c.x), "r"(c.y), "r"(c.z), "r"(c.w),
      "r"(d.x), "r"(d.y), "r"(d.z), "r"(d.w)
      : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tile load into this CTA's shared memory whose completion is counted on a barrier that may belong to the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
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

__global__ void __launch_bounds__(kPairThreads, 1)
    nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const PairParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sf_ring = smem + (size_t)kPStages * kPStageOp;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_ring + (size_t)kPSfStages * kPSfStage);
  uint64_t* full_bar = bars;                         // leader's: the operands of both CTAs have landed
  uint64_t* empty_bar = full_bar + kPStages;         // own: the MMAs that read the stage (and its scale slot) are done
  uint64_t* sf_ready = empty_bar + kPStages;         // leader's: both CTAs' scales of the stage are in tensor memory
  uint64_t* sf_full = sf_ready + kPStages;           // own: scale-factor slot has landed in shared memory
  uint64_t* sf_free = sf_full + kPSfStages;          // own: scale-factor slot has been copied to tensor memory
  uint64_t* acc_full = sf_free + kPSfStages;         // own: accumulator complete
  uint64_t* acc_empty = acc_full + 1;                // leader's: both epilogues have drained
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_empty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int n_pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
  const int n_tiles_total = p.m_pairs * p.n_tiles;
  if (blockIdx.x == 0 && threadIdx.x == 0) *p.status = 0;    // a wait writes it only after its ~1 s budget

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_ready[s]), 8);       // one arrival per scale warp of both CTAs
    }
    for (int j = 0; j < kPSfStages; ++j) {
      mbar_init(smem_u32(&sf_full[j]), 1);
      mbar_init(smem_u32(&sf_free[j]), 4);        // one arrival per scale warp
    }
    mbar_init(smem_u32(acc_full), 1);
    mbar_init(smem_u32(acc_empty), 32);           // one arrival per epilogue warp of both CTAs
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
    // ------------------------------------------------------------------ operand loads (both CTAs)
    if (lane == 0) {
      const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[0]), 0);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs) {
        const int mp = tile % p.m_pairs, nt = tile / p.m_pairs;
        const int a_row0 = mp * 256 + (int)rank * 128, b_row0 = nt * 256 + (int)rank * 128;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kPStages, ph = (it / kPStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, 21)) { ok = false; break; }
          unsigned char* st = smem + (size_t)s * kPStageOp;
          // the leader announces the bytes of both CTAs; the peer's copies may complete before or after that
          if (leader) mbar_expect_tx(smem_u32(&full_bar[s]), 2u * kPStageOp);
          tma_load_2d_pair(smem_u32(st), &map_a, ks * 128, a_row0, full_leader + s * 8);
          tma_load_2d_pair(smem_u32(st + kPStageA), &map_b, ks * 128, b_row0, full_leader + s * 8);
        }
      }
    }
  } else if (warp == 14) {
    // ------------------------------------------------------------------ scale-factor loads (both CTAs)
    if (lane == 0) {
      uint32_t jt = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs) {
        const int mp = tile % p.m_pairs, nt = tile / p.m_pairs;
        const int sfa_tile = mp * 2 + (int)rank;
        const bool sfa_ok = sfa_tile * 128 < p.M;        // the peer's A rows may lie entirely past M
        int sf_tiles = 0;
        for (int j = 0; j < 2; ++j) sf_tiles += ((nt * 2 + j) * 128 < p.N) ? 1 : 0;
        for (int ks = 0; ks < p.k_stages; ++ks, ++jt) {
          const uint32_t j = jt % kPSfStages, ph = (jt / kPSfStages) & 1;
          if (!mbar_wait(smem_u32(&sf_free[j]), ph ^ 1, p.status, 22)) { ok = false; break; }
          unsigned char* sf = sf_ring + (size_t)j * kPSfStage;
          const int kblocks = min(4, KT - ks * 4);
          const uint32_t bar = smem_u32(&sf_full[j]);
          mbar_expect_tx(bar, (uint32_t)(kblocks * 512 * ((sfa_ok ? 1 : 0) + sf_tiles)));
          if (sfa_ok)
            bulk_load_1d(smem_u32(sf), p.sfa + ((size_t)sfa_tile * KT + (size_t)ks * 4) * 512, (uint32_t)kblocks * 512, bar);
          for (int t = 0; t < sf_tiles; ++t)
            bulk_load_1d(smem_u32(sf + kPSfA + t * 2048), p.sfb + ((size_t)(nt * 2 + t) * KT + (size_t)ks * 4) * 512,
                         (uint32_t)kblocks * 512, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs, ++tcount) {
        if (!mbar_wait(smem_u32(acc_empty), (tcount & 1) ^ 1, p.status, 23)) { ok = false; break; }
        tcgen05_fence_after();
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % kPStages, ph = (it / kPStages) & 1;
          if (!mbar_wait(smem_u32(&sf_ready[s]), ph, p.status, 24)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, p.status, 25)) { ok = false; break; }
          tcgen05_fence_after();
          unsigned char* st = smem + (size_t)s * kPStageOp;
          const int kblocks = min(4, KT - ks * 4);
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + kPStageA);
          const uint32_t sfa_tmem = tmem_base + kPSfBase + s * kPSfCols, sfb_tmem = sfa_tmem + 16;
          for (int kb = 0; kb < kblocks; ++kb)
            tcgen05_mma_nvf4_pair(tmem_base, desc_kmajor<128>(a_addr + kb * 32), desc_kmajor<128>(b_addr + kb * 32), kPIdesc,
                                  sfa_tmem + kb * 4, sfb_tmem + kb * 8, (ks > 0 || kb > 0) ? 1u : 0u);
          tcgen05_commit_pair(smem_u32(&empty_bar[s]), 3);     // both CTAs may refill this stage and its scale slot
        }
        if (ok) tcgen05_commit_pair(smem_u32(acc_full), 3);     // both epilogues may start
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ------------------------------------------------------------------ scale factors (both CTAs)
    // One warp per tensor-memory lane quarter.  (A second group of four warps taking alternate stages, and stores left
    // in flight across the next stage's waits, were both measured: no gain.)
    const int quarter = warp & 3;
    const uint32_t ready_leader = map_to_cta(smem_u32(&sf_ready[0]), 0);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs) {
      for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
        const uint32_t s = it % kPStages, ph = (it / kPStages) & 1;
        const uint32_t j = it % kPSfStages, jph = (it / kPSfStages) & 1;
        ok = mbar_wait(smem_u32(&sf_full[j]), jph, p.status, 26);
        // the tensor-memory slot is free once the MMAs of the stage's previous use are done
        ok = ok && mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, 27);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const unsigned char* sf = sf_ring + (size_t)j * kPSfStage;
        const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + kPSfBase + s * kPSfCols;
        // columns [0,16): A scales of k-blocks 0..3; [16,48): B scales, k-block-major, two 128-row tiles each.
        // A short last stage copies stale bytes for the k-blocks it lacks; no MMA reads them.
        const uint4* sa = reinterpret_cast<const uint4*>(sf + lane * 16);
        const uint4* sb = reinterpret_cast<const uint4*>(sf + kPSfA + lane * 16);
        tcgen05_st_32x32_x16(t0, sa[0], sa[32], sa[64], sa[96]);                          // 512 bytes per k-block
        tcgen05_st_32x32_x16(t0 + 16, sb[0], sb[128], sb[32], sb[128 + 32]);              // k-blocks 0, 1: tile 0, tile 1
        tcgen05_st_32x32_x16(t0 + 32, sb[64], sb[128 + 64], sb[96], sb[128 + 96]);        // k-blocks 2, 3
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&sf_free[j]));
          mbar_arrive_cluster(ready_leader + s * 8);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, warps 2..5, 10..13, 15..22)
    // Four warps per tensor-memory lane quarter, each draining and storing 64 of the tile's 256 columns (with two warps per
    // quarter the MMA thread waited about 1200 cycles per tile for the drain; M=4096: 121 us against 123 us).
    const int quarter = warp & 3;
    const int grp = warp < 6 ? 0 : (warp < 14 ? 1 : (warp < 19 ? 2 : 3));     // warps 2-5, 10-13, 15-18, 19-22
    const int c_first = grp * 2;
    const float alpha = p.alpha[0];
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(acc_empty), 0);
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < n_tiles_total; tile += n_pairs, ++tcount) {
      const int mp = tile % p.m_pairs, nt = tile / p.m_pairs;
      ok = mbar_wait(smem_u32(acc_full), tcount & 1, p.status, 28);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = mp * 256 + (int)rank * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
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
      // hand the accumulator back before the global stores, which then overlap the next tile's main loop
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      if (row < p.M) {
        uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.out) + (size_t)row * p.N;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = nt * 256 + (c_first + c) * 32;
          if (col0 < p.N) {
            uint16_t* dst = dst_row + col0;
            if (col0 + 32 <= p.N && (p.N % 16) == 0 && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
              for (int i = 0; i < 2; ++i) st_global_v8(dst + 16 * i, &packed[c * 16 + 8 * i]);
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
  // every role of both CTAs ends here, also after an expired wait
  tcgen05_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

// Launches the CTA-pair kernel (clusters of two CTAs).  Tensor maps: A box = 128 rows, B box = 128 rows, 128-byte
// rows.  16-bit output.  The grid is the number of pairs that can be resident at once (a GPC with an odd number of SMs
// leaves one of them without a partner), because the kernel strides over the tiles with its grid size.
int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
                     void* out, int out_bf16, int M, int N, int K, int* status, cudaStream_t st) {
  static int max_pairs_of[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return B200FP4_STATUS_NOT_SUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs_of[dev] == 0) {
    if (cudaFuncSetAttribute(nvfp4_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairSmemBytes) !=
        cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    cfg.gridDim = dim3((unsigned)(sm_count() & ~1));
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, nvfp4_gemm_pair_kernel, &cfg) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    max_pairs_of[dev] = clusters;
  }
  PairParams p;
  p.sfa = sfa; p.sfb = sfb; p.alpha = alpha; p.out = out; p.out_bf16 = out_bf16;
  p.M = M; p.N = N; p.K = K;
  p.m_pairs = (M + 255) / 256;
  p.n_tiles = (N + 255) / 256;
  p.k_stages = (K + 255) / 256;
  p.status = status;
  long long pairs = (long long)p.m_pairs * p.n_tiles;
  if (pairs > max_pairs_of[dev]) pairs = max_pairs_of[dev];
  if (pairs < 1) pairs = 1;
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  if (cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair_kernel, ma, mb, p) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  return B200FP4_STATUS_SUCCESS;
}

}  // namespace b200fp4
