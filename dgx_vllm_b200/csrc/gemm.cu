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
#include <cuda.h>

#include "common.cuh"

namespace b200fp4 {
namespace {

constexpr int kBM = 128;
constexpr int kBKBytes = 128;             // bytes of packed codes per row per stage (= 256 k)
constexpr int kKPerStage = 256;
constexpr int kGemmThreads = 320;         // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-9 scale factors
constexpr uint32_t kTmemCols = 512;
constexpr long long kWaitCycles = 2000000000LL;   // ~1 s at 2 GHz

struct GemmParams {
  const uint8_t* sfa;   // swizzled [ceil(M/128)*128, ceil(K/64)*4]
  const uint8_t* sfb;   // swizzled [ceil(N/128)*128, ceil(K/64)*4]
  const float* alpha;
  void* out;
  int out_bf16;
  int M, N, K;
  int m_tiles, n_tiles, k_stages;
  int* status;          // 0 = ok; otherwise the code of the wait that expired
};

// ---------------------------------------------------------------------------------------- PTX

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and records `code`) if the phase does not complete in ~1 s.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitCycles) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void tcgen05_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// each lane writes 16 bytes (4 columns) of its own tensor-memory lane
__device__ __forceinline__ void tcgen05_st_32x32_x4(uint32_t taddr, const uint4& v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void tcgen05_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (K-major).  Fields: start address >> 4 in bits [0,14), leading
// byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in
// [46,48), swizzle mode in [61,64) (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  // rows of 128 bytes, 8-row swizzle atoms 1024 bytes apart
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// ---------------------------------------------------------------------------------------- kernel

template <int BN>
struct Cfg {
  static constexpr int kAcc = BN == 128 ? 2 : 1;                    // accumulator buffers in tensor memory
  static constexpr int kSfTiles = BN / 128;                         // 128-row scale tiles on the B side
  static constexpr int kStageA = kBM * kBKBytes;                    // 16 KiB
  static constexpr int kStageB = BN * kBKBytes;
  static constexpr int kStageSFA = 4 * 512;
  static constexpr int kStageSFB = kSfTiles * 4 * 512;
  static constexpr int kStageBytes = kStageA + kStageB + kStageSFA + kStageSFB;
  static constexpr int kStages = BN == 128 ? 6 : 4;
  // tensor-memory column map: accumulators, then one scale-factor block per shared-memory stage
  // (16 columns for A, 16*kSfTiles for B) so that the tcgen05.cp of stage s+1 never has to wait
  // for the MMAs of stage s to finish reading their scales
  static constexpr uint32_t kSfCols = 16 + 16 * kSfTiles;
  static constexpr uint32_t kSfBase = kAcc * BN;
  static_assert(kSfBase + kStages * kSfCols <= 512, "tensor memory budget");
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // instruction descriptor: E2M1 x E2M1, UE4M3 scales, K-major A and B, N = BN, M = 128, dense K = 64
  static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
};

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* acc_full = bars + 2 * C::kStages;
  uint64_t* acc_empty = acc_full + C::kAcc;
  uint64_t* sf_ready = acc_empty + C::kAcc;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(sf_ready + C::kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles_total = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&sf_ready[s]), 128);
    }
    for (int a = 0; a < C::kAcc; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 128);
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
        const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
        for (int ks = 0; ks < p.k_stages; ++ks, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, 1)) { ok = false; break; }
          unsigned char* st = smem + (size_t)s * C::kStageBytes;
          const int kblocks = min(4, KT - ks * 4);
          int sf_tiles = 0;
          for (int j = 0; j < C::kSfTiles; ++j) sf_tiles += ((nt * C::kSfTiles + j) * 128 < p.N) ? 1 : 0;
          const uint32_t bar = smem_u32(&full_bar[s]);
          mbar_expect_tx(bar, (uint32_t)(C::kStageA + C::kStageB + kblocks * 512 * (1 + sf_tiles)));
          tma_load_2d(smem_u32(st), &map_a, ks * kBKBytes, mt * kBM, bar);
          tma_load_2d(smem_u32(st + C::kStageA), &map_b, ks * kBKBytes, nt * BN, bar);
          bulk_load_1d(smem_u32(st + C::kStageA + C::kStageB), p.sfa + ((size_t)mt * KT + (size_t)ks * 4) * 512,
                       (uint32_t)kblocks * 512, bar);
          for (int j = 0; j < sf_tiles; ++j)
            bulk_load_1d(smem_u32(st + C::kStageA + C::kStageB + C::kStageSFA + j * 2048),
                         p.sfb + ((size_t)(nt * C::kSfTiles + j) * KT + (size_t)ks * 4) * 512, (uint32_t)kblocks * 512, bar);
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
          const int kblocks = min(4, KT - ks * 4);
          const uint32_t a_addr = smem_u32(st), b_addr = smem_u32(st + C::kStageA);
          const uint32_t sfa_tmem = tmem_base + C::kSfBase + s * C::kSfCols, sfb_tmem = sfa_tmem + 16;
          if (!mbar_wait(smem_u32(&sf_ready[s]), ph, p.status, 5)) { ok = false; break; }
          tcgen05_fence_after();
          for (int kb = 0; kb < kblocks; ++kb) {
            // each 64-wide k-block is 32 bytes further along the swizzled 128-byte rows
            tcgen05_mma_nvf4(d_tmem, desc_sw128(a_addr + kb * 32), desc_sw128(b_addr + kb * 32), C::kIdesc,
                             sfa_tmem + kb * 4, sfb_tmem + kb * (4 * C::kSfTiles), (ks > 0 || kb > 0) ? 1u : 0u);
          }
          tcgen05_commit(smem_u32(&empty_bar[s]));    // frees the stage when these MMAs have read it
        }
        if (ok) tcgen05_commit(smem_u32(&acc_full[acc]));
      }
    }
  } else if (warp >= 6) {
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
        ok = mbar_wait(smem_u32(&full_bar[s]), ph, p.status, 6);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const unsigned char* sf = smem + (size_t)s * C::kStageBytes + C::kStageA + C::kStageB;
        const uint32_t t0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::kSfBase + s * C::kSfCols;
        const int kblocks = min(4, KT - ks * 4);
        for (int kb = 0; kb < kblocks; ++kb) {
          tcgen05_st_32x32_x4(t0 + kb * 4, *reinterpret_cast<const uint4*>(sf + kb * 512 + lane * 16));
#pragma unroll
          for (int j = 0; j < C::kSfTiles; ++j)
            tcgen05_st_32x32_x4(t0 + 16 + kb * (4 * C::kSfTiles) + j * 4,
                                *reinterpret_cast<const uint4*>(sf + C::kStageSFA + j * 2048 + kb * 512 + lane * 16));
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        mbar_arrive(smem_u32(&sf_ready[s]));
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
      const uint32_t acc = tcount % C::kAcc, aph = (tcount / C::kAcc) & 1;
      ok = mbar_wait(smem_u32(&acc_full[acc]), aph, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = mt * kBM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      // drain this thread's row of the accumulator into packed 16-bit registers ...
      uint32_t packed[BN / 2];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
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
      // ... hand the accumulator back to the MMA warp, and only then write to global memory, so
      // that the stores overlap the next tile's main loop
      tcgen05_fence_before();
      mbar_arrive(smem_u32(&acc_empty[acc]));
      if (row < p.M) {
        uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.out) + (size_t)row * p.N;
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = nt * BN + c * 32;
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
  // all roles fall through to here (also after a timed-out wait), so tensor memory is always freed
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
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

// [rows, row_bytes] u8 row-major; box = 128 bytes x box_rows, 128-byte swizzle, zero fill out of bounds
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)kBKBytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(nvfp4_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)Cfg<BN>::kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    attr_set[dev] = true;
  }
  p.n_tiles = (p.N + BN - 1) / BN;
  int grid = p.m_tiles * p.n_tiles;
  if (grid > sm_count()) grid = sm_count();
  nvfp4_gemm_kernel<BN><<<grid, kGemmThreads, Cfg<BN>::kSmemBytes, st>>>(ma, mb, p);
  return B200FP4_STATUS_SUCCESS;
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
  if (out_dtype != B200FP4_DTYPE_BF16 && out_dtype != B200FP4_DTYPE_F16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!a_codes || !b_codes || !sfa || !sfb || !alpha || !out) return B200FP4_STATUS_INVALID_VALUE;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(sfa, 16) || !aligned(sfb, 16) || !aligned(out, 16) ||
      ((K / 2) % 16) != 0)
    return B200FP4_STATUS_INVALID_VALUE;
  if (!workspace || workspace_bytes < 256 || !aligned(workspace, 16)) return B200FP4_STATUS_ALLOC_FAILED;
  if (tile_n != 0 && tile_n != 128 && tile_n != 256) return B200FP4_STATUS_INVALID_VALUE;
  if (M > (1 << 24) || N > (1 << 24) || K > (1 << 24)) return B200FP4_STATUS_NOT_SUPPORTED;
  if (b200fp4_has_hardware_acceleration() != 1) return B200FP4_STATUS_ARCH_MISMATCH;
  cudaStream_t st = (cudaStream_t)stream;
  GemmParams p;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa);
  p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.alpha = alpha;
  p.out = out;
  p.out_bf16 = out_dtype == B200FP4_DTYPE_BF16;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.m_tiles = (int)((M + kBM - 1) / kBM);
  p.k_stages = (int)((K + kKPerStage - 1) / kKPerStage);
  p.status = reinterpret_cast<int*>(workspace);
  // Wide tiles once there are enough of them to fill the GPU; narrow tiles (double-buffered
  // accumulator, twice the CTAs) for small problems.
  int bn = tile_n;
  if (bn == 0) bn = (p.m_tiles * ((N + 255) / 256) >= sm_count()) ? 256 : 128;
  CUtensorMap ma, mb;
  if (!make_map(&ma, a_codes, (uint64_t)M, (uint64_t)K / 2, kBM) ||
      !make_map(&mb, b_codes, (uint64_t)N, (uint64_t)K / 2, (uint32_t)bn))
    return B200FP4_STATUS_INTERNAL_ERROR;
  if (cudaMemsetAsync(workspace, 0, 16, st) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  int rc = bn == 256 ? launch_gemm<256>(ma, mb, p, st) : launch_gemm<128>(ma, mb, p, st);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  return finish_launch(2);
}
