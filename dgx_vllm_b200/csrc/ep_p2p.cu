// Expert-parallel exchange over peer memory: dispatch and combine without a collective library call.
//
// Every rank owns three buffers that all ranks can address (peer mappings over NVLink; the caller allocates them, for
// instance with torch's symmetric memory, and passes the per-rank pointers as device arrays):
//   records [G][B] dispatch records -- slot g is written by rank g
//   parts   [G][B][H] fp32          -- slot g holds the partial output rows that rank g computed for this rank's tokens
//   flags   [2][G] int32            -- [0][g]: rank g's records of step `seq` have landed; [1][g]: its partial rows have
// A step is numbered by `seq` (1, 2, 3, ... the same on every rank); flags only grow, so nothing is ever reset.
//   dispatch kernel  block b packs token b's record and stores it into slot `rank` of EVERY rank's records buffer (plain
//                    16-byte peer stores); the last block to finish publishes flags[0][rank] = seq on every rank
//                    (release, system scope) and then waits until all G flags[0][*] of its own rank have reached seq,
//                    so the kernels that follow on the stream see all records.
//   (the fused MoE layer runs over the G*B records; its last kernel stores the partial rows of rank g's tokens straight
//    into slot `rank` of rank g's parts buffer -- b200fp4_fused_sparse_moe_records_scatter)
//   combine kernel   publishes flags[1][rank] = seq on every rank, waits for all G flags[1][*] of its own rank, then adds
//                    the G partial rows of every token in fp32 and rounds once.
// Why one buffer of each kind is enough: a rank writes step s+1 records only after its own combine of step s, which
// waited for every peer's partial rows of step s, which a peer sends after it has read the records of step s; and a peer
// reaches the partial rows of step s+1 only after this rank's step s+1 records, which follow its combine of step s on the
// stream.
// Every wait is bounded (clock64 budget); a wait that runs out records a code in the status word and the kernel carries
// on to its end, so a missing peer cannot hang the GPU.  Plain peer loads and stores only: no multicast objects.
// The reference has no multi-GPU code of its own (it serves with tensor parallelism through vLLM).
#include "common.cuh"

extern "C" size_t b200fp4_ep_record_bytes(int64_t H, int64_t topk);

namespace b200fp4 {
namespace {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// thread g < G waits until flags[g] >= seq; returns false when the budget ran out
__device__ __forceinline__ bool wait_flag(const int* flag, int seq, long long budget) {
  if (ld_acquire_sys(flag) >= seq) return true;
  const long long t0 = clock64();
  while (ld_acquire_sys(flag) < seq)
    if (clock64() - t0 > budget) return false;
  return true;
}

__global__ void __launch_bounds__(256)
    ep_dispatch_p2p_kernel(const uint4* __restrict__ hidden, const int32_t* __restrict__ ids, const float* __restrict__ w, int B,
                           int H, int topk, int G, int rank, int64_t rec_chunks, uint4* const* __restrict__ rec_ptrs,
                           int* const* __restrict__ flag_ptrs, int seq, int* scratch, long long budget) {
  // launched with the programmatic attribute: resident early, but nothing is read or stored before the kernels ahead on
  // the stream (the producer of the activations, this rank's combine of the previous step) have completed
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int h_chunks = H / 8;
  __shared__ uint4 s_tail[64];
  __shared__ int s_last;
  const int tail_chunks = (int)rec_chunks - h_chunks;
  if ((int)threadIdx.x < tail_chunks * 4) {
    const int i = threadIdx.x;            // 32-bit word index inside the tail: ids first, then weights
    uint32_t v = 0;
    if (i < topk) v = (uint32_t)ids[(int64_t)b * topk + i];
    else if (i < 2 * topk) v = __float_as_uint(w[(int64_t)b * topk + i - topk]);
    reinterpret_cast<uint32_t*>(s_tail)[i] = v;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < rec_chunks; c += blockDim.x) {
    const uint4 v = c < h_chunks ? hidden[(int64_t)b * h_chunks + c] : s_tail[c - h_chunks];
    for (int g = 0; g < G; ++g) rec_ptrs[g][((int64_t)rank * B + b) * rec_chunks + c] = v;
  }
  // the last block to get here publishes the flag: its fence covers the other blocks' stores, which it has observed
  // through the counter
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&scratch[0], 1) == B - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if ((int)threadIdx.x < G) {
    st_release_sys(flag_ptrs[threadIdx.x] + rank, seq);
    if (!wait_flag(flag_ptrs[rank] + threadIdx.x, seq, budget)) atomicCAS(&scratch[1], 0, 1 + (int)threadIdx.x);
  }
  if (threadIdx.x == 0) scratch[0] = 0;      // ready for the next step
}

template <typename T>
__global__ void __launch_bounds__(256)
    ep_combine_p2p_kernel(const float* __restrict__ parts, int B, int H, int G, int rank, int* const* __restrict__ flag_ptrs,
                          int seq, int* scratch, long long budget, T* __restrict__ out) {
  pdl_wait();          // the kernel before this one on the stream stored this rank's partial rows into the peers' buffers
  pdl_launch_dependents();
  if ((int)threadIdx.x < G) {
    // the kernel before this one on the stream stored this rank's partial rows into the peers' buffers
    if (blockIdx.x == 0) {
      __threadfence_system();
      st_release_sys(flag_ptrs[threadIdx.x] + G + rank, seq);
    }
    if (!wait_flag(flag_ptrs[rank] + G + threadIdx.x, seq, budget)) atomicCAS(&scratch[1], 0, 101 + (int)threadIdx.x);
  }
  __syncthreads();
  const int64_t n = (int64_t)B * H;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int g = 0; g < G; ++g) {
      const float4 v = *reinterpret_cast<const float4*>(parts + (int64_t)g * n + i);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    out[i] = from_f32<T>(a.x);
    out[i + 1] = from_f32<T>(a.y);
    out[i + 2] = from_f32<T>(a.z);
    out[i + 3] = from_f32<T>(a.w);
  }
}

constexpr long long kEpWaitCycles = 2000000000LL;    // ~1 s of SM clocks

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" int b200fp4_ep_dispatch_p2p(const void* hidden, const int32_t* topk_ids, const float* topk_weights, int64_t B,
                                       int64_t H, int64_t topk, int64_t G, int64_t rank, void* const* record_ptrs,
                                       int32_t* const* flag_ptrs, int32_t seq, int32_t* scratch, void* stream) {
  if (B <= 0 || H <= 0 || (H % 8) != 0 || topk <= 0 || topk > 64 || G <= 0 || G > 64 || rank < 0 || rank >= G || seq <= 0)
    return B200FP4_STATUS_INVALID_VALUE;
  if (!hidden || !topk_ids || !topk_weights || !record_ptrs || !flag_ptrs || !scratch || !aligned(hidden, 16))
    return B200FP4_STATUS_INVALID_VALUE;
  const int64_t rec_chunks = (int64_t)b200fp4_ep_record_bytes(H, topk) / 16;
  launch_pdl(ep_dispatch_p2p_kernel, dim3((unsigned)B), dim3(256), 0, (cudaStream_t)stream,
             reinterpret_cast<const uint4*>(hidden), topk_ids, topk_weights, (int)B, (int)H, (int)topk, (int)G, (int)rank, rec_chunks,
             reinterpret_cast<uint4* const*>(record_ptrs), reinterpret_cast<int* const*>(flag_ptrs), (int)seq, scratch,
             kEpWaitCycles);
  return finish_launch(1);
}

extern "C" int b200fp4_ep_combine_p2p(const float* parts, int64_t B, int64_t H, int64_t G, int64_t rank,
                                      int32_t* const* flag_ptrs, int32_t seq, int32_t* scratch, void* out, int out_dtype,
                                      void* stream) {
  if (B <= 0 || H <= 0 || (H % 4) != 0 || G <= 0 || G > 64 || rank < 0 || rank >= G || seq <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (out_dtype != B200FP4_DTYPE_BF16 && out_dtype != B200FP4_DTYPE_F16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (!parts || !flag_ptrs || !scratch || !out || !aligned(parts, 16)) return B200FP4_STATUS_INVALID_VALUE;
  int64_t blocks = (B * H / 4 + 255) / 256;
  if (blocks > 2 * (int64_t)sm_count()) blocks = 2 * (int64_t)sm_count();
  if (out_dtype == B200FP4_DTYPE_BF16)
    launch_pdl(ep_combine_p2p_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, parts, (int)B,
               (int)H, (int)G, (int)rank, reinterpret_cast<int* const*>(flag_ptrs), (int)seq, scratch, kEpWaitCycles,
               reinterpret_cast<__nv_bfloat16*>(out));
  else
    launch_pdl(ep_combine_p2p_kernel<__half>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, parts, (int)B, (int)H,
               (int)G, (int)rank, reinterpret_cast<int* const*>(flag_ptrs), (int)seq, scratch, kEpWaitCycles,
               reinterpret_cast<__half*>(out));
  return finish_launch(1);
}
