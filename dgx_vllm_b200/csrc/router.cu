// MoE router for decode: gate projection (16-bit weights), softmax over the experts, top-k, renormalisation.
//
// The reference leaves routing to vLLM (its benches build it in torch: softmax of the gate logits, topk, weights
// divided by their sum -- sparse_fp4_kernel/bench_moe_layer_e2e.py:230-236); here it is two small kernels whose
// outputs (topk_weights f32, topk_ids i32) are exactly the device tensors the fused MoE layer and the expert-parallel
// dispatch take, so no host round trip sits between the router and the experts.
//   router_logits_kernel   block = 64 experts x 8 tokens; the tokens' activations sit in shared memory, every warp
//                          streams whole weight rows (16-byte loads) and keeps 8 fp32 dot products per row
//   router_topk_kernel     one warp per token: k rounds of warp-wide arg-max (ties -> lower expert id), weights
//                          exp(l - max) normalised over the selected experts (or over all of them)
#include "common.cuh"

namespace b200fp4 {
namespace {

constexpr int kRtTokens = 8;
constexpr int kRtExperts = 64;
constexpr int kRtThreads = 256;

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float* v);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& raw, float* v) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& raw, float* v) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename T>
__global__ void __launch_bounds__(kRtThreads)
    router_logits_kernel(const T* __restrict__ hidden, int64_t ld_h, const T* __restrict__ gate_w, int M, int H, int E,
                         float* __restrict__ logits) {
  extern __shared__ __align__(16) unsigned char smem[];
  T* sx = reinterpret_cast<T*>(smem);                     // [kRtTokens][H]
  const int m0 = blockIdx.y * kRtTokens, e0 = blockIdx.x * kRtExperts;
  const int chunks = H >> 3;
  for (int i = threadIdx.x; i < kRtTokens * chunks; i += kRtThreads) {
    const int tk = i / chunks, c = i - tk * chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m0 + tk < M) v = *reinterpret_cast<const uint4*>(hidden + (int64_t)(m0 + tk) * ld_h + c * 8);
    reinterpret_cast<uint4*>(sx)[i] = v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = warp; i < kRtExperts; i += kRtThreads / 32) {
    const int e = e0 + i;
    if (e >= E) break;
    float acc[kRtTokens];
#pragma unroll
    for (int tk = 0; tk < kRtTokens; ++tk) acc[tk] = 0.f;
    for (int c = lane; c < chunks; c += 32) {
      float w[8];
      unpack8<T>(ldg_stream_u4(gate_w + (int64_t)e * H + c * 8), w);
#pragma unroll
      for (int tk = 0; tk < kRtTokens; ++tk) {
        float x[8];
        unpack8<T>(reinterpret_cast<const uint4*>(sx)[tk * chunks + c], x);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[tk] = fmaf(w[k], x[k], acc[tk]);
      }
    }
#pragma unroll
    for (int tk = 0; tk < kRtTokens; ++tk) {
      float v = acc[tk];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
      if (lane == 0 && m0 + tk < M) logits[(int64_t)(m0 + tk) * E + e] = v;
    }
  }
}

// One warp per token; E <= 32 * kRtPerLane.
constexpr int kRtPerLane = 32;

__global__ void __launch_bounds__(128)
    router_topk_kernel(const float* __restrict__ logits, int M, int E, int topk, int renormalize,
                       float* __restrict__ topk_w, int32_t* __restrict__ topk_ids) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  float v[kRtPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kRtPerLane; ++i) {
    const int e = i * 32 + lane;                 // lane-interleaved: expert e lives in lane e % 32, slot e / 32
    v[i] = e < E ? logits[(int64_t)m * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  float total = 0.f;
  if (!renormalize) {
#pragma unroll
    for (int i = 0; i < kRtPerLane; ++i) total += (i * 32 + lane < E) ? __expf(v[i] - mx) : 0.f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
  }
  float sel_sum = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int r = 0; r < topk; ++r) {
    // this lane's best remaining (lowest slot wins ties, which is the lowest expert id within the lane)
    float best = -INFINITY;
    int slot = 0;
#pragma unroll
    for (int i = 0; i < kRtPerLane; ++i)
      if (v[i] > best) {
        best = v[i];
        slot = i;
      }
    int id = slot * 32 + lane;
    float cand = best;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, cand, d);
      const int oid = __shfl_xor_sync(0xffffffffu, id, d);
      if (ov > cand || (ov == cand && oid < id)) {
        cand = ov;
        id = oid;
      }
    }
    if ((id & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kRtPerLane; ++i)
        if (i == (id >> 5)) v[i] = -INFINITY;      // compile-time indexed: keeps v[] in registers
    }
    const float w = __expf(cand - mx);
    sel_sum += w;
    if (lane == r) {
      my_w = w;
      my_id = id;
    }
  }
  const float denom = renormalize ? sel_sum : total;
  if (lane < topk) {
    topk_w[(int64_t)m * topk + lane] = my_w / denom;
    topk_ids[(int64_t)m * topk + lane] = my_id;
  }
}

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" size_t b200fp4_moe_router_workspace_bytes(int64_t M, int64_t E) {
  if (M < 0 || E < 0) return 0;
  return (size_t)M * (size_t)E * sizeof(float);
}

extern "C" int b200fp4_moe_router(const void* hidden, int64_t ld_h, int dtype, const void* gate_w, int64_t M, int64_t H,
                                  int64_t E, int64_t topk, int renormalize, float* topk_weights, int32_t* topk_ids,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  if (M < 0 || H <= 0 || E <= 0 || topk <= 0 || (H % 8) != 0 || ld_h < H || (ld_h % 8) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (dtype != B200FP4_DTYPE_BF16 && dtype != B200FP4_DTYPE_F16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (topk > 32 || topk > E || E > 32 * kRtPerLane || (size_t)kRtTokens * H * 2 > 200 * 1024) return B200FP4_STATUS_NOT_SUPPORTED;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!hidden || !gate_w || !topk_weights || !topk_ids || !aligned(hidden, 16) || !aligned(gate_w, 16))
    return B200FP4_STATUS_INVALID_VALUE;
  if (!workspace || workspace_bytes < b200fp4_moe_router_workspace_bytes(M, E) || !aligned(workspace, 4))
    return B200FP4_STATUS_ALLOC_FAILED;
  cudaStream_t st = (cudaStream_t)stream;
  float* logits = static_cast<float*>(workspace);
  const size_t smem = (size_t)kRtTokens * H * 2;
  dim3 grid((unsigned)((E + kRtExperts - 1) / kRtExperts), (unsigned)((M + kRtTokens - 1) / kRtTokens));
  if (dtype == B200FP4_DTYPE_BF16) {
    static bool set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !set[dev]) {
      cudaFuncSetAttribute(router_logits_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      set[dev] = true;
    }
    router_logits_kernel<__nv_bfloat16><<<grid, kRtThreads, smem, st>>>(static_cast<const __nv_bfloat16*>(hidden), ld_h,
                                                                        static_cast<const __nv_bfloat16*>(gate_w), (int)M,
                                                                        (int)H, (int)E, logits);
  } else {
    static bool set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !set[dev]) {
      cudaFuncSetAttribute(router_logits_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      set[dev] = true;
    }
    router_logits_kernel<__half><<<grid, kRtThreads, smem, st>>>(static_cast<const __half*>(hidden), ld_h,
                                                                 static_cast<const __half*>(gate_w), (int)M, (int)H, (int)E,
                                                                 logits);
  }
  // the top-k kernel may become resident while the projection drains (programmatic dependent launch)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((M + 3) / 4));
  cfg.blockDim = dim3(128);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cfg.numAttrs = (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) ? 1 : 0;
  cudaLaunchKernelEx(&cfg, router_topk_kernel, (const float*)logits, (int)M, (int)E, (int)topk, renormalize, topk_weights,
                     topk_ids);
  return finish_launch(2);
}
