// Shared helpers for the sm_100a NVFP4 kernels: status codes, launch bookkeeping, codecs.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/b200_nvfp4.h"

namespace b200fp4 {

extern std::atomic<uint64_t> g_launch_count;

inline int finish_launch(int n_kernels) {
  g_launch_count.fetch_add((uint64_t)n_kernels, std::memory_order_relaxed);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  return B200FP4_STATUS_SUCCESS;
}

// Programmatic dependent launch: a kernel launched with the attribute may become resident while the kernel before it
// on the stream drains; it must not touch that kernel's data before pdl_wait() returns (the earlier grid has then
// completed and its writes are visible).  pdl_launch_dependents() lets the NEXT kernel do the same with this one.
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // not while a CUDA graph is being captured: replayed graphs have no launch gap to hide, and the 48-layer decode stack
  // measured 3-4 % slower with programmatic edges than with plain ones
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cfg.numAttrs = (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ------------------------------------------------------------------------------------------ device

// 16-byte read-only global load that does not allocate in L1 (streamed weights are read once).
__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// Eight floats -> eight E2M1 codes in one u32 (element i in nibble i), round-to-nearest-even with
// finite saturation, using the native sm_100a conversion.
__device__ __forceinline__ uint32_t f32x8_to_e2m1(float f0, float f1, float f2, float f3, float f4, float f5,
                                                  float f6, float f7) {
  uint32_t v;
  asm("{\n"
      ".reg .b8 q0, q1, q2, q3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 q3, %8, %7;\n"
      "mov.b32 %0, {q0, q1, q2, q3};\n"
      "}\n"
      : "=r"(v)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
  return v;
}

// float -> e4m3 byte (RNE, finite saturation) and back.
__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// The quantizer's SiLU and output-scale arithmetic; shared by the stand-alone quantize kernels and the GEMM
// epilogue that quantizes in place, so that both produce the same bytes.
__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

// 1 / (decoded block scale / global scale), with the reference's "x == 0 -> x + 1e8" guards
__device__ __forceinline__ float out_scale_of(uint8_t sfb, float rcp_gs) {
  const float t = __fmul_rn(e4m3_to_f32(sfb), rcp_gs);
  return __frcp_rn(t + (t == 0.f ? 1.0e8f : 0.f));
}

// Byte offset of scale factor (row m, k-block kb) in the padded 128x4 tile layout with KT = ceil(KB/4).
__host__ __device__ __forceinline__ int64_t sf_swizzled_offset(int64_t m, int64_t kb, int64_t KT) {
  return ((((m >> 7) * KT + (kb >> 2)) * 32 + (m & 31)) * 4 + ((m & 127) >> 5)) * 4 + (kb & 3);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }

}  // namespace b200fp4
