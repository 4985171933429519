// The C API that the reference declares in cutlass_nvfp4/cuda_fp4_gemm.h (and never defines), exported
// under the reference's own symbol names and argument lists, as a thin layer over this library's
// kernels: a program written against that header links against libb200nvfp4.so unchanged.
//
//   cudaFP4Create / Destroy / SetStream      cuda_fp4_gemm.h:48-63   handle = stream + device scratch
//   cudaFP4GemmEx                            cuda_fp4_gemm.h:94-105  linear [rows, K/16] E4M3 scales, global scales by
//                                                                    value, fp32 C:  C = (A.sA)(B.sB)^T * gA * gB
//   cudaFP4Gemm                              cuda_fp4_gemm.h:113-120 no block scales:  C = alpha * A B^T
//   cudaFP4GetVersion* / HasHardware... / GetErrorString             cuda_fp4_gemm.h:124-147
//   cudaFP4ConvertFromFP32 / ToFP32 / Quantize                       cuda_fp4_gemm.h:161-203
//
// What differs from the reference's header-only kernels on purpose: the E2M1 value table is the NVFP4 one
// (0, 0.5, 1, 1.5, 2, 3, 4, 6 with round-to-nearest-even and finite saturation -- the reference's
// nvfp4_types.cuh uses 0.25 for code 1), and group_size must be 16, the only block size the tensor cores
// take.  "Global scale" follows the header's formula: a dequantized element is code * block_scale * global,
// so cudaFP4Quantize reports amax / (6 * 448).
//
// The handle owns device scratch for the two scale tensors in the tensor cores' 128x4-tile layout and a
// device float for alpha.  It is sized at cudaFP4Create for problems up to 8192 x 8192 x 8192 and grows
// (cudaMalloc, which synchronises) on the first call that needs more; calls within the capacity
// allocate nothing.  B's scales are re-laid-out on every call: the API gives no way to say that B is a
// weight that stays the same.
#include <cstring>
#include <new>

#include "common.cuh"

namespace b200fp4 {
namespace {

struct Handle {
  int device;
  cudaStream_t stream;
  unsigned char* scratch;
  size_t scratch_bytes;
};

size_t round256(size_t v) { return (v + 255) / 256 * 256; }

// scratch layout: [0,256) GEMM workspace (status word) | [256,512) alpha | swizzled A scales | swizzled B scales
size_t scratch_need(int64_t M, int64_t N, int64_t K) {
  return 512 + round256(b200fp4_sf_swizzled_bytes(M, K / 16)) + round256(b200fp4_sf_swizzled_bytes(N, K / 16));
}

bool ensure_scratch(Handle* h, size_t need) {
  if (h->scratch_bytes >= need) return true;
  unsigned char* p = nullptr;
  if (cudaMalloc(&p, need) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (h->scratch) cudaFree(h->scratch);
  h->scratch = p;
  h->scratch_bytes = need;
  return true;
}

// linear [rows, KB] -> padded 128x4-tile layout; padding bytes become zero
__global__ void sf_swizzle_kernel(const uint8_t* __restrict__ lin, int64_t rows, int64_t KB, int64_t rows_pad, int64_t KT,
                                  uint8_t* __restrict__ out) {
  const int64_t total = rows_pad * KT * 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / (KT * 4), kb = i - m * (KT * 4);
    out[sf_swizzled_offset(m, kb, KT)] = (m < rows && kb < KB) ? lin[m * KB + kb] : (uint8_t)0;
  }
}

__global__ void fill_bytes_kernel(uint8_t* p, int64_t n, uint8_t v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

__global__ void set_float_kernel(float* p, float v) { *p = v; }

// eight floats -> four bytes of packed E2M1 (element 2i in the low nibble)
__global__ void from_fp32_kernel(const float* __restrict__ src, int64_t n8, uint32_t* __restrict__ dst) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(src)[2 * i], b = reinterpret_cast<const float4*>(src)[2 * i + 1];
    dst[i] = f32x8_to_e2m1(a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w);
  }
}

__device__ __forceinline__ float e2m1_value(uint32_t nib) {
  const uint32_t c = nib & 7u;
  const float v = c < 4u ? 0.5f * (float)c : (c == 4u ? 2.f : (c == 5u ? 3.f : (c == 6u ? 4.f : 6.f)));
  return (nib & 8u) ? -v : v;
}

__global__ void to_fp32_kernel(const uint8_t* __restrict__ src, int64_t n2, float* __restrict__ dst) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t b = src[i];
    reinterpret_cast<float2*>(dst)[i] = make_float2(e2m1_value(b & 15u), e2m1_value(b >> 4));
  }
}

// max |x| as the bit pattern of a non-negative float (ordered like an unsigned integer)
__global__ void amax_kernel(const float* __restrict__ src, int64_t n, unsigned int* __restrict__ out) {
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(src[i]));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));
}

// One thread per block of 16: the quantizer's arithmetic (ref_nvfp4_quant order, IEEE fp32) on fp32 input,
// with the global scale 448*6/amax computed from the device-side amax.  Linear scales [rows, cols/16].
__global__ void quantize_f32_kernel(const float* __restrict__ src, int64_t rows, int64_t cols,
                                    const unsigned int* __restrict__ amax_bits, uint32_t* __restrict__ codes,
                                    uint8_t* __restrict__ sf) {
  const int64_t KB = cols >> 4, total = rows * KB;
  const float amax_all = __uint_as_float(*amax_bits);
  const float gs = __fdiv_rn(448.0f * 6.0f, amax_all);
  const float rcp_gs = __frcp_rn(gs + (gs == 0.f ? 1.0e8f : 0.f));
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float x[16];
    const float4* p = reinterpret_cast<const float4*>(src + i * 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 v = p[j];
      x[4 * j] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(x[j]));
    float scale = __fmul_rn(gs, __fmul_rn(amax, 0.16666667163372039794921875f));
    scale = fminf(scale, 448.f);
    const uint8_t sfb = f32_to_e4m3(scale);
    const float os = out_scale_of(sfb, rcp_gs);
    codes[2 * i] = f32x8_to_e2m1(__fmul_rn(x[0], os), __fmul_rn(x[1], os), __fmul_rn(x[2], os), __fmul_rn(x[3], os),
                                 __fmul_rn(x[4], os), __fmul_rn(x[5], os), __fmul_rn(x[6], os), __fmul_rn(x[7], os));
    codes[2 * i + 1] = f32x8_to_e2m1(__fmul_rn(x[8], os), __fmul_rn(x[9], os), __fmul_rn(x[10], os), __fmul_rn(x[11], os),
                                     __fmul_rn(x[12], os), __fmul_rn(x[13], os), __fmul_rn(x[14], os), __fmul_rn(x[15], os));
    sf[i] = sfb;
  }
}

unsigned blocks_for(int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads;
  const int64_t cap = 8 * (int64_t)sm_count();
  if (b > cap) b = cap;
  return (unsigned)(b < 1 ? 1 : b);
}

int gemm_common(Handle* h, int M, int N, int K, const void* A, const uint8_t* A_scales, const void* B,
                const uint8_t* B_scales, float alpha, float* C) {
  if (M < 0 || N <= 0 || K <= 0 || (K % 64) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!A || !B || !C) return B200FP4_STATUS_INVALID_VALUE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != h->device) {
    cudaGetLastError();
    return B200FP4_STATUS_INVALID_VALUE;   // the handle belongs to the device that was current at cudaFP4Create
  }
  if (!ensure_scratch(h, scratch_need(M, N, K))) return B200FP4_STATUS_ALLOC_FAILED;
  const int64_t KB = K / 16, KT = (KB + 3) / 4;
  const int64_t mp = ((int64_t)M + 127) / 128 * 128, np = ((int64_t)N + 127) / 128 * 128;
  float* d_alpha = reinterpret_cast<float*>(h->scratch + 256);
  uint8_t* sfa = h->scratch + 512;
  uint8_t* sfb = sfa + round256(b200fp4_sf_swizzled_bytes(M, KB));
  cudaStream_t st = h->stream;
  if (A_scales) sf_swizzle_kernel<<<blocks_for(mp * KT * 4, 256), 256, 0, st>>>(A_scales, M, KB, mp, KT, sfa);
  else fill_bytes_kernel<<<blocks_for(mp * KT * 4, 256), 256, 0, st>>>(sfa, mp * KT * 4, 0x38);   // E4M3 1.0
  if (B_scales) sf_swizzle_kernel<<<blocks_for(np * KT * 4, 256), 256, 0, st>>>(B_scales, N, KB, np, KT, sfb);
  else fill_bytes_kernel<<<blocks_for(np * KT * 4, 256), 256, 0, st>>>(sfb, np * KT * 4, 0x38);
  set_float_kernel<<<1, 1, 0, st>>>(d_alpha, alpha);
  const int rc = finish_launch(3);
  if (rc != B200FP4_STATUS_SUCCESS) return rc;
  return b200fp4_gemm_nvfp4(A, B, sfa, sfb, d_alpha, C, B200FP4_DTYPE_F32, M, N, K, 0, h->scratch, 256, st);
}

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" int b200fp4_sf_swizzle(const void* sf_linear, int64_t rows, int64_t k_blocks, void* sf_swizzled, void* stream) {
  if (rows < 0 || k_blocks < 0) return B200FP4_STATUS_INVALID_VALUE;
  if (rows == 0 || k_blocks == 0) return B200FP4_STATUS_SUCCESS;
  if (!sf_linear || !sf_swizzled) return B200FP4_STATUS_INVALID_VALUE;
  const int64_t KT = (k_blocks + 3) / 4, rp = (rows + 127) / 128 * 128;
  sf_swizzle_kernel<<<blocks_for(rp * KT * 4, 256), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const uint8_t*>(sf_linear), rows, k_blocks, rp, KT, static_cast<uint8_t*>(sf_swizzled));
  return finish_launch(1);
}

extern "C" {

B200FP4_API int cudaFP4Create(cudaFP4Handle_t* handle) {
  if (!handle) return B200FP4_STATUS_INVALID_VALUE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_NOT_INITIALIZED;
  }
  if (b200fp4_has_hardware_acceleration() != 1) return B200FP4_STATUS_ARCH_MISMATCH;
  Handle* h = new (std::nothrow) Handle();
  if (!h) return B200FP4_STATUS_ALLOC_FAILED;
  h->device = dev;
  h->stream = nullptr;
  h->scratch = nullptr;
  h->scratch_bytes = 0;
  if (!ensure_scratch(h, scratch_need(8192, 8192, 8192))) {
    delete h;
    return B200FP4_STATUS_ALLOC_FAILED;
  }
  *handle = reinterpret_cast<cudaFP4Handle_t>(h);
  return B200FP4_STATUS_SUCCESS;
}

B200FP4_API int cudaFP4Destroy(cudaFP4Handle_t handle) {
  if (!handle) return B200FP4_STATUS_NOT_INITIALIZED;
  Handle* h = reinterpret_cast<Handle*>(handle);
  if (h->scratch) cudaFree(h->scratch);
  delete h;
  return B200FP4_STATUS_SUCCESS;
}

B200FP4_API int cudaFP4SetStream(cudaFP4Handle_t handle, void* stream) {
  if (!handle) return B200FP4_STATUS_NOT_INITIALIZED;
  reinterpret_cast<Handle*>(handle)->stream = (cudaStream_t)stream;
  return B200FP4_STATUS_SUCCESS;
}

B200FP4_API int cudaFP4GemmEx(cudaFP4Handle_t handle, int M, int N, int K, const void* A, const void* A_scales, float A_scale_global,
                              const void* B, const void* B_scales, float B_scale_global, float* C, int group_size) {
  if (!handle) return B200FP4_STATUS_NOT_INITIALIZED;
  if (group_size != 16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (!A_scales || !B_scales) return B200FP4_STATUS_INVALID_VALUE;
  return gemm_common(reinterpret_cast<Handle*>(handle), M, N, K, A, static_cast<const uint8_t*>(A_scales), B,
                     static_cast<const uint8_t*>(B_scales), A_scale_global * B_scale_global, C);
}

B200FP4_API int cudaFP4Gemm(cudaFP4Handle_t handle, int M, int N, int K, float alpha, const void* A, const void* B, float* C) {
  if (!handle) return B200FP4_STATUS_NOT_INITIALIZED;
  return gemm_common(reinterpret_cast<Handle*>(handle), M, N, K, A, nullptr, B, nullptr, alpha, C);
}

B200FP4_API const char* cudaFP4GetVersionString(void) { return b200fp4_version_string(); }
B200FP4_API int cudaFP4GetVersion(void) { return b200fp4_version(); }
B200FP4_API int cudaFP4HasHardwareAcceleration(void) { return b200fp4_has_hardware_acceleration(); }
B200FP4_API const char* cudaFP4GetErrorString(int status) { return b200fp4_get_error_string(status); }

B200FP4_API int cudaFP4ConvertFromFP32(void* dst, const float* src, int rows, int cols, void* stream) {
  if (rows < 0 || cols < 0 || (cols % 8) != 0) return B200FP4_STATUS_INVALID_VALUE;
  const int64_t n8 = (int64_t)rows * cols / 8;
  if (n8 == 0) return B200FP4_STATUS_SUCCESS;
  if (!dst || !src || !aligned(src, 16) || !aligned(dst, 4)) return B200FP4_STATUS_INVALID_VALUE;
  from_fp32_kernel<<<blocks_for(n8, 256), 256, 0, (cudaStream_t)stream>>>(src, n8, static_cast<uint32_t*>(dst));
  return finish_launch(1);
}

B200FP4_API int cudaFP4ConvertToFP32(float* dst, const void* src, int rows, int cols, void* stream) {
  if (rows < 0 || cols < 0 || (cols % 2) != 0) return B200FP4_STATUS_INVALID_VALUE;
  const int64_t n2 = (int64_t)rows * cols / 2;
  if (n2 == 0) return B200FP4_STATUS_SUCCESS;
  if (!dst || !src || !aligned(dst, 8)) return B200FP4_STATUS_INVALID_VALUE;
  to_fp32_kernel<<<blocks_for(n2, 256), 256, 0, (cudaStream_t)stream>>>(static_cast<const uint8_t*>(src), n2, dst);
  return finish_launch(1);
}

// dst_scale_global is a HOST pointer (cuda_fp4_gemm.h:186): the call synchronises `stream` to deliver it.  The
// amax lives for the duration of the call in a small device buffer allocated and freed here: this entry point
// has no handle to borrow scratch from.
B200FP4_API int cudaFP4Quantize(void* dst_data, void* dst_scales, float* dst_scale_global, const float* src, int rows,
                                int cols, int group_size, void* stream) {
  if (group_size != 16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (rows < 0 || cols < 0 || (cols % 16) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (!dst_scale_global) return B200FP4_STATUS_INVALID_VALUE;
  const int64_t n = (int64_t)rows * cols;
  if (n == 0) {
    *dst_scale_global = 0.f;
    return B200FP4_STATUS_SUCCESS;
  }
  if (!dst_data || !dst_scales || !src || !aligned(src, 16) || !aligned(dst_data, 4)) return B200FP4_STATUS_INVALID_VALUE;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned int* d_amax = nullptr;
  if (cudaMalloc(&d_amax, sizeof(unsigned int)) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_ALLOC_FAILED;
  }
  unsigned int bits = 0;
  int rc = B200FP4_STATUS_SUCCESS;
  if (cudaMemsetAsync(d_amax, 0, sizeof(unsigned int), st) != cudaSuccess) rc = B200FP4_STATUS_EXECUTION_FAILED;
  if (rc == B200FP4_STATUS_SUCCESS) {
    amax_kernel<<<blocks_for(n, 256), 256, 0, st>>>(src, n, d_amax);
    quantize_f32_kernel<<<blocks_for(n / 16, 128), 128, 0, st>>>(src, rows, cols, d_amax, static_cast<uint32_t*>(dst_data),
                                                                 static_cast<uint8_t*>(dst_scales));
    rc = finish_launch(2);
  }
  if (rc == B200FP4_STATUS_SUCCESS &&
      (cudaMemcpyAsync(&bits, d_amax, sizeof(bits), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
       cudaStreamSynchronize(st) != cudaSuccess))
    rc = B200FP4_STATUS_EXECUTION_FAILED;
  if (rc != B200FP4_STATUS_SUCCESS) cudaGetLastError();
  cudaFree(d_amax);
  if (rc == B200FP4_STATUS_SUCCESS) {
    float amax;
    memcpy(&amax, &bits, sizeof(float));
    *dst_scale_global = amax / (6.0f * 448.0f);
  }
  return rc;
}

}  // extern "C"
