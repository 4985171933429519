// bf16/f16 -> NVFP4 quantizer for sm_100a.
//
// One thread owns 8 consecutive elements (one 16-byte load); two neighbouring lanes form one
// 16-element scale block and share the block maximum (found with packed 16-bit max) through a warp
// shuffle.  The per-block reciprocal depends only on the scale byte, so it is tabulated per block.  Codes leave as one
// 4-byte store per thread, so a warp reads 512 contiguous bytes per row segment and writes 128.
// Arithmetic follows ref_nvfp4_quant (vllm/model_executor/layers/quantization/utils/
// nvfp4_emulation_utils.py:439-453) operation by operation in IEEE fp32 -- explicit _rn
// intrinsics keep the compiler from contracting or approximating -- so codes and scales are
// bit-identical to the reference's emulation path; the E2M1 rounding itself is the native
// cvt.rn.satfinite.e2m1x2.f32 that replaces the reference's software routine
// (patch_nvfp4_utils_sw_e2m1.py:31-63).
#include "common.cuh"

namespace b200fp4 {

std::atomic<uint64_t> g_launch_count{0};

namespace {

constexpr int kTX = 64;    // threads along K (each 8 elements): 512 elements per block row
constexpr int kTY = 4;     // rows per block per pass
constexpr int kRows = 4;   // passes (rows) per thread, loads issued together

// Packed helpers on two 16-bit floats in one register.
template <typename T>
struct Pk;
template <>
struct Pk<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
};
template <>
struct Pk<__half> {
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  static __device__ __forceinline__ float lo(uint32_t w) { return __low2float(*reinterpret_cast<const __half2*>(&w)); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __high2float(*reinterpret_cast<const __half2*>(&w)); }
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float* v) {
  v[0] = Pk<T>::lo(raw.x); v[1] = Pk<T>::hi(raw.x); v[2] = Pk<T>::lo(raw.y); v[3] = Pk<T>::hi(raw.y);
  v[4] = Pk<T>::lo(raw.z); v[5] = Pk<T>::hi(raw.z); v[6] = Pk<T>::lo(raw.w); v[7] = Pk<T>::hi(raw.w);
}

// max |x| over the 8 packed values (exact: the maximum of 16-bit floats is one of them)
template <typename T>
__device__ __forceinline__ float amax8(const uint4& raw) {
  const uint32_t m = 0x7FFF7FFFu;
  const uint32_t w = Pk<T>::max2(Pk<T>::max2(raw.x & m, raw.y & m), Pk<T>::max2(raw.z & m, raw.w & m));
  return fmaxf(Pk<T>::lo(w), Pk<T>::hi(w));
}

// kExperts: per-row expert lookup (global scale + scale-factor row offset per expert).
// kSilu:    input is [M, 2K]; quantize round_to_T(silu(x[:, :K]) * x[:, K:]).
template <typename T, bool kSwizzled, bool kExperts, bool kSilu>
__global__ void __launch_bounds__(kTX* kTY)
    quantize_kernel(const T* __restrict__ x, int64_t M, int64_t K, int64_t ldx, const float* __restrict__ gs_ptr,
                    const int32_t* __restrict__ expert_offsets, const int32_t* __restrict__ blockscale_offsets,
                    int num_experts, uint8_t* __restrict__ codes, uint8_t* __restrict__ sf,
                    const int32_t* __restrict__ row_map, int row_div) {
  const int64_t kc = (int64_t)blockIdx.x * kTX + threadIdx.x;  // 8-element chunk index along K
  const int64_t CPR = K >> 3;
  const int64_t KB = K >> 4;
  const int64_t KT = (KB + 3) >> 2;
  const int64_t m0 = ((int64_t)blockIdx.y * kTY + threadIdx.y) * kRows;
  const bool col_ok = kc < CPR;

  uint4 raw[kRows], raw2[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    raw[r] = make_uint4(0, 0, 0, 0);
    raw2[r] = make_uint4(0, 0, 0, 0);
    const int64_t m = m0 + r;
    if (col_ok && m < M) {
      // optional gather: output row m is source row row_map[m] / row_div (a negative entry reads as zeros)
      int64_t src = m;
      if (row_map != nullptr) {
        const int v = row_map[m];
        src = v < 0 ? -1 : (int64_t)(v / row_div);
      }
      if (src >= 0) {
        raw[r] = *reinterpret_cast<const uint4*>(x + src * ldx + kc * 8);
        if (kSilu) raw2[r] = *reinterpret_cast<const uint4*>(x + src * ldx + K + kc * 8);
      }
    }
  }

  // With one global scale for the whole call the multiplier applied to the elements depends only on the
  // block-scale byte (127 values): each block tabulates it once with the exact arithmetic.
  __shared__ float s_os[128];
  // Per-expert mode: the block's 16 rows look their expert up once each (not once per thread):
  // global scale, its guarded reciprocal and the row of the scale-factor tensor.
  __shared__ float s_gs[kTY * kRows], s_rcp[kTY * kRows];
  __shared__ long long s_sfrow[kTY * kRows];
  float gs_shared = 0.f;
  if (!kExperts) {
    gs_shared = gs_ptr[0];
    const int t = threadIdx.y * kTX + threadIdx.x;
    if (t < 128) s_os[t] = out_scale_of((uint8_t)t, __frcp_rn(gs_shared + (gs_shared == 0.f ? 1.0e8f : 0.f)));
    __syncthreads();
  } else {
    const int t = threadIdx.y * kTX + threadIdx.x;
    if (t < kTY * kRows) {
      // slot t = (threadIdx.y = t / kRows, pass r = t % kRows) holds row (blockIdx.y * kTY + t / kRows) * kRows + t % kRows
      const int64_t m = ((int64_t)blockIdx.y * kTY + t / kRows) * kRows + t % kRows;
      float gs = 0.f;
      long long row = m;
      if (m < M) {
        int lo = 0, hi = num_experts - 1;      // largest e with expert_offsets[e] <= m
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if ((int64_t)expert_offsets[mid] <= m) lo = mid;
          else hi = mid - 1;
        }
        gs = gs_ptr[lo];
        row = (long long)blockscale_offsets[lo] + (m - (long long)expert_offsets[lo]);
      }
      s_gs[t] = gs;
      s_rcp[t] = __frcp_rn(gs + (gs == 0.f ? 1.0e8f : 0.f));
      s_sfrow[t] = row;
    }
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const int64_t m = m0 + r;
    const bool ok = col_ok && m < M;
    float v[8];
    float amax;
    if (kSilu) {
      float u[8];
      unpack8<T>(raw[r], v);
      unpack8<T>(raw2[r], u);
      amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = to_f32<T>(from_f32<T>(silu_f32(v[i]) * u[i]));
        amax = fmaxf(amax, fabsf(v[i]));
      }
    } else {
      amax = amax8<T>(raw[r]);
      unpack8<T>(raw[r], v);
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));

    float gs = gs_shared;
    int64_t sf_row = m;
    if (kExperts) {
      gs = s_gs[threadIdx.y * kRows + r];
      sf_row = s_sfrow[threadIdx.y * kRows + r];
    }

    float scale = __fmul_rn(gs, __fmul_rn(amax, 0.16666667163372039794921875f));  // fl32(1/6)
    scale = fminf(scale, 448.f);
    const uint8_t sfb = f32_to_e4m3(scale);
    float os;
    if (kExperts) os = out_scale_of(sfb, s_rcp[threadIdx.y * kRows + r]);
    else os = s_os[sfb & 127];

    const uint32_t packed =
        f32x8_to_e2m1(__fmul_rn(v[0], os), __fmul_rn(v[1], os), __fmul_rn(v[2], os), __fmul_rn(v[3], os),
                      __fmul_rn(v[4], os), __fmul_rn(v[5], os), __fmul_rn(v[6], os), __fmul_rn(v[7], os));
    if (ok) {
      *reinterpret_cast<uint32_t*>(codes + m * (K >> 1) + kc * 4) = packed;
      if ((kc & 1) == 0) {
        const int64_t kb = kc >> 1;
        if (kSwizzled) sf[sf_swizzled_offset(sf_row, kb, KT)] = sfb;
        else sf[sf_row * KB + kb] = sfb;
      }
    }
  }
}

// Token-major form of the gather above: block t reads source row t once and quantizes it for each of its
// `topk` destination rows src2dst[t*topk + s] (negative = no destination), each with the global scale of the
// expert that owns the destination row.  Same bytes as quantizing the gathered rows one by one; the source is
// read once instead of topk times.
constexpr int kScatterMaxTopk = 32;
constexpr int kScatterThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kScatterThreads)
    experts_quantize_scatter_kernel(const T* __restrict__ x, int64_t K, int topk, const int32_t* __restrict__ src2dst,
                                    const float* __restrict__ gs_ptr, const int32_t* __restrict__ expert_offsets,
                                    const int32_t* __restrict__ blockscale_offsets, int num_experts,
                                    const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map,
                                    int global_E, uint8_t* __restrict__ codes, uint8_t* __restrict__ sf) {
  __shared__ float s_gs[kScatterMaxTopk], s_rcp[kScatterMaxTopk];
  __shared__ long long s_sfrow[kScatterMaxTopk], s_code[kScatterMaxTopk];
  __shared__ int s_dst[kScatterMaxTopk];
  const int64_t t = blockIdx.x;
  const int64_t CPR = K >> 3, KB = K >> 4, KT = (KB + 3) >> 2;
  // the first chunk of the row is requested before the destination lookup, so the two latencies overlap
  uint4 raw_first = make_uint4(0, 0, 0, 0);
  if ((int64_t)threadIdx.x < CPR) raw_first = *reinterpret_cast<const uint4*>(x + t * K + (int64_t)threadIdx.x * 8);
  if ((int)threadIdx.x < topk) {
    const int dst = src2dst[t * topk + threadIdx.x];
    float gs = 0.f;
    long long row = 0;
    if (dst >= 0) {
      int lo;
      if (topk_ids != nullptr) {
        // the pair's routing entry names the expert directly
        lo = topk_ids[t * topk + threadIdx.x];
        if (expert_map != nullptr) lo = (lo >= 0 && lo < global_E) ? expert_map[lo] : 0;
        lo = min(max(lo, 0), num_experts - 1);
      } else {
        lo = 0;
        int hi = num_experts - 1;            // largest e with expert_offsets[e] <= dst
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (expert_offsets[mid] <= dst) lo = mid;
          else hi = mid - 1;
        }
      }
      gs = gs_ptr[lo];
      row = (long long)blockscale_offsets[lo] + (dst - expert_offsets[lo]);
    }
    s_dst[threadIdx.x] = dst;
    s_gs[threadIdx.x] = gs;
    s_rcp[threadIdx.x] = __frcp_rn(gs + (gs == 0.f ? 1.0e8f : 0.f));
    // byte offsets of the destination row in the code tensor and of its first scale byte, computed once per block
    s_sfrow[threadIdx.x] = sf_swizzled_offset(row, 0, KT);
    s_code[threadIdx.x] = (long long)dst * (long long)(K >> 1);
  }
  __syncthreads();
  for (int64_t base = 0; base < CPR; base += kScatterThreads) {
    const int64_t kc = base + threadIdx.x;
    const bool ok = kc < CPR;
    uint4 raw = raw_first;
    if (base > 0) {
      raw = make_uint4(0, 0, 0, 0);
      if (ok) raw = *reinterpret_cast<const uint4*>(x + t * K + kc * 8);
    }
    float amax = amax8<T>(raw);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    float v[8];
    unpack8<T>(raw, v);
    const float sixth = __fmul_rn(amax, 0.16666667163372039794921875f);
    const int64_t kb = kc >> 1;
    const int64_t sf_col = (kb >> 2) * 512 + (kb & 3);     // scale byte of this block of 16 relative to its row's first
    for (int sl = 0; sl < topk; ++sl) {
      const int dst = s_dst[sl];
      if (dst < 0 || !ok) continue;
      const float scale = fminf(__fmul_rn(s_gs[sl], sixth), 448.f);
      const uint8_t sfb = f32_to_e4m3(scale);
      const float os = out_scale_of(sfb, s_rcp[sl]);
      const uint32_t packed =
          f32x8_to_e2m1(__fmul_rn(v[0], os), __fmul_rn(v[1], os), __fmul_rn(v[2], os), __fmul_rn(v[3], os),
                        __fmul_rn(v[4], os), __fmul_rn(v[5], os), __fmul_rn(v[6], os), __fmul_rn(v[7], os));
      *reinterpret_cast<uint32_t*>(codes + s_code[sl] + kc * 4) = packed;
      if ((kc & 1) == 0) sf[s_sfrow[sl] + sf_col] = sfb;
    }
  }
}

template <typename T, bool kSwz, bool kExp, bool kSilu>
void launch(const void* x, int64_t M, int64_t K, int64_t ldx, const float* gs, const int32_t* eo, const int32_t* bo,
            int ne, void* codes, void* sf, cudaStream_t st, const int32_t* row_map = nullptr, int row_div = 1) {
  dim3 block(kTX, kTY);
  dim3 grid((unsigned)(((K >> 3) + kTX - 1) / kTX), (unsigned)((M + kTY * kRows - 1) / (kTY * kRows)));
  quantize_kernel<T, kSwz, kExp, kSilu><<<grid, block, 0, st>>>(reinterpret_cast<const T*>(x), M, K, ldx, gs, eo, bo,
                                                                ne, (uint8_t*)codes, (uint8_t*)sf, row_map, row_div);
}

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" size_t b200fp4_sf_swizzled_bytes(int64_t rows, int64_t k_blocks) {
  if (rows < 0 || k_blocks < 0) return 0;
  return (size_t)(((rows + 127) / 128) * 128 * (((k_blocks + 3) / 4) * 4));
}

extern "C" int b200fp4_quantize(const void* x, int in_dtype, int64_t M, int64_t K, int64_t ldx,
                                const float* global_scale, void* codes, void* sf, int sf_swizzled, void* stream) {
  if (M < 0 || K <= 0 || (K % 16) != 0 || ldx < K || (ldx % 8) != 0) return B200FP4_STATUS_INVALID_VALUE;
  if (in_dtype != B200FP4_DTYPE_F16 && in_dtype != B200FP4_DTYPE_BF16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (M == 0) return B200FP4_STATUS_SUCCESS;
  if (!x || !global_scale || !codes || !sf) return B200FP4_STATUS_INVALID_VALUE;
  if (!aligned(x, 16) || !aligned(codes, 4)) return B200FP4_STATUS_INVALID_VALUE;
  if (M > (int64_t)65535 * kTY * kRows) return B200FP4_STATUS_NOT_SUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  int n_launch = 1;
  const int64_t KB = K / 16;
  if (sf_swizzled && ((M % 128) != 0 || (KB % 4) != 0)) {
    if (cudaMemsetAsync(sf, 0, b200fp4_sf_swizzled_bytes(M, KB), st) != cudaSuccess) {
      cudaGetLastError();
      return B200FP4_STATUS_EXECUTION_FAILED;
    }
    ++n_launch;
  }
  const bool bf = in_dtype == B200FP4_DTYPE_BF16;
  if (sf_swizzled) {
    if (bf) launch<__nv_bfloat16, true, false, false>(x, M, K, ldx, global_scale, nullptr, nullptr, 0, codes, sf, st);
    else launch<__half, true, false, false>(x, M, K, ldx, global_scale, nullptr, nullptr, 0, codes, sf, st);
  } else {
    if (bf) launch<__nv_bfloat16, false, false, false>(x, M, K, ldx, global_scale, nullptr, nullptr, 0, codes, sf, st);
    else launch<__half, false, false, false>(x, M, K, ldx, global_scale, nullptr, nullptr, 0, codes, sf, st);
  }
  return finish_launch(n_launch);
}

static int experts_quantize_impl(const void* x, int in_dtype, int64_t M, int64_t K, const float* global_scales,
                                 const int32_t* expert_offsets, const int32_t* blockscale_offsets, int32_t num_experts,
                                 int64_t sf_rows_padded, int silu_mul, void* codes, void* sf, void* stream,
                                 const int32_t* row_map, int row_div) {
  if (M < 0 || K <= 0 || (K % 16) != 0 || num_experts <= 0 || sf_rows_padded < 0 || (sf_rows_padded % 128) != 0)
    return B200FP4_STATUS_INVALID_VALUE;
  if (in_dtype != B200FP4_DTYPE_F16 && in_dtype != B200FP4_DTYPE_BF16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (!global_scales || !expert_offsets || !blockscale_offsets || !sf) return B200FP4_STATUS_INVALID_VALUE;
  if (M > 0 && (!x || !codes || !aligned(x, 16) || !aligned(codes, 4))) return B200FP4_STATUS_INVALID_VALUE;
  if (M > (int64_t)65535 * kTY * kRows) return B200FP4_STATUS_NOT_SUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t KB = K / 16;
  if (cudaMemsetAsync(sf, 0, (size_t)(sf_rows_padded * (((KB + 3) / 4) * 4)), st) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  if (M == 0) return finish_launch(1);
  const bool bf = in_dtype == B200FP4_DTYPE_BF16;
  const int64_t ldx = silu_mul ? 2 * K : K;
  if (silu_mul) {
    if (bf) launch<__nv_bfloat16, true, true, true>(x, M, K, ldx, global_scales, expert_offsets, blockscale_offsets, num_experts, codes, sf, st, row_map, row_div);
    else launch<__half, true, true, true>(x, M, K, ldx, global_scales, expert_offsets, blockscale_offsets, num_experts, codes, sf, st, row_map, row_div);
  } else {
    if (bf) launch<__nv_bfloat16, true, true, false>(x, M, K, ldx, global_scales, expert_offsets, blockscale_offsets, num_experts, codes, sf, st, row_map, row_div);
    else launch<__half, true, true, false>(x, M, K, ldx, global_scales, expert_offsets, blockscale_offsets, num_experts, codes, sf, st, row_map, row_div);
  }
  return finish_launch(2);
}

extern "C" int b200fp4_experts_quantize(const void* x, int in_dtype, int64_t M, int64_t K, const float* global_scales,
                                        const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                        int32_t num_experts, int64_t sf_rows_padded, int silu_mul, void* codes,
                                        void* sf, void* stream) {
  return experts_quantize_impl(x, in_dtype, M, K, global_scales, expert_offsets, blockscale_offsets, num_experts,
                               sf_rows_padded, silu_mul, codes, sf, stream, nullptr, 1);
}

extern "C" int b200fp4_experts_quantize_scatter(const void* x, int in_dtype, int64_t n_src, int64_t K, int64_t topk,
                                                const int32_t* src2dst, const float* global_scales,
                                                const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                                int32_t num_experts, int64_t sf_rows_padded, const int32_t* topk_ids,
                                                const int32_t* expert_map, int64_t global_E, void* codes, void* sf,
                                                void* stream) {
  if (expert_map && (!topk_ids || global_E <= 0)) return B200FP4_STATUS_INVALID_VALUE;
  if (n_src < 0 || K <= 0 || (K % 16) != 0 || topk <= 0 || num_experts <= 0 || sf_rows_padded < 0 ||
      (sf_rows_padded % 128) != 0)
    return B200FP4_STATUS_INVALID_VALUE;
  if (in_dtype != B200FP4_DTYPE_F16 && in_dtype != B200FP4_DTYPE_BF16) return B200FP4_STATUS_NOT_SUPPORTED;
  if (topk > kScatterMaxTopk || n_src > 0x7FFFFFFF) return B200FP4_STATUS_NOT_SUPPORTED;
  if (!global_scales || !expert_offsets || !blockscale_offsets || !sf) return B200FP4_STATUS_INVALID_VALUE;
  if (n_src > 0 && (!x || !codes || !src2dst || !aligned(x, 16) || !aligned(codes, 4))) return B200FP4_STATUS_INVALID_VALUE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t KB = K / 16;
  if (cudaMemsetAsync(sf, 0, (size_t)(sf_rows_padded * (((KB + 3) / 4) * 4)), st) != cudaSuccess) {
    cudaGetLastError();
    return B200FP4_STATUS_EXECUTION_FAILED;
  }
  if (n_src == 0) return finish_launch(1);
  if (in_dtype == B200FP4_DTYPE_BF16)
    experts_quantize_scatter_kernel<__nv_bfloat16><<<(unsigned)n_src, kScatterThreads, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), K, (int)topk, src2dst, global_scales, expert_offsets, blockscale_offsets,
        num_experts, topk_ids, expert_map, (int)global_E, (uint8_t*)codes, (uint8_t*)sf);
  else
    experts_quantize_scatter_kernel<__half><<<(unsigned)n_src, kScatterThreads, 0, st>>>(
        reinterpret_cast<const __half*>(x), K, (int)topk, src2dst, global_scales, expert_offsets, blockscale_offsets,
        num_experts, topk_ids, expert_map, (int)global_E, (uint8_t*)codes, (uint8_t*)sf);
  return finish_launch(2);
}

extern "C" int b200fp4_experts_quantize_gather(const void* x, int in_dtype, int64_t M, int64_t K, const float* global_scales,
                                               const int32_t* expert_offsets, const int32_t* blockscale_offsets,
                                               int32_t num_experts, int64_t sf_rows_padded, const int32_t* row_map,
                                               int32_t row_div, void* codes, void* sf, void* stream) {
  if (!row_map || row_div <= 0) return B200FP4_STATUS_INVALID_VALUE;
  return experts_quantize_impl(x, in_dtype, M, K, global_scales, expert_offsets, blockscale_offsets, num_experts,
                               sf_rows_padded, 0, codes, sf, stream, row_map, row_div);
}
