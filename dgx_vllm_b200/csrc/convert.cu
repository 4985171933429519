// NVFP4 checkpoint layout -> 2:4 compressed layout of the sparse GEMV, on the GPU.
//
// Replaces the load-time Python loop of the reference (unpack_fp4_nibbles, apply_2of4_sparsity_fast,
// convert_expert_to_v7_gpu, convert_weight_batch_to_v7: sparse_fp4_kernel/sparse_v7_moe_patch.py:39-129),
// which runs torch.topk per expert for 512 experts x 48 layers.  One thread handles one metadata byte:
// eight consecutive k of one output row, i.e. two groups of four.  In every group the two codes of
// largest magnitude are kept; among equal magnitudes the LOWER index wins (torch.topk leaves that
// order unspecified, this rule is deterministic), and the kept indices are stored ascending.
// Outputs are transposed so that N is contiguous: comp_T [E, K/4, N], meta_T [E, K/8, N],
// scale_T [E, G, N] (plain transpose of the [E, N, G] block scales).
#include "common.cuh"

namespace b200fp4 {
namespace {

// magnitude rank of an E2M1 code is its low three bits (0, .5, 1, 1.5, 2, 3, 4, 6 are increasing)
__device__ __forceinline__ void top2_of4(uint32_t nibbles16, uint32_t& comp, uint32_t& meta) {
  uint32_t nib[4], mag[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    nib[j] = (nibbles16 >> (4 * j)) & 15u;
    mag[j] = nib[j] & 7u;
  }
  int a = 0;
#pragma unroll
  for (int j = 1; j < 4; ++j)
    if (mag[j] > mag[a]) a = j;
  int b = -1;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j == a) continue;
    if (b < 0 || mag[j] > mag[b]) b = j;
  }
  const int i0 = a < b ? a : b, i1 = a < b ? b : a;
  comp = nib[i0] | (nib[i1] << 4);
  meta = (uint32_t)i0 | ((uint32_t)i1 << 2);
}

__global__ void convert_2of4_kernel(const uint8_t* __restrict__ codes, int64_t E, int N, int K, uint8_t* __restrict__ comp_T,
                                    uint8_t* __restrict__ meta_T) {
  // x: output row n (fastest, so that the transposed stores are coalesced); y: metadata row; z: expert
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int mrow = blockIdx.y;
  const int64_t e = blockIdx.z;
  if (n >= N) return;
  const uint32_t w = *reinterpret_cast<const uint32_t*>(codes + (e * N + n) * (int64_t)(K / 2) + (int64_t)mrow * 4);
  uint32_t c0, m0, c1, m1;
  top2_of4(w & 0xFFFFu, c0, m0);
  top2_of4(w >> 16, c1, m1);
  comp_T[(e * (K / 4) + 2 * (int64_t)mrow) * N + n] = (uint8_t)c0;
  comp_T[(e * (K / 4) + 2 * (int64_t)mrow + 1) * N + n] = (uint8_t)c1;
  meta_T[(e * (K / 8) + mrow) * N + n] = (uint8_t)(m0 | (m1 << 4));
}

__global__ void transpose_scales_kernel(const uint8_t* __restrict__ sf, int64_t E, int N, int G, uint8_t* __restrict__ sf_T) {
  __shared__ uint8_t tile[32][33];
  const int64_t e = blockIdx.z;
  const int n0 = blockIdx.x * 32, g0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int n = n0 + i, g = g0 + threadIdx.x;
    if (n < N && g < G) tile[i][threadIdx.x] = sf[(e * N + n) * (int64_t)G + g];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int g = g0 + i, n = n0 + threadIdx.x;
    if (n < N && g < G) sf_T[(e * G + g) * (int64_t)N + n] = tile[threadIdx.x][i];
  }
}

}  // namespace
}  // namespace b200fp4

using namespace b200fp4;

extern "C" int b200fp4_convert_to_sparse_2of4(const uint8_t* codes, const uint8_t* scales, int64_t E, int64_t N, int64_t K,
                                              int64_t G, uint8_t* comp_T, uint8_t* meta_T, uint8_t* scale_T, void* stream) {
  if (E <= 0 || N <= 0 || K <= 0 || (K % 8) != 0 || G <= 0) return B200FP4_STATUS_INVALID_VALUE;
  if (!codes || !comp_T || !meta_T || !aligned(codes, 4)) return B200FP4_STATUS_INVALID_VALUE;
  if ((scales == nullptr) != (scale_T == nullptr)) return B200FP4_STATUS_INVALID_VALUE;
  if (E > 65535 || K / 8 > 65535 || N > (1 << 24)) return B200FP4_STATUS_NOT_SUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)(K / 8), (unsigned)E);
  convert_2of4_kernel<<<grid, 128, 0, st>>>(codes, E, (int)N, (int)K, comp_T, meta_T);
  int launches = 1;
  if (scales) {
    if ((G + 31) / 32 > 65535) return B200FP4_STATUS_NOT_SUPPORTED;
    dim3 tg((unsigned)((N + 31) / 32), (unsigned)((G + 31) / 32), (unsigned)E);
    transpose_scales_kernel<<<tg, dim3(32, 8), 0, st>>>(scales, E, (int)N, (int)G, scale_T);
    ++launches;
  }
  return finish_launch(launches);
}
