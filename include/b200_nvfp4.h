/*
 * b200_nvfp4.h -- C ABI of libb200nvfp4.so: the NVFP4 hot path for NVIDIA B200 (sm_100a).
 *
 * Conventions (all entry points)
 *   - Every function returns a b200fp4Status_t (values identical to the reference's
 *     cudaFP4Status_t, cutlass_nvfp4/cuda_fp4_gemm.h:33-42).  No function prints, synchronises
 *     the device, reads device memory on the host or allocates device memory.
 *   - Tensor arguments are BORROWED device pointers with explicit sizes; dtype selectors are the
 *     B200FP4_DTYPE_* ints.  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *   - Scalars that the caller keeps on the device (global scales, alpha) are passed as device
 *     pointers so a call sequence can be captured into a CUDA graph.
 *   - Work is enqueued on `stream`; a non-zero status means nothing was enqueued, except
 *     B200FP4_STATUS_EXECUTION_FAILED which reports a launch error from the CUDA runtime.
 *   - Packed E2M1 codes: element 2i in the low nibble, 2i+1 in the high nibble of byte i
 *     (patch_nvfp4_utils_sw_e2m1.py:48-63).  Block scales are E4M3 bytes, one per 16 elements
 *     along K.
 *
 * Each declaration names the reference interface it replaces (path:line inside the
 * Avarok-Cybersecurity/dgx-vllm tree; "vllm/..." = the vLLM tree that project patches).
 */
#ifndef B200_NVFP4_H_
#define B200_NVFP4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200FP4_API
#else
#define B200FP4_API __attribute__((visibility("default")))
#endif

/* Replaces cudaFP4Status_t, cutlass_nvfp4/cuda_fp4_gemm.h:33-42 (same numeric values). */
typedef enum {
  B200FP4_STATUS_SUCCESS = 0,
  B200FP4_STATUS_NOT_INITIALIZED = 1,
  B200FP4_STATUS_ALLOC_FAILED = 3,
  B200FP4_STATUS_INVALID_VALUE = 7,
  B200FP4_STATUS_ARCH_MISMATCH = 8,
  B200FP4_STATUS_EXECUTION_FAILED = 13,
  B200FP4_STATUS_INTERNAL_ERROR = 14,
  B200FP4_STATUS_NOT_SUPPORTED = 15
} b200fp4Status_t;

enum { B200FP4_DTYPE_F16 = 0, B200FP4_DTYPE_BF16 = 1, B200FP4_DTYPE_F32 = 2 };

/* ---------------------------------------------------------------------------------------------
 * Utilities.  Replace cudaFP4GetErrorString / cudaFP4GetVersion / cudaFP4GetVersionString /
 * cudaFP4HasHardwareAcceleration, cutlass_nvfp4/cuda_fp4_gemm.h:124-147.
 * ------------------------------------------------------------------------------------------- */
B200FP4_API const char* b200fp4_get_error_string(int status);
B200FP4_API int b200fp4_version(void);
B200FP4_API const char* b200fp4_version_string(void);
/* 1 when the current device is compute capability 10.x (tcgen05 / native E2M1 cvt), else 0. */
B200FP4_API int b200fp4_has_hardware_acceleration(void);
/* Number of kernels this library has launched in the calling process (monotonic counter). */
B200FP4_API uint64_t b200fp4_launch_count(void);

/* ---------------------------------------------------------------------------------------------
 * Part 1 -- activation quantizer.
 * Replaces the scaled_fp4_quant op (vllm/_custom_ops.py:1600-1671) whose device code the
 * reference patches with fp32_vec8_to_e2m1 / fp32_vec16_to_e2m1
 * (patch_nvfp4_utils_sw_e2m1.py:105-131,168-193,236-274); arithmetic order is that of
 * ref_nvfp4_quant as called at fix_nvfp4_emulation_backend.py:72.
 *
 *   x            [M, K] bf16 or f16 (in_dtype), row stride ldx elements, K % 16 == 0
 *   global_scale device pointer to one f32 (= 448*6/amax, vLLM's input_global_scale)
 *   codes        [M, K/2] u8 out
 *   sf           e4m3 out: linear [M, K/16], or, when sf_swizzled != 0, the padded 128x4 tile
 *                layout of b200fp4_sf_swizzled_bytes(M, K/16) bytes.  Padding bytes of the
 *                swizzled layout are written as zero by this call.
 * ------------------------------------------------------------------------------------------- */
B200FP4_API size_t b200fp4_sf_swizzled_bytes(int64_t rows, int64_t k_blocks);
/* Linear block scales [rows, k_blocks] -> the padded 128x4 tile layout (padding = 0): what a checkpoint's weight
 * scales need once at load time.  Replaces swizzle_blockscale, vllm/model_executor/layers/quantization/utils/
 * nvfp4_utils.py:38-51. */
B200FP4_API int b200fp4_sf_swizzle(const void* sf_linear, int64_t rows, int64_t k_blocks, void* sf_swizzled,
                                   void* stream);
B200FP4_API int b200fp4_quantize(const void* x, int in_dtype, int64_t M, int64_t K, int64_t ldx,
                                 const float* global_scale, void* codes, void* sf, int sf_swizzled,
                                 void* stream);

/* Per-expert variant.  Replaces scaled_fp4_experts_quant(output, output_scales, input,
 * input_global_scale, expert_offsets, blockscale_offsets), vllm/_custom_ops.py:1674-1733 (one of
 * the five NVFP4 sources the reference force-compiles, cmake_patch_gb10_nvfp4_v6_full_kernels.sh:58-62).
 * Rows [expert_offsets[e], expert_offsets[e+1]) use global_scales[e]; their scale factors go to
 * swizzled rows starting at blockscale_offsets[e] (a multiple of 128).  sf must hold
 * sf_rows_padded * ceil(K/64)*4 bytes and is fully written (padding = 0).
 * If silu_mul != 0 the input is [M, 2K] and SiLU(x[:, :K]) * x[:, K:] is quantized instead
 * (silu_and_mul_scaled_fp4_experts_quant, same file list). */
B200FP4_API int b200fp4_experts_quantize(const void* x, int in_dtype, int64_t M, int64_t K,
                                         const float* global_scales, const int32_t* expert_offsets,
                                         const int32_t* blockscale_offsets, int32_t num_experts,
                                         int64_t sf_rows_padded, int silu_mul, void* codes, void* sf,
                                         void* stream);

/* The same with the row permutation folded in: output row m quantizes source row
 * row_map[m] / row_div of x (a negative entry quantizes a row of zeros), i.e. shuffle_rows
 * (vllm/_custom_ops.py:1017-1054) followed by scaled_fp4_experts_quant without the [M, K] copy in
 * between.  x has as many rows as the map refers to. */
B200FP4_API int b200fp4_experts_quantize_gather(const void* x, int in_dtype, int64_t M, int64_t K,
                                                const float* global_scales, const int32_t* expert_offsets,
                                                const int32_t* blockscale_offsets, int32_t num_experts,
                                                int64_t sf_rows_padded, const int32_t* row_map,
                                                int32_t row_div, void* codes, void* sf, void* stream);

/* The same result computed token-major: source row t (of n_src) is read once and quantized for each of
 * its topk destination rows src2dst[t*topk + s] (the pair -> permuted row map of b200fp4_moe_permute;
 * negative = the pair has no local destination), each with the global scale of the expert owning the
 * destination row.  Destination rows that no pair maps to are not written.  topk <= 32.
 * topk_ids [n_src, topk] (+ expert_map [global_E] or NULL), when given, must be the routing the map was
 * built from: the owning expert is then read from it instead of searched for in expert_offsets. */
B200FP4_API int b200fp4_experts_quantize_scatter(const void* x, int in_dtype, int64_t n_src, int64_t K,
                                                 int64_t topk, const int32_t* src2dst,
                                                 const float* global_scales,
                                                 const int32_t* expert_offsets,
                                                 const int32_t* blockscale_offsets, int32_t num_experts,
                                                 int64_t sf_rows_padded, const int32_t* topk_ids,
                                                 const int32_t* expert_map, int64_t global_E,
                                                 void* codes, void* sf, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Part 2 -- dense block-scaled NVFP4 GEMM:  out[M,N] = alpha * (a . sfa)(b . sfb)^T.
 * Replaces cudaFP4GemmEx (declared, never defined) of cutlass_nvfp4/cuda_fp4_gemm.h:94-105 and the
 * software kernel launch_nvfp4_gemm (cutlass_nvfp4/nvfp4_gemm_kernel.cuh:350-386), with the
 * argument convention of the op vLLM serves with, cutlass_scaled_fp4_mm(out, a, b, block_scale_a,
 * block_scale_b, alpha) (vllm/_custom_ops.py:741-753), which the reference enables at
 * cmake_patch_gb10_nvfp4_v6_full_kernels.sh:50-64.
 *
 *   a_codes [M, K/2] u8, b_codes [N, K/2] u8 (K-major packed E2M1), K % 64 == 0
 *   sfa, sfb  E4M3 block scales in the padded 128x4-tile swizzled layout
 *             (b200fp4_sf_swizzled_bytes(rows, K/16) bytes each)
 *   alpha     device pointer to one f32 (= 1 / (global_scale_a * global_scale_b))
 *   out       [M, N] bf16, f16 or f32 (f32: the accumulator times alpha, unrounded)
 *   tile_n    0 = choose; 128 or 256 forces the CTA tile width (128 x tile_n output tiles);
 *             512 forces 256 x 256 tiles on pairs of CTAs (tcgen05 cta_group::2; 16-bit output only)
 *   workspace b200fp4_gemm_workspace_bytes() bytes; its first int is a status word the kernel
 *             leaves at 0 unless one of its bounded barrier waits expired (then nothing it wrote
 *             may be trusted): read it after synchronising when diagnosing.
 * ------------------------------------------------------------------------------------------- */
B200FP4_API size_t b200fp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
B200FP4_API int b200fp4_gemm_nvfp4(const void* a_codes, const void* b_codes, const void* sfa,
                                   const void* sfb, const float* alpha, void* out, int out_dtype,
                                   int64_t M, int64_t N, int64_t K, int tile_n, void* workspace,
                                   size_t workspace_bytes, void* stream);

/* The whole linear layer y = NVFP4(x) @ W^T in one call: b200fp4_quantize (swizzled scales) into the workspace, then
 * b200fp4_gemm_nvfp4.  What NvFp4LinearKernel.apply_weights does with two ops (scaled_fp4_quant then
 * cutlass_scaled_fp4_mm: vllm/model_executor/layers/quantization/utils/nvfp4_utils.py, the call pair the reference's
 * emulation replaces at fix_nvfp4_emulation_backend.py:60-102); one host call keeps the two launches a few
 * microseconds apart.  x [M, K] bf16/f16 with row stride ldx; x_global_scale, alpha device pointers as above.
 * workspace: b200fp4_linear_workspace_bytes(M, N, K) bytes, 256-byte aligned. */
B200FP4_API size_t b200fp4_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
B200FP4_API int b200fp4_linear_nvfp4(const void* x, int x_dtype, int64_t ldx, const float* x_global_scale,
                                     const void* w_codes, const void* w_sf, const float* alpha, void* out,
                                     int out_dtype, int64_t M, int64_t N, int64_t K, int tile_n,
                                     void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Part 3 -- 2:4-sparse / dense NVFP4 batched GEMV for MoE decode.
 * Replace the pybind functions of sparse_fp4_kernel/sparse_fp4_v7.cu:744-749.
 *
 * Common arguments
 *   A          [P, K] activations (a_dtype f16 or bf16), one row per (token, expert) pair
 *   scales_T   [E, G, N] e4m3, G = K/16 or K/8 (one scale per K/G consecutive k)
 *   g_scales   [E] f32
 *   expert_ids [P] i32; ids outside [0, E) produce a zero row (the reference indexes out of
 *              bounds there)
 *   out        [P, N] (out_dtype f16 or bf16)
 *   workspace  b200fp4_sparse_workspace_bytes(P, K, E) bytes of scratch, 256-byte aligned
 * N % 16 == 0 selects the vectorised kernel; other N fall back to a scalar kernel.
 *
 * flags (also the `flags` of the fused layer below):
 *   B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT  fused layer only, see there
 *   B200FP4_SPARSE_META_ORDERED         the caller promises that in every 4-group of Meta_T_pk the
 *       first 2-bit index is smaller than the second.  That is how the reference's converter writes
 *       them (sparse_v7_moe_patch.py:59-60, top-2 positions sorted) and what
 *       b200fp4_convert_to_sparse_2of4 produces.  With the promise (and G = K/16, N a multiple of
 *       512, or of 256 / 128 as K allows) the GEMV runs on the tensor cores (mma.sp, whose metadata
 *       operand requires ordered indices); results with unordered or repeated indices are then
 *       undefined.  Without it any index pair is accepted, as in the reference kernel.
 * ------------------------------------------------------------------------------------------- */
#define B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT 1
#define B200FP4_SPARSE_META_ORDERED 2
#define B200FP4_MOE_SEPARATE_LAUNCHES 4   /* fused layer: one launch per projection even where one cooperative launch is possible */
#define B200FP4_MOE_HOST_DIRECT_OUT 8     /* b200fp4_fused_sparse_moe_host_async only, see there */

B200FP4_API size_t b200fp4_sparse_workspace_bytes(int64_t P, int64_t K, int64_t E);

/* batched_sparse_v7(A, B_comp_T, Meta_T_pk, scales_T, g_scales, expert_ids),
 * sparse_fp4_v7.cu:374-406.  B_comp_T [E, K/4, N], Meta_T_pk [E, K/8, N]. */
B200FP4_API int b200fp4_sparse_gemv(const void* A, int a_dtype, const uint8_t* B_comp_T,
                                    const uint8_t* Meta_T_pk, const uint8_t* scales_T,
                                    const float* g_scales, const int32_t* expert_ids, void* out,
                                    int out_dtype, int64_t P, int64_t N, int64_t K, int64_t G,
                                    int64_t E, int flags, void* workspace, size_t workspace_bytes,
                                    void* stream);

/* b200fp4_sparse_gemv (flags = 0) without a caller workspace.  No counterpart in the reference: it exists
 * for hosts that cannot allocate device memory around the call -- e.g. a plug-in inside a serving
 * process whose pool already owns the GPU's memory, or a loop that bans cudaMalloc/cudaFree because
 * they synchronise the device.  The scratch is a fixed ~4.2 MB array inside the library (resident on
 * every GPU that loads it, until exit), so the call is limited to P <= 512 pairs, K <= 4096 and
 * E <= 4096; larger sizes return B200FP4_STATUS_NOT_SUPPORTED and enqueue nothing.  Same arguments,
 * results and validation as b200fp4_sparse_gemv otherwise; it calls no allocator.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress): make
 * that first call outside any stream capture.  All calls on a GPU share the array, which keeps the
 * previous call's contents (nothing needs clearing: every word read is rewritten first); calls
 * that overlap on the GPU race on it, so issue them on one stream or otherwise serialise them. */
B200FP4_API int b200fp4_sparse_gemv_static(const void* A, int a_dtype, const uint8_t* B_comp_T,
                                           const uint8_t* Meta_T_pk, const uint8_t* scales_T,
                                           const float* g_scales, const int32_t* expert_ids,
                                           void* out, int out_dtype, int64_t P, int64_t N, int64_t K,
                                           int64_t G, int64_t E, void* stream);

/* batched_dense_v7(A, B_dense_T, scales_T, g_scales, expert_ids), sparse_fp4_v7.cu:341-372.
 * B_dense_T [E, K/2, N]. */
B200FP4_API int b200fp4_dense_gemv(const void* A, int a_dtype, const uint8_t* B_dense_T,
                                   const uint8_t* scales_T, const float* g_scales,
                                   const int32_t* expert_ids, void* out, int out_dtype, int64_t P,
                                   int64_t N, int64_t K, int64_t G, int64_t E, void* workspace,
                                   size_t workspace_bytes, void* stream);

/* batched_sparse_packed_v7(A, B_packed_T, g_scales, expert_ids, orig_K), sparse_fp4_v7.cu:408-436.
 * B_packed_T [E, K/8, 4N]: per row comp0 | comp1 | meta | scale, one scale per 8 k. */
B200FP4_API int b200fp4_sparse_packed_gemv(const void* A, int a_dtype, const uint8_t* B_packed_T,
                                           const float* g_scales, const int32_t* expert_ids,
                                           void* out, int out_dtype, int64_t P, int64_t N, int64_t K,
                                           int64_t E, void* workspace, size_t workspace_bytes,
                                           void* stream);

/* Load-time converter: NVFP4 expert weights [E, N, K/2] (+ block scales [E, N, G]) -> the 2:4
 * compressed, N-contiguous tensors above (comp_T [E,K/4,N], meta_T [E,K/8,N], scale_T [E,G,N]).
 * Replaces unpack_fp4_nibbles / apply_2of4_sparsity_fast / convert_expert_to_v7_gpu /
 * convert_weight_batch_to_v7, sparse_fp4_kernel/sparse_v7_moe_patch.py:39-129.  Per group of four the
 * two largest magnitudes are kept, ties resolved towards the lower index (the reference's
 * torch.topk leaves ties unspecified), indices stored ascending.  scales / scale_T may both be NULL. */
B200FP4_API int b200fp4_convert_to_sparse_2of4(const uint8_t* codes, const uint8_t* scales, int64_t E,
                                               int64_t N, int64_t K, int64_t G, uint8_t* comp_T,
                                               uint8_t* meta_T, uint8_t* scale_T, void* stream);

/* fused_sparse_moe_v7(hidden_states, topk_weights, topk_ids, expert_map, w13_*, w2_*, inter_size,
 * apply_router_weight_on_input), sparse_fp4_v7.cu:607-742: gate_up GEMV -> SiLU(gate)*up ->
 * down GEMV -> router-weighted sum per token.
 *   hidden      [M, H] (h_dtype)            topk_weights [M, topk] f32   topk_ids [M, topk] i32
 *   expert_map  [global_E] i32 or NULL (identity); entries < 0 mark experts that are not local:
 *               such pairs contribute nothing (the reference does not handle them)
 *   w13_*       comp [E, H/4, 2I], meta [E, H/8, 2I], scale [E, G13, 2I], g [E]
 *   w2_*        comp [E, I/4, H],  meta [E, I/8, H],  scale [E, G2, H],  g [E]
 *   out         [M, H] (out_dtype)
 *   workspace   b200fp4_fused_moe_workspace_bytes(M, topk, H, I, E) bytes
 * flags: B200FP4_MOE_ROUTER_WEIGHT_ON_INPUT (the reference's apply_router_weight_on_input) sums the
 * expert outputs unweighted, exactly as the reference kernel does (sparse_fp4_v7.cu:592-594);
 * B200FP4_SPARSE_META_ORDERED as described above, for both weight sets.  With ordered metadata, the
 * usual shapes and up to 256 (token, expert) pairs both projections run in ONE cooperative launch
 * (blocks that finish their share of gate_up move on to the down projection of passes that are
 * already complete); B200FP4_MOE_SEPARATE_LAUNCHES keeps one launch per projection.
 *
 * Status word.  In the one-launch form a down-projection item waits (bounded, ~1 s of SM clocks by default)
 * for the gate_up items of its pass.  A wait that runs out writes B200FP4_MOE_STATUS_WAIT_EXPIRED to the
 * layer's status word -- the fourth int of `workspace` -- skips every later wait of the launch and lets the
 * kernel finish; the output of that call is then not to be trusted.  Every call clears the word first.
 * b200fp4_fused_moe_last_status copies it to *status after synchronising `stream` (the one function of this
 * library, with the *_host entry, that synchronises); the host-buffer entry checks it itself and returns
 * B200FP4_STATUS_INTERNAL_ERROR.  b200fp4_fused_moe_set_wait_limit(cycles, extra_need) sets the clock64 budget
 * of such a wait for later calls (cycles <= 0 restores the default) and, for diagnosis, adds `extra_need` to the
 * number of finished gate_up items a wait asks for (0 in normal use; 1 makes every wait run out, which is how
 * the time-out path is tested).  Process-global, not thread-safe.  No counterpart in the reference, whose
 * kernels never wait on one another. */
#define B200FP4_MOE_STATUS_WAIT_EXPIRED (-1)
B200FP4_API void b200fp4_fused_moe_set_wait_limit(int64_t cycles, int extra_need);
B200FP4_API int b200fp4_fused_moe_last_status(const void* workspace, void* stream, int* status);
B200FP4_API size_t b200fp4_fused_moe_workspace_bytes(int64_t M, int64_t topk, int64_t H, int64_t I,
                                                     int64_t E);
B200FP4_API int b200fp4_fused_sparse_moe(
    const void* hidden, int h_dtype, const float* topk_weights, const int32_t* topk_ids,
    const int32_t* expert_map, int64_t global_E, const uint8_t* w13_comp, const uint8_t* w13_meta,
    const uint8_t* w13_scale, const float* w13_g, int64_t G13, const uint8_t* w2_comp,
    const uint8_t* w2_meta, const uint8_t* w2_scale, const float* w2_g, int64_t G2, void* out,
    int out_dtype, int64_t M, int64_t topk, int64_t H, int64_t I, int64_t E,
    int flags, void* workspace, size_t workspace_bytes, void* stream);

/* The same layer for a caller that holds activations, routing and result in HOST memory (the
 * position of a serving process that calls the reference's op from outside the GPU framework):
 * hidden_host, topk_weights_host, topk_ids_host and out_host are host pointers (pinned memory keeps
 * the copies asynchronous), every other pointer is device memory as above.  Copies the three inputs
 * to the device, runs b200fp4_fused_sparse_moe, copies the result back and synchronises the stream,
 * so out_host is valid on return.  workspace: b200fp4_fused_moe_host_workspace_bytes(...) bytes of
 * device memory.  out_dtype F16 or BF16. */
B200FP4_API size_t b200fp4_fused_moe_host_workspace_bytes(int64_t M, int64_t topk, int64_t H,
                                                          int64_t I, int64_t E);
B200FP4_API int b200fp4_fused_sparse_moe_host(
    const void* hidden_host, int h_dtype, const float* topk_weights_host,
    const int32_t* topk_ids_host, const int32_t* expert_map, int64_t global_E,
    const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale, const float* w13_g,
    int64_t G13, const uint8_t* w2_comp, const uint8_t* w2_meta, const uint8_t* w2_scale,
    const float* w2_g, int64_t G2, void* out_host, int out_dtype, int64_t M, int64_t topk, int64_t H,
    int64_t I, int64_t E, int flags, void* workspace, size_t workspace_bytes, void* stream);

/* Enqueue-only form of b200fp4_fused_sparse_moe_host for a caller that keeps several steps in flight: the
 * three copies in, the layer and the copies out are queued and the call returns without waiting.
 *   copy_stream   NULL: everything runs on `stream`.  Otherwise the copies in run on copy_stream and
 *                 the layer waits for them through an event, so the inputs of the next step travel
 *                 while this step computes; before it overwrites the staging buffers of `workspace`
 *                 copy_stream waits for the layer of the previous submission that used the same
 *                 workspace -- a caller that alternates two workspaces gets the overlap, one that
 *                 reuses a single workspace stays correct.  The events live in a table of 32
 *                 (workspace, device) entries; ALLOC_FAILED beyond that.
 *   status_host   NULL, or host memory (pinned) that receives the layer's status word after the result
 *                 (0, or B200FP4_MOE_STATUS_WAIT_EXPIRED).
 *   flags         those of b200fp4_fused_sparse_moe, and B200FP4_MOE_HOST_DIRECT_OUT: where out_host
 *                 (and status_host) is pinned memory that the device can address, the layer's last
 *                 kernel stores the result rows (and the status word) straight into it over the host
 *                 link and no copy out is queued for it -- a copy between two layers costs the stream
 *                 about 5 us of engine switching; for pageable memory the flag changes nothing.
 * out_host and status_host are valid once the work queued on `stream` has completed (synchronise the
 * stream or an event recorded after the call); the caller gives every step in flight its own out_host.
 * No counterpart in the reference, which is always called with device tensors. */
B200FP4_API int b200fp4_fused_sparse_moe_host_async(
    const void* hidden_host, int h_dtype, const float* topk_weights_host,
    const int32_t* topk_ids_host, const int32_t* expert_map, int64_t global_E,
    const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale, const float* w13_g,
    int64_t G13, const uint8_t* w2_comp, const uint8_t* w2_meta, const uint8_t* w2_scale,
    const float* w2_g, int64_t G2, void* out_host, int out_dtype, int32_t* status_host, int64_t M,
    int64_t topk, int64_t H, int64_t I, int64_t E, int flags, void* workspace, size_t workspace_bytes,
    void* stream, void* copy_stream);

/* ---------------------------------------------------------------------------------------------
 * Part 4 -- grouped (per-expert) NVFP4 GEMM for MoE prefill and its routing helpers.
 * The reference's own grouped kernel is an FP8 CUTLASS configuration behind
 * extern "C" cutlass_moe_mm_gb10(out, a, b, a_scales, b_scales, expert_offsets, problem_sizes,
 * strides..., per_act_token, per_out_ch) (grouped_mm_gb10_native.cu:196-208; tile policy :44-100,
 * :141-156); the NVFP4 contract mirrored here is the upstream op that path stands in for,
 * cutlass_fp4_group_mm(out, a, b, a_scales, b_scales, alphas, problem_sizes, expert_offsets,
 * sf_offsets) with get_cutlass_moe_mm_data / shuffle_rows (vllm/_custom_ops.py:854-933,1017-1054).
 * ------------------------------------------------------------------------------------------- */

/* get_cutlass_moe_mm_data: group the M*topk (token, expert) pairs by local expert.
 *   expert_offsets[E+1], blockscale_offsets[E+1] (each expert padded to 128 rows),
 *   dst2src[M*topk]: permuted row -> pair index token*topk+slot (-1 past the last valid row),
 *   src2dst[M*topk]: pair index -> permuted row (-1 when the pair's expert is not local).
 * expert_map [global_E] or NULL as in b200fp4_fused_sparse_moe. */
B200FP4_API int b200fp4_moe_permute(const int32_t* topk_ids, const int32_t* expert_map,
                                    int64_t global_E, int64_t M, int64_t topk, int64_t E,
                                    int32_t* expert_offsets, int32_t* blockscale_offsets,
                                    int32_t* dst2src, int32_t* src2dst, void* stream);

/* shuffle_rows: out[i,:] = in[dst2src[i] / src_div, :] (rows of row_bytes bytes, multiple of 16);
 * negative map entries give zero rows. */
B200FP4_API int b200fp4_shuffle_rows(const void* in, int64_t row_bytes, const int32_t* dst2src,
                                     int64_t n_dst, int64_t src_div, void* out, void* stream);

/* cutlass_fp4_group_mm: rows [expert_offsets[e], expert_offsets[e+1]) of a (packed codes
 * [rows_capacity, K/2], scales swizzled with expert e's rows starting at sf_offsets[e]) times
 * expert e's weight b[e] ([E, N, K/2] codes, b_sf [E, swizzled(N, K/16)]), scaled by alphas[e],
 * into out[rows_capacity, N].  Rows past expert_offsets[E] are not written.  The first int of the
 * workspace is the same status word as for b200fp4_gemm_nvfp4. */
B200FP4_API size_t b200fp4_grouped_gemm_workspace_bytes(int64_t rows_capacity, int64_t E);
B200FP4_API int b200fp4_grouped_gemm_nvfp4(const void* a_codes, const void* b_codes, const void* a_sf,
                                           const void* b_sf, const float* alphas,
                                           const int32_t* expert_offsets, const int32_t* sf_offsets,
                                           void* out, int out_dtype, int64_t rows_capacity, int64_t N,
                                           int64_t K, int64_t E, int tile_n, void* workspace,
                                           size_t workspace_bytes, void* stream);

/* The gate_up projection of a gated MoE layer with the activation and the next quantization in the
 * GEMM's epilogue: cutlass_fp4_group_mm into a [rows, N] tensor of mid_dtype followed by
 * silu_and_mul_scaled_fp4_experts_quant (vllm/_custom_ops.py:1706-1733), without writing that tensor.
 * b [E, N, K/2] holds the gate rows [0, N/2) before the up rows [N/2, N) (N/2 a multiple of 128).
 * Each product is scaled by alphas[e] and rounded to mid_dtype (F16/BF16), SiLU(gate)*up is rounded to
 * mid_dtype, and blocks of 16 are quantized with out_global_scales[e]: out_codes [rows_capacity, N/4]
 * (32-byte aligned) and out_sf, swizzled with expert e's rows at sf_offsets[e], receive the same bytes
 * as the two separate calls for every row below expert_offsets[E]; other rows are not written. */
B200FP4_API int b200fp4_grouped_gemm_nvfp4_silu_quant(
    const void* a_codes, const void* b_codes, const void* a_sf, const void* b_sf, const float* alphas,
    const int32_t* expert_offsets, const int32_t* sf_offsets, const float* out_global_scales,
    int mid_dtype, void* out_codes, void* out_sf, int64_t rows_capacity, int64_t N, int64_t K,
    int64_t E, void* workspace, size_t workspace_bytes, void* stream);

/* Un-permute and router-weighted sum: out[m,:] = sum_t w[m,t] * expert_out[src2dst[m*topk+t], :]
 * over local pairs (the shuffle_rows + weighted sum at the end of
 * vllm/model_executor/layers/fused_moe/experts/cutlass_moe.py:567-663). */
B200FP4_API int b200fp4_moe_unpermute_reduce(const void* expert_out, int dtype, const int32_t* src2dst,
                                             const float* topk_weights, int64_t M, int64_t topk,
                                             int64_t H, void* out, void* stream);

/* MoE router for decode: gate projection, softmax over the experts, top-k, renormalisation -- the step in front of
 * the fused layer.  The reference leaves it to vLLM's torch code (its benches restate it:
 * sparse_fp4_kernel/bench_moe_layer_e2e.py:230-236, softmax(logits).topk(k), weights / their sum); here the outputs are
 * the device tensors b200fp4_fused_sparse_moe and b200fp4_ep_pack take, so routing never leaves the GPU.
 *   hidden [M, H] and gate_w [E, H] of `dtype` (BF16 or F16), hidden rows ld_h elements apart; logits accumulate in f32
 *   topk_weights [M, topk] f32 = exp(l - max) / sum over the selected experts (renormalize != 0) or over all experts
 *   topk_ids [M, topk] i32 in decreasing order of logit; equal logits go to the lower expert id
 *   workspace b200fp4_moe_router_workspace_bytes(M, E) bytes (the f32 logits).  topk <= 32, E <= 1024. */
B200FP4_API size_t b200fp4_moe_router_workspace_bytes(int64_t M, int64_t E);
B200FP4_API int b200fp4_moe_router(const void* hidden, int64_t ld_h, int dtype, const void* gate_w, int64_t M, int64_t H,
                                   int64_t E, int64_t topk, int renormalize, float* topk_weights, int32_t* topk_ids,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Expert-parallel helpers (no counterpart in the reference, which has no multi-GPU code of its
 * own: it serves with tensor parallelism through vLLM, entrypoint.sh:100-116).  A dispatch record
 * is [H activations (16-bit) | topk ids (i32) | topk router weights (f32)], padded to 16 bytes.
 *   b200fp4_ep_pack       writes records[g][b] for every destination rank g (send buffer of the
 *                         fixed-capacity all-to-all)
 *   b200fp4_fused_sparse_moe_records   b200fp4_fused_sparse_moe over T received records read in
 *                         place (router weights always applied to the output; flags as above)
 *   b200fp4_ep_combine    out[b] = sum_g parts[g][b] in fp32 (partial rows returned by the ranks)
 * ------------------------------------------------------------------------------------------- */
B200FP4_API size_t b200fp4_ep_record_bytes(int64_t H, int64_t topk);
B200FP4_API int b200fp4_ep_pack(const void* hidden, const int32_t* topk_ids, const float* topk_weights,
                                int64_t B, int64_t H, int64_t topk, int64_t G, void* records,
                                void* stream);
B200FP4_API int b200fp4_fused_sparse_moe_records(
    const void* records, int64_t record_bytes, int h_dtype, const int32_t* expert_map, int64_t global_E,
    const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale, const float* w13_g,
    int64_t G13, const uint8_t* w2_comp, const uint8_t* w2_meta, const uint8_t* w2_scale,
    const float* w2_g, int64_t G2, void* out, int out_dtype, int64_t T, int64_t topk, int64_t H,
    int64_t I, int64_t E, int flags, void* workspace, size_t workspace_bytes, void* stream);
B200FP4_API int b200fp4_ep_combine(const void* parts, int dtype, int64_t B, int64_t H, int64_t G,
                                   void* out, void* stream);

/* The same exchange without a collective library: dispatch and combine over peer memory (NVLink), initiated by the
 * kernels themselves.  Every rank owns three buffers that all ranks can address (peer mappings; the caller allocates
 * them, e.g. with torch's symmetric memory): records [G][B] dispatch records (slot g written by rank g), parts
 * [G][B][H] f32 (slot g = the partial rows rank g computed for this rank's tokens), flags [2][G] i32, zero before the
 * first step.  record_ptrs / part_ptrs / flag_ptrs are DEVICE arrays of the G ranks' pointers to those buffers; seq =
 * 1, 2, 3, ... numbers the steps, the same on every rank; scratch = 4 ints of local device memory, zero before the first
 * step (scratch[1] != 0 after a step: a bounded wait for a peer ran out, the step's result is not valid).
 *   b200fp4_ep_dispatch_p2p   stores this rank's B records into slot `rank` of every rank's records buffer, publishes
 *                             flags[0][rank] = seq on every rank, and waits (bounded, ~1 s) until all G ranks' records
 *                             of this step have landed here
 *   b200fp4_fused_sparse_moe_records_scatter   the fused layer over the G*B records; row m of its result goes to row
 *                             dest_row0 + m % rows_per_dest of the buffer out_ptrs[m / rows_per_dest] (out_ptrs = part_ptrs,
 *                             rows_per_dest = B, dest_row0 = rank * B: plain peer stores)
 *   b200fp4_ep_combine_p2p    publishes flags[1][rank] = seq everywhere, waits for all G ranks' partial rows, adds them in
 *                             f32: out [B, H] bf16 / f16
 * Plain peer loads and stores only (no multicast).  Not capturable into a CUDA graph as is: seq is a launch argument. */
B200FP4_API int b200fp4_ep_dispatch_p2p(const void* hidden, const int32_t* topk_ids, const float* topk_weights, int64_t B,
                                        int64_t H, int64_t topk, int64_t G, int64_t rank, void* const* record_ptrs,
                                        int32_t* const* flag_ptrs, int32_t seq, int32_t* scratch, void* stream);
B200FP4_API int b200fp4_fused_sparse_moe_records_scatter(
    const void* records, int64_t record_bytes, int h_dtype, const int32_t* expert_map, int64_t global_E,
    const uint8_t* w13_comp, const uint8_t* w13_meta, const uint8_t* w13_scale, const float* w13_g, int64_t G13,
    const uint8_t* w2_comp, const uint8_t* w2_meta, const uint8_t* w2_scale, const float* w2_g, int64_t G2,
    void* const* out_ptrs, int64_t rows_per_dest, int64_t dest_row0, int out_dtype, int64_t T, int64_t topk, int64_t H,
    int64_t I, int64_t E, int flags, void* workspace, size_t workspace_bytes, void* stream);
B200FP4_API int b200fp4_ep_combine_p2p(const float* parts, int64_t B, int64_t H, int64_t G, int64_t rank,
                                       int32_t* const* flag_ptrs, int32_t seq, int32_t* scratch, void* out, int out_dtype,
                                       void* stream);

/* ---------------------------------------------------------------------------------------------
 * The reference's declared C API, exported under its own names so that a program written against
 * cutlass_nvfp4/cuda_fp4_gemm.h links against this library unchanged (the reference declares these
 * functions and defines none of them).  Prototypes follow cuda_fp4_gemm.h:48-63 (handle), :94-105
 * (cudaFP4GemmEx), :113-120 (cudaFP4Gemm), :124-147 (utilities), :161-203 (conversions); the
 * reference's one-byte structs cuda_fp4x2_t / __nv_fp8_e4m3 appear as void pointers and cudaStream_t
 * as void*, which is the same C ABI.  Skipped when the reference's header was included first.
 *
 *   cudaFP4GemmEx   C[M,N] f32 = (A . A_scales)(B . B_scales)^T * A_scale_global * B_scale_global with
 *                   A [M,K/2], B [N,K/2] packed E2M1 and LINEAR E4M3 scales [M,K/16], [N,K/16];
 *                   group_size must be 16 and K a multiple of 64.  Runs on the handle's stream.
 *   cudaFP4Gemm     the same without block scales: C = alpha * A B^T.
 *   cudaFP4Quantize fp32 [rows, cols] -> codes, linear E4M3 scales and *dst_scale_global (HOST
 *                   pointer) = amax / (6 * 448); synchronises `stream` to return that scalar.
 *   cudaFP4ConvertFromFP32 / ToFP32   element-wise E2M1 rounding (RNE, saturating) and decoding.
 * E2M1 values are the NVFP4 set {0, .5, 1, 1.5, 2, 3, 4, 6}, not the reference header kernels'
 * non-standard table (cutlass_nvfp4/nvfp4_types.cuh:56-64).  The handle keeps device scratch sized
 * at cudaFP4Create for problems up to 8192^3 and grows it with cudaMalloc when a call needs more.
 * ------------------------------------------------------------------------------------------- */
#ifndef __CUDA_FP4_GEMM_H__
typedef struct cudaFP4Handle_st* cudaFP4Handle_t;
B200FP4_API int cudaFP4Create(cudaFP4Handle_t* handle);
B200FP4_API int cudaFP4Destroy(cudaFP4Handle_t handle);
B200FP4_API int cudaFP4SetStream(cudaFP4Handle_t handle, void* stream);
B200FP4_API int cudaFP4GemmEx(cudaFP4Handle_t handle, int M, int N, int K, const void* A, const void* A_scales,
                              float A_scale_global, const void* B, const void* B_scales, float B_scale_global,
                              float* C, int group_size);
B200FP4_API int cudaFP4Gemm(cudaFP4Handle_t handle, int M, int N, int K, float alpha, const void* A, const void* B,
                            float* C);
B200FP4_API const char* cudaFP4GetVersionString(void);
B200FP4_API int cudaFP4GetVersion(void);
B200FP4_API int cudaFP4HasHardwareAcceleration(void);
B200FP4_API const char* cudaFP4GetErrorString(int status);
B200FP4_API int cudaFP4ConvertFromFP32(void* dst, const float* src, int rows, int cols, void* stream);
B200FP4_API int cudaFP4ConvertToFP32(float* dst, const void* src, int rows, int cols, void* stream);
B200FP4_API int cudaFP4Quantize(void* dst_data, void* dst_scales, float* dst_scale_global, const float* src, int rows,
                                int cols, int group_size, void* stream);
#endif

/* Benchmark hook (no counterpart in the reference): when the three cudaEvent_t handles are non-NULL,
 * b200fp4_fused_sparse_moe records them on its stream before the gate_up GEMV, between the two
 * GEMVs and after the down GEMV, so a caller can time the two dominant kernels inside a fused
 * call.  Pass NULLs to switch it off.  Process-global, not thread-safe. */
B200FP4_API void b200fp4_fused_moe_profile_events(void* before_gate_up, void* after_gate_up,
                                                  void* after_down);

#ifdef __cplusplus
}
#endif
#endif /* B200_NVFP4_H_ */
