/*
 * b200moe.h -- C ABI of the B200 (sm_100a) expert-parallel quantized MoE kernels.
 *
 * One shared library, plain pointers and sizes, no framework types.  Every
 * function launches asynchronously on the CUDA stream it is given (a
 * cudaStream_t passed as void*; NULL = the legacy default stream), never
 * allocates or frees device memory, never synchronises, and returns a status
 * code (0 = ok).  All pointers are device pointers unless stated otherwise;
 * all tensors are dense row-major unless a stride is an argument.
 *
 * Each entry point names the reference interface it stands in for (paths are
 * relative to the reference project root).
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define B200MOE_API __attribute__((visibility("default")))
#else
#define B200MOE_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (the reference returns 0 / -1 from simple_marlin_cuda,
 *      fast_dequant/simple_marlin/marlin_w4a16_gemm.cu:300-302,325, and raises
 *      from bare asserts in its Python wrappers) ---- */
enum {
  B200MOE_OK = 0,
  B200MOE_BAD_SHAPE = 1,         /* a size the kernel does not support            */
  B200MOE_BAD_ALIGN = 2,         /* pointer or stride not aligned as required     */
  B200MOE_BAD_DTYPE = 3,
  B200MOE_BAD_ARG = 4,           /* null pointer, inconsistent arguments          */
  B200MOE_WORKSPACE_TOO_SMALL = 5,
  B200MOE_LAUNCH_FAILED = 6,     /* CUDA reported an error at launch              */
  B200MOE_DEVICE_TIMEOUT = 7,    /* a bounded device-side wait expired            */
  B200MOE_UNSUPPORTED_DEVICE = 8 /* not an sm_100 device / driver too old         */
};

/* ---- element types ---- */
enum {
  B200MOE_F32 = 0,
  B200MOE_F16 = 1,
  B200MOE_BF16 = 2,
  B200MOE_FP8_E4M3 = 3,
  B200MOE_I8 = 4
};

B200MOE_API const char* b200moe_status_string(int status);
/* Message of the last non-zero status returned on the calling host thread. */
B200MOE_API const char* b200moe_last_error(void);
B200MOE_API int b200moe_abi_version(void);

/* ======================= quantization/fp8_kernel.py ======================= */

/* act_quant (quantization/fp8_kernel.py:33-52; kernel :9-30).
 * x [rows, cols] (f32/f16/bf16), cols % 128 == 0.  Per 128 contiguous values
 * s = amax/448 (f32) and y = e4m3(x / s), round-to-nearest-even.  amax == 0
 * gives s == 0 and y == NaN, as in the reference.
 * y [rows, cols] e4m3 with row stride y_row_stride_bytes, s [rows, cols/128]
 * f32 with row stride s_row_stride (in floats). */
B200MOE_API int b200moe_act_quant_fp8(const void* x, int x_dtype, int64_t rows, int64_t cols,
                          void* y, int64_t y_row_stride_bytes,
                          float* s, int64_t s_row_stride, void* stream);

/* weight_dequant (quantization/fp8_kernel.py:84-105): y = x * s[i/128, j/128]. */
B200MOE_API int b200moe_weight_dequant_fp8(const void* x, const float* s, void* y, int y_dtype,
                               int64_t M, int64_t N, void* stream);

/* 128x128-block e4m3 weight quantizer, s = amax/448.  The reference ships the
 * int8 form only (quantization/int8_kernel.py:59-113); this is its fp8 twin
 * with the same block grid and scale shape [ceil(M/128), ceil(N/128)]. */
B200MOE_API int b200moe_weight_quant_fp8(const void* w, int w_dtype, void* y, float* s,
                             int64_t M, int64_t N, void* stream);

/* fp8_gemm (quantization/fp8_kernel.py:170-190; kernel :108-167).
 * c[M,N] = a[M,K] . b[N,K]^T with acc += dot_kb * a_s[m,kb] * b_s[n/128,kb]
 * per 128-wide K block.  a, b e4m3; a_s [M,K/128], b_s [N/128,K/128] f32;
 * c f32/f16/bf16.  K % 128 == 0, N % 128 == 0; a, b 16-byte aligned. */
B200MOE_API int b200moe_gemm_fp8_block(const void* a, const float* a_s, const void* b, const float* b_s,
                           void* c, int c_dtype, int64_t M, int64_t N, int64_t K,
                           void* stream);

/* Same product with the K loop split over `ksplits` sets of tiles, for small M: one m-tile times
 * N/256 n-tiles keeps only N/256 SMs streaming the weights, ksplits times as many tiles keep the
 * chip busy.  Each split writes f32 partial products to `partials` (caller-owned scratch of
 * ksplits * M * N * 4 bytes, 16-byte aligned); a second kernel adds them in split order and
 * casts to c_dtype.  ceil(K/128 / ksplits) * (ksplits - 1) < K/128 (no empty split), ksplits <= 16.
 * No counterpart in the reference. */
B200MOE_API int b200moe_gemm_fp8_block_splitk(const void* a, const float* a_s, const void* b, const float* b_s,
                                  void* c, int c_dtype, int64_t M, int64_t N, int64_t K, int ksplits,
                                  float* partials, int64_t partials_bytes, void* stream);

/* ======================= quantization/int8_kernel.py ====================== */

/* act_quant: s = amax/127 stored as f16, y = round(x/s) as int8.
 * rounding 0 = half away from zero (quantization/int8_kernel.py:23-31),
 *          1 = floor(v + 0.5)      (quantization/w4a8_kernel.py:159-168). */
B200MOE_API int b200moe_act_quant_int8(const void* x, int x_dtype, int64_t rows, int64_t cols,
                           void* y, void* s_f16, int rounding, void* stream);

/* weight_quant (quantization/int8_kernel.py:59-113): per 128x128 block s = amax/qmax stored as
 * f16 [ceil(M/128), ceil(N/128)], y int8 [M,N] = round(w / s) with the f32 scale.
 * qmax 127, rounding 0 (half away from zero, unclamped) is int8_kernel.weight_quant;
 * qmax 119, rounding 1 (floor(v + 0.5) clamped to +-qmax) is the first level of the two-level
 * int4 quantizer (weight_quant_int8_kernel, quantization/w4a8_kernel.py:196-225). */
B200MOE_API int b200moe_weight_quant_int8(const void* w, int w_dtype, void* y_int8, void* s_f16,
                              int64_t M, int64_t N, float qmax, int rounding, void* stream);

/* weight_dequant (quantization/int8_kernel.py:116-170): y = float(x) * s[i/128, j/128]. */
B200MOE_API int b200moe_weight_dequant_int8(const void* x_int8, const void* s_f16, void* y, int y_dtype,
                                int64_t M, int64_t N, void* stream);

/* Middle step of the quantized all-reduce (quant_communication/quant_all2all_allreduce.py:73-80): the chunks
 * received from n_src ranks -- payload q (e4m3 with f32 scales, or int8 with f16 scales; one scale per 128
 * values of a row), source `i` at q + i * q_src_stride_bytes and s + i * s_src_stride (elements) -- are
 * dequantized (product formed in the scales' dtype as the reference's dequant kernels do,
 * quant_communication/quant_utils.py:75-83, 176-180, then cast to out_dtype), summed in f32 in source order and
 * the sum is rounded to out_dtype (bf16/f16).  A group whose scale is 0 (all-zero input, whose payload is
 * NaN by the quantizers' x / s) decodes to zero.  With n_src == 1 this is the plain dequantization of the
 * all-gather step (:96-99).  cols % 128 == 0. */
B200MOE_API int b200moe_dequant_sum(const void* q, int q_dtype, int64_t q_row_stride_bytes, int64_t q_src_stride_bytes,
                        const void* s, int s_dtype, int64_t s_row_stride, int64_t s_src_stride, int n_src,
                        int64_t rows, int64_t cols, void* out, int out_dtype, void* stream);

/* ========================= moe/all2all_moe.py ============================= */

/* MoEGate.forward (moe/all2all_moe.py:60-118).
 * logits = x[T,H] (f32/f16/bf16) . w[E,H]^T (f32) in f32; scoring 0 = sigmoid,
 * 1 = softmax over experts; selection scores = scores + bias (bias may be
 * NULL); group-limited top-k: group score = sum of its top 2, keep topk_group
 * of n_group groups, other experts' selection scores become 0.0, then top_k.
 * Ties go to the lower expert id.  topk_weight gathers the unbiased scores,
 * divides by (sum + 1e-20) when norm_topk_prob and top_k > 1, and multiplies
 * by routed_scaling_factor.  topk_idx int64 [T,top_k] in descending selection
 * score order; topk_weight f32 [T,top_k].  E <= 256, E % n_group == 0,
 * top_k <= 32, H % 8 == 0. */
B200MOE_API int b200moe_router_topk(const void* x, int x_dtype, const float* w, const float* bias,
                        int64_t T, int64_t H, int E, int top_k, int n_group, int topk_group,
                        int scoring, int norm_topk_prob, float routed_scaling_factor,
                        int64_t* topk_idx, float* topk_weight, void* stream);

/* Tensor-core form of the same router for large expert counts, in two launches.
 * b200moe_router_logits_bf16x3: logits x . W^T with f32-equivalent precision out of bf16
 * MMAs: w3 bf16 [E, 3H] holds, per expert row, the three bf16 parts hi | mid | lo of the f32
 * router weight (hi = bf16(w), mid = bf16(w - hi), lo = bf16(w - hi - mid)); x is bf16
 * [T,H].  The K loop is split over `ksplits` CTAs per tile; partials f32 [ksplits, T, E]
 * receives the partial sums.  E % 128 == 0, H % 64 == 0; a model with another expert count
 * pads w3 with zero rows to the next multiple of 128 and passes the padded count here.
 * b200moe_router_select: adds the partials in index order and applies the scoring,
 * group-limited selection and weight normalisation exactly as b200moe_router_topk, over
 * the first E columns of rows that are partials_row_stride floats apart (the padded count). */
B200MOE_API int b200moe_router_logits_bf16x3(const void* x_bf16, const void* w3_bf16, float* partials,
                                 int64_t T, int64_t H, int E, int ksplits, void* stream);
B200MOE_API int b200moe_router_select(const float* partials, int nsplit, int64_t partials_row_stride,
                          const float* bias, int64_t T, int E,
                          int top_k, int n_group, int topk_group, int scoring,
                          int norm_topk_prob, float routed_scaling_factor, int64_t* topk_idx,
                          float* topk_weight, void* stream);

/* ======================= moe/group_gemm_kernel.py ========================= */

/* run_moe_ep_preproess (moe/group_gemm_kernel.py:48-78): stable counting sort
 * of the num_slots = T*k expert ids.
 *   reorder_topk_ids int64 [num_slots]  ids in sorted order        (:52)
 *   src2dst          int32 [num_slots]  flat slot -> sorted row    (:37-45)
 *   seg_indptr       int64 [E+1]        exclusive prefix of counts (:19-34)
 * workspace: b200moe_route_metadata_workspace_bytes() bytes of scratch,
 * 16-byte aligned.  Bit-exact and deterministic (no order-dependent atomics).
 * num_experts <= 1024. */
B200MOE_API size_t b200moe_route_metadata_workspace_bytes(int64_t num_slots, int num_experts);
B200MOE_API int b200moe_route_metadata(const int64_t* topk_ids, int64_t num_slots, int num_experts,
                           int64_t* reorder_topk_ids, int32_t* src2dst, int64_t* seg_indptr,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Same result as b200moe_route_metadata, for callers that cannot supply a workspace: code
 * running inside a process whose framework took all device memory for its own pool, a plug-in
 * that only ever sees its input and output buffers, or a loop that must never reach cudaMalloc
 * because that call synchronises the device.  This entry point has no counterpart in the
 * reference.  Its scratch is a 1 MiB array built into the library (resident on every GPU that
 * loads the library, until the process exits), which bounds the problem size:
 *     ceil(num_slots / 1024) * num_experts <= 262144
 * (e.g. 1 M slots x 256 experts, or 262 k slots x 1024 experts); larger requests return
 * B200MOE_BAD_SHAPE and launch nothing.  It performs no device allocation of any kind.
 * The first call on each GPU looks up the array's device address (once, with that GPU
 * current); make that first call outside any stream capture.  All calls on one GPU share the
 * array: two calls whose kernels may overlap on the GPU (different streams without an
 * ordering between them) race and give wrong results -- order them on one stream or with
 * events.  Nothing needs zeroing between calls. */
B200MOE_API int b200moe_route_metadata_noalloc(const int64_t* topk_ids, int64_t num_slots, int num_experts,
                                   int64_t* reorder_topk_ids, int32_t* src2dst,
                                   int64_t* seg_indptr, void* stream);

/* pre_reorder_triton_kernel (moe/group_gemm_kernel.py:81-117): for every slot
 * whose expert is in [start_expert_id, end_expert_id] (inclusive) copy the
 * token's row to out[src2dst[slot]], multiplied by 1/a1_scales[e-start] when
 * a1_scales != NULL, cast to out_dtype (f16/bf16/e4m3).  H % 8 == 0. */
B200MOE_API int b200moe_pre_reorder(const void* x, int x_dtype, void* out, int out_dtype,
                        const int32_t* src2dst, const int64_t* topk_ids,
                        const float* a1_scales, int start_expert_id, int end_expert_id,
                        int64_t T, int topk, int64_t H, void* stream);

/* Fused permute + 1x128 e4m3 activation quantizer: pre_reorder
 * (moe/group_gemm_kernel.py:81-117) followed by act_quant
 * (quantization/fp8_kernel.py:33-52) without the [T*k,H] 16-bit round trip.
 * The token row is quantized once and written to each of its local slots.
 * out_q rows are out_q_row_stride_bytes apart, out_s rows out_s_row_stride
 * floats apart, so payload and scales may live in one packed record per row.
 * H % 128 == 0. */
B200MOE_API int b200moe_permute_quant_fp8(const void* x, int x_dtype, const int32_t* src2dst,
                              const int64_t* topk_ids, int start_expert_id, int end_expert_id,
                              int64_t T, int topk, int64_t H,
                              void* out_q, int64_t out_q_row_stride_bytes,
                              float* out_s, int64_t out_s_row_stride, void* stream);

/* Same fusion with the int8 per-token-group quantizer (s = amax/127; rounding as in
 * b200moe_act_quant_int8).  The scale is rounded to f16 as the reference stores it
 * (quantization/w4a8_kernel.py:163-168) and written as f32 so that the payload record can
 * be fed to b200moe_grouped_gemm_i8 directly. */
B200MOE_API int b200moe_permute_quant_int8(const void* x, int x_dtype, const int32_t* src2dst,
                               const int64_t* topk_ids, int start_expert_id, int end_expert_id,
                               int64_t T, int topk, int64_t H,
                               void* out_q, int64_t out_q_row_stride_bytes,
                               float* out_s, int64_t out_s_row_stride, int rounding, void* stream);

/* Row gather: dst row i = src row row_map[i] (rows of row_bytes bytes, a multiple of 16;
 * negative entries skip the row).  Used to bring rows received in (source rank, expert)
 * order into expert order; the reference does this on the host with numpy
 * (moe/all2all_moe.py:229-240). */
B200MOE_API int b200moe_gather_rows(const void* src, void* dst, const int32_t* row_map, int64_t n,
                        int64_t row_bytes, void* stream);

/* silu_and_mul_triton_kernel / gelu_and_mul_triton_kernel
 * (moe/group_gemm_kernel.py:120-168, 176-235).  gateup [rows, two_I] =
 * [gate | up]; rows whose reorder_topk_ids is outside [start,end] are skipped
 * (reorder_topk_ids may be NULL = all rows).  act 0 = silu, 1 = tanh-gelu.
 * Activation in f32, rounded to the input dtype, product in the input dtype,
 * times 1/scales[e-start] when scales != NULL, cast to out_dtype. */
B200MOE_API int b200moe_act_and_mul(const void* gateup, int dtype, void* down_input, int out_dtype,
                        int64_t rows, int64_t two_I, const int64_t* reorder_topk_ids,
                        const float* scales, int start_expert_id, int end_expert_id,
                        int act, void* stream);

/* post_reorder_triton_kernel (moe/group_gemm_kernel.py:238-288) and the
 * weighted un-permute of moe/all2all_moe.py:270-278:
 * out[t] = sum over local slots of down_output[src2dst[t,j]] * w[t,j],
 * accumulated in f32 (as moe/all2all_moe.py:273-277 does), zero when the token
 * has no local slot.  H % 8 == 0. */
B200MOE_API int b200moe_post_reorder(const void* down_output, int dtype, void* out,
                         const int32_t* src2dst, const int64_t* topk_ids,
                         const float* topk_weights, int start_expert_id, int end_expert_id,
                         int64_t T, int topk, int64_t H, void* stream);

/* Per-call launch options of the grouped tcgen05 GEMMs (a NULL pointer means all zeros).  No counterpart in the
 * reference (its Triton grids are sized by the tile count, moe/group_gemm_kernel.py:484-487).
 *   max_ctas   upper bound on the persistent grid; 0 = one CTA per SM.  A GEMM CTA owns its whole SM, so a
 *              collective that is meant to run beside the GEMM only progresses if some SMs are left free.
 *   pair_mode  0 = one CTA per 128 x 256 tile; 1 = clusters of two CTAs sharing a 256 x 256 tile (tcgen05
 *              cta_group::2: each SM then moves 32 KB instead of 48 KB per K block).  Results are identical. */
typedef struct b200moe_gemm_opts {
  int32_t max_ctas;
  int32_t pair_mode;
} b200moe_gemm_opts;

/* grouped_gemm_triton with block_shape = [128,128]
 * (moe/group_gemm_kernel.py:442-513; kernel :291-428), fp8 operands.
 * For every group g, rows [seg_indptr[g], seg_indptr[g+1]) of a use weight
 * b[weight_indices[g]] ([N,K] e4m3, K-major = weight_column_major) and scales
 * b_s[weight_indices[g]] ([N/128, K/128] f32); acc += dot_kb * a_s * b_s per
 * K block.  a [M_total, K] e4m3 with row stride a_row_stride_bytes, a_s
 * [M_total, K/128] f32 with row stride a_s_row_stride (floats).
 * seg_indptr / weight_indices are int64 device arrays (weight_indices NULL =
 * identity).  Unlike the reference the activations arrive already quantized
 * (the reference quantizes inside the call, :459-469).
 *
 * epilogue 0: c [M_total, N] in c_dtype (f32/f16/bf16), row stride N.
 * epilogue 1: SwiGLU + 1x128 e4m3 re-quantization fused (replaces
 *   silu_and_mul_triton_kernel :120-168 plus the act_quant of the second
 *   grouped_gemm_triton call).  b rows [0,N/2) are gate, [N/2,N) are up
 *   (moe/moe_numerical_equivalence_validation.py:87-88); c is e4m3
 *   [M_total, N/2] with row stride c_row_stride_bytes and c_s f32
 *   [M_total, N/2/128] with row stride c_s_row_stride.  Intermediates are
 *   rounded to bf16 where the reference rounds to its activation dtype.
 * epilogue 4: as 1 with the tanh-GELU of gelu_and_mul_triton_kernel (:176-235) in place of SiLU.
 * c_row_map (epilogue 0 only, may be NULL): int32 [M_total]; output row r is stored at row
 * c_row_map[r], which un-does a row gather in the store instead of in a separate pass.
 * c_row_addr (epilogue 0 only, may be NULL, exclusive with c_row_map): int64 [M_total]; output row
 * r is stored at the byte address c_row_addr[r] (16-byte aligned), which may be a peer mapping of
 * another GPU's memory: the expert-parallel return trip (the second all_to_all_single of
 * moe/all2all_moe.py:248-262) then happens in the stores of the down projection.
 * Rows outside every group are not written.  K % 128 == 0, N % 128 == 0
 * (epilogues 1 and 4: N % 256 == 0).  status_word (may be NULL): a device int32 that
 * receives B200MOE_DEVICE_TIMEOUT if a bounded wait inside the kernel expires. */
B200MOE_API int b200moe_grouped_gemm_fp8(const void* a, int64_t a_row_stride_bytes,
                             const float* a_s, int64_t a_s_row_stride,
                             const void* b, const float* b_s,
                             void* c, int c_dtype, int64_t c_row_stride_bytes,
                             float* c_s, int64_t c_s_row_stride,
                             int64_t M_total, int64_t N, int64_t K,
                             int num_groups, int num_weights,
                             const int64_t* seg_indptr, const int64_t* weight_indices,
                             int epilogue, const int32_t* c_row_map, const int64_t* c_row_addr,
                             int32_t* status_word, const b200moe_gemm_opts* opts, void* stream);

/* ===================== int4 weight paths (w4a8, w4a16) ==================== */

/* int4 -> int8 step of the two-level format (weight_dequant_int4_kernel,
 * quantization/w4a8_kernel.py:44-101; the unpack inside w4a8_gemm_kernel :362-380).
 * packed int32 [W, N/8, K]: word (n/8, k), field n%8 = q[n,k]
 * (pack_weights_over_rows, quantization/bitpack.py:9-36); s4, z4 int8 [W, N, K/128].
 * out int8 [W, N, K] = int8((q - z4) * s4) with int8 wrap-around as in the reference.
 * N % 8 == 0, K % 128 == 0. */
B200MOE_API int b200moe_w4a8_expand_int8(const void* packed, const int8_t* s4, const int8_t* z4, void* out,
                             int64_t W, int64_t N, int64_t K, void* stream);

/* Asymmetric group-128 int4 -> bf16: w = (q - zero) * scale rounded once to bf16.
 * Extends the symmetric dequantization of the reference's w4a16 kernel
 * (fast_dequant/simple_marlin/marlin_w4a16_gemm.cu:44-64, utils.py:98-136) with a
 * zero-point.  packed int32 [rows, K/8]: word k/8, field k%8 = q[row,k]
 * (pack_weights_over_cols, quantization/bitpack.py:38-67); scale, zero bf16 [rows, K/128].
 * out bf16 [rows, K].  K % 128 == 0. */
B200MOE_API int b200moe_w4a16_expand_bf16(const void* packed, const void* scale_bf16, const void* zero_bf16,
                              void* out_bf16, int64_t rows, int64_t K, void* stream);

/* weight_quant of the two-level format in one kernel (quantization/w4a8_kernel.py:196-309):
 * level 1 per 128x128 block s = amax/119 (f16 out), y8 = clamp(floor(w/s + 0.5), +-119);
 * level 2 per (row, 128 columns): s4 = floor((max - min)/15 + 0.5), z4 = floor(-min/s4 + 0.5),
 * q = clamp(floor(y8/s4 + 0.5) + z4, 0, 15); packed over rows (pack_weights_over_rows,
 * quantization/bitpack.py:9-36).  w [M,N]; packed int32 [M/8, N]; s f16 [M/128, N/128];
 * s4, z4 int8 [M, N/128].  M % 128 == 0, N % 128 == 0. */
B200MOE_API int b200moe_weight_quant_w4a8(const void* w, int w_dtype, void* packed_i32, void* s_f16,
                              int8_t* s4, int8_t* z4, int64_t M, int64_t N, void* stream);

/* Asymmetric group-128 int4 quantizer, the inverse of b200moe_w4a16_expand_bf16 (extends
 * QuantUtils.fake_quantize, fast_dequant/simple_marlin/utils.py:98-136, with a zero-point): per
 * (row, 128 columns) scale = bf16(max((max - min)/15, 1e-8)), zero = bf16(clamp(rint(-min/scale),
 * 0, 15)), q = clamp(rint(w/scale) + zero, 0, 15), packed over columns (quantization/bitpack.py:38-67).
 * w [rows, K]; packed int32 [rows, K/8]; scale, zero bf16 [rows, K/128].  K % 128 == 0. */
B200MOE_API int b200moe_weight_quant_w4a16(const void* w, int w_dtype, void* packed_i32, void* scale_bf16,
                               void* zero_bf16, int64_t rows, int64_t K, void* stream);

/* Grouped int8 x int8 GEMM with 1x128 / 128x128 f32 scales: the grouped form of
 * w4a8_gemm (quantization/w4a8_kernel.py:317-448) once the weights are int8
 * (b200moe_w4a8_expand_int8): acc += float(dot_kb in s32) * a_s[m,kb] * b_s[n/128,kb].
 * Arguments as b200moe_grouped_gemm_fp8 with epilogue 0; a, b are int8. */
B200MOE_API int b200moe_grouped_gemm_i8(const void* a, int64_t a_row_stride_bytes, const float* a_s,
                            int64_t a_s_row_stride, const void* b, const float* b_s, void* c,
                            int c_dtype, int64_t c_row_stride_bytes, int64_t M_total, int64_t N,
                            int64_t K, int num_groups, int num_weights,
                            const int64_t* seg_indptr, const int64_t* weight_indices,
                            int32_t* status_word, const b200moe_gemm_opts* opts, void* stream);

/* Grouped w4a8 GEMM with the int4 -> int8 step inside the kernel: w4a8_gemm (quantization/w4a8_kernel.py:317-448,
 * unpack and (q - z4) * s4 in its K loop at :362-380), grouped as grouped_gemm_triton
 * (moe/group_gemm_kernel.py:291-513).  The packed weights go from HBM to shared memory as they are (0.5 byte per
 * weight); converter warps split the words into nibbles with byte permutes, apply (q - z4) * s4 four values at a time
 * and write the int8 operand tile the tensor core reads.  Results are bit-identical to b200moe_w4a8_expand_int8
 * followed by b200moe_grouped_gemm_i8.  Each weight tile is converted once per m-tile, so this is the entry point
 * for few rows per group (decode); with many rows per expert, expand once and use b200moe_grouped_gemm_i8.
 *   a int8 [M_total, K], a_s f32 [M_total, K/128] (row strides given); b_packed int32 [num_weights, N/8, K]
 *   (pack_weights_over_rows, quantization/bitpack.py:9-36); s4z4_t int8 [num_weights, K/128, N, 2]: the pairs
 *   (s4[n,kb], z4[n,kb]) of quantization/w4a8_kernel.py:228-262, transposed so that one K block's pairs are
 *   contiguous; b_s f32 [num_weights, N/128, K/128].
 *   epilogue 0: c [M_total, N] f32/f16/bf16.  epilogue 1 / 4: SiLU(gate)*up / GELU(gate)*up with the roundings of the
 *   unfused chain (moe/group_gemm_kernel.py:120-235), then act_quant of quantization/w4a8_kernel.py:145-193
 *   (s = amax/127, y = floor(h/s + 0.5)): c int8 [M_total, N/2], c_s f32 [M_total, N/256] holding the f16-rounded
 *   scales.  K % 128 == 0, N % 128 == 0 (fused epilogues: N % 256 == 0). */
B200MOE_API int b200moe_grouped_gemm_w4a8(const void* a, int64_t a_row_stride_bytes, const float* a_s,
                              int64_t a_s_row_stride, const void* b_packed, const void* s4z4_t,
                              const float* b_s, void* c, int c_dtype, int64_t c_row_stride_bytes,
                              float* c_s, int64_t c_s_row_stride, int64_t M_total, int64_t N, int64_t K,
                              int num_groups, int num_weights, const int64_t* seg_indptr,
                              const int64_t* weight_indices, int epilogue, int32_t* status_word,
                              void* stream);

/* Grouped w4a16 GEMM (asymmetric group-128 int4 weights, bf16 activations) with the dequantization inside the kernel:
 * the counterpart, for few rows per group, of the reference's w4a16 kernel that dequantizes in registers
 * (fast_dequant/simple_marlin/marlin_w4a16_gemm.cu:44-64, 86-280), here with a zero-point and bf16.  Packed words travel
 * from HBM as they are; converter warps turn each word into eight bf16 values (q - zero) * scale (0x4300 | q is the bf16
 * number 128 + q; two exact subtractions, one rounded product) and write the operand tile the tensor core reads; the
 * K loop accumulates in TMEM.  Bit-identical to b200moe_w4a16_expand_bf16 followed by b200moe_grouped_gemm_bf16.
 *   a bf16 [M_total, K]; b_packed int32 [num_weights, N, K/8] (pack_weights_over_cols, quantization/bitpack.py:38-67);
 *   scale_zero_t bf16 [num_weights, K/128, N, 2]: (scale, zero) pairs with one K group's pairs contiguous.
 *   epilogue 0: c [M_total, N] f32/f16/bf16; 2 / 5: SiLU(gate)*up / GELU(gate)*up, c bf16 [M_total, N/2].
 *   K % 128 == 0, N % 128 == 0 (fused epilogues: N % 256 == 0). */
B200MOE_API int b200moe_grouped_gemm_w4a16(const void* a, int64_t a_row_stride_bytes, const void* b_packed,
                               const void* scale_zero_t, void* c, int c_dtype, int64_t c_row_stride_bytes,
                               int64_t M_total, int64_t N, int64_t K, int num_groups, int num_weights,
                               const int64_t* seg_indptr, const int64_t* weight_indices, int epilogue,
                               int32_t* status_word, void* stream);

/* Grouped bf16 x bf16 GEMM with f32 accumulation in TMEM (the unquantized branch of
 * grouped_gemm_triton, moe/group_gemm_kernel.py:410-412; used by the w4a16 path after
 * b200moe_w4a16_expand_bf16).  a bf16 [M_total, K] (row stride in bytes), b bf16
 * [num_weights, N, K].  epilogue 0: c [M_total, N] f32/f16/bf16.  epilogue 2: SwiGLU
 * (moe/group_gemm_kernel.py:120-168) fused, b rows [0,N/2) gate and [N/2,N) up,
 * c bf16 [M_total, N/2].  epilogue 3: c (f16/bf16) = round(c + round(a . b^T)), the sum formed when
 * a module's output is added to a tensor of the same dtype (shared experts,
 * moe/all2all_moe.py:182-183).  epilogue 5: as 2 with the tanh-GELU of :176-235.
 * K % 64 == 0, N % 128 == 0 (epilogues 2 and 5: N % 256 == 0). */
B200MOE_API int b200moe_grouped_gemm_bf16(const void* a, int64_t a_row_stride_bytes, const void* b, void* c,
                              int c_dtype, int64_t c_row_stride_bytes, int64_t M_total, int64_t N,
                              int64_t K, int num_groups, int num_weights,
                              const int64_t* seg_indptr, const int64_t* weight_indices,
                              int epilogue, int32_t* status_word, const b200moe_gemm_opts* opts, void* stream);

/* Same with f16 operands (plain epilogue only): the matrix product of the reference's w4a16
 * `mul` (fast_dequant/simple_marlin/marlin_w4a16_gemm.cpp:23-111) after
 * b200moe_marlin_expand_f16. */
B200MOE_API int b200moe_grouped_gemm_f16(const void* a, int64_t a_row_stride_bytes, const void* b, void* c,
                             int c_dtype, int64_t c_row_stride_bytes, int64_t M_total, int64_t N,
                             int64_t K, int num_groups, int num_weights,
                             const int64_t* seg_indptr, const int64_t* weight_indices,
                             int32_t* status_word, const b200moe_gemm_opts* opts, void* stream);

/* Expands Marlin-order symmetric int4 weights (QuantUtils.pack,
 * fast_dequant/simple_marlin/utils.py:53-95; dequantization of
 * marlin_w4a16_gemm.cu:44-64: (q - 8) * scale) to f16 in nn.Linear layout.
 * packed int32 [K/16, N*2]; scales f16 [K/groupsize, N] (one row when groupsize == -1) in the
 * permuted order QuantUtils.pack returns; out f16 [N, K].  The weight and scale permutations of
 * utils.py:20-46 are evaluated inside the kernel (no tables, no state shared between calls).
 * K % 16 == 0, N % 64 == 0. */
B200MOE_API int b200moe_marlin_expand_f16(const void* packed, const void* scales_f16, void* out_f16,
                              int64_t K, int64_t N, int64_t groupsize, void* stream);

/* QuantUtils.pack (fast_dequant/simple_marlin/utils.py:53-95) on the device: q int32 [K, N] with
 * values 0..15 -> packed int32 [K/16, N*2]; scales f16 [K/groupsize, N] -> scales_out in the
 * permuted column order (blocks of 64 columns, or of 32 when groupsize == -1). */
B200MOE_API int b200moe_marlin_pack(const int32_t* q, void* packed_i32, const void* scales_f16,
                        void* scales_out_f16, int64_t K, int64_t N, int64_t groupsize, void* stream);

/* ============ expert-parallel exchange folded into the kernels ============= */
/* Replaces the two all_to_all_single calls and the host-side split lists of
 * moe/all2all_moe.py:131-262 when every rank has peer mappings of every rank's buffers.
 *
 * b200moe_ep_plan: counts_all int64 [ep_size, num_experts] (row s = slots rank s routes to each
 * global expert; expert e lives on rank e / (num_experts / ep_size)), all on the device.
 * recv_base / back_base: int64 [ep_size] device arrays with the address, as mapped in THIS
 * process, of each rank's receive buffer ([cap_rows] records of rec_bytes) and return buffer
 * (rows of back_row_bytes in the owner's sorted slot order).  Outputs, all on the device:
 *   dst_base  int64 [num_experts]  where my first record for expert e goes (0 = dropped: the block
 *                                  (expert, source rank) does not fit whole into the owner's buffer;
 *                                  the owner applies the same rule and computes only the rows before
 *                                  the first block it rejects; info[1] is set on both sides)
 *   local_seg int64 [E/ep + 1]     group table of my local experts over my receive buffer, rows
 *                                  ordered (expert, source rank)
 *   back_addr int64 [cap_rows]     return address of every row I receive (c_row_addr of the
 *                                  down projection)
 *   info      int32 [2]            {rows received, overflow flag}
 * workspace: b200moe_ep_plan_workspace_bytes(ep_size, num_experts) bytes, 8-byte aligned. */
B200MOE_API int64_t b200moe_ep_plan_workspace_bytes(int ep_size, int num_experts);
B200MOE_API int b200moe_ep_plan(const int64_t* counts_all, int rank, int ep_size, int num_experts,
                    int64_t cap_rows, const int64_t* recv_base, int64_t rec_bytes,
                    const int64_t* back_base, int64_t back_row_bytes, int64_t* dst_base,
                    int64_t* local_seg, int64_t* back_addr, int32_t* info, void* workspace,
                    int64_t workspace_bytes, void* stream);

/* permute_quant_fp8 whose records go straight to their owners: the record of a slot routed to
 * expert e, at position d = src2dst[slot] of my sorted order, is stored at
 * dst_base[e] + (d - seg_indptr[e]) * rec_bytes: H e4m3 bytes, then H/128 f32 scales at byte H.
 * The stores may cross NVLink; the kernel ends with a system-scope fence, and the caller orders
 * the owner's reads behind a barrier across ranks.  back_local (may be NULL): this rank's own return
 * buffer, rows of back_row_bytes in sorted slot order; the rows of slots whose records were dropped
 * (dst_base == 0) are cleared, so a later weighted sum adds zeros for them. */
B200MOE_API int b200moe_permute_quant_fp8_push(const void* x, int x_dtype, const int32_t* src2dst,
                                   const int64_t* topk_ids, const int64_t* seg_indptr,
                                   const int64_t* dst_base, int num_experts, int64_t T, int topk,
                                   int64_t H, int64_t rec_bytes, void* back_local,
                                   int64_t back_row_bytes, void* stream);

/* ========================= quantization/bitpack.py ======================== */

/* pack_weights_over_rows / _cols (quantization/bitpack.py:9-67, 84-149,
 * 228-293): fields of nbits (1,2,4,8) packed little-end-first into words of
 * width bits (8,16,32).  over_rows != 0: out [R/e, C], word r field i =
 * w[e*r+i, c]; else out [R, C/e], word c field i = w[r, e*c+i]; e = width/nbits.
 * w is uint8 [R, C]. */
B200MOE_API int b200moe_pack_bits(const uint8_t* w, void* out, int64_t R, int64_t C,
                      int nbits, int width, int over_rows, void* stream);
/* unpack_over_rows / _cols (quantization/bitpack.py:152-226, 296-373): inverse
 * of the above into uint8 [R, C]. */
B200MOE_API int b200moe_unpack_bits(const void* packed, uint8_t* out, int64_t R, int64_t C,
                        int nbits, int width, int over_rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
