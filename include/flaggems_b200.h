/*
 * flaggems_b200 — C ABI of the B200 (sm_100a) FP8 quantized-inference kernels.
 *
 * Every entry point takes raw device pointers, explicit sizes and strides
 * (strides in ELEMENTS unless a name says bytes) and the CUDA stream to launch
 * on (a cudaStream_t passed as void*; NULL = legacy default stream).  Nothing is
 * allocated inside unless stated, nothing is retained after return, and there is
 * no host synchronisation.  Return value: FG_OK or a negative FG_ERR_* code;
 * fg_last_error() gives the text for the calling thread.
 *
 * Each declaration names the function of the reference (FlagGems, paths relative
 * to its repository root) whose device work it replaces.
 */
#ifndef FLAGGEMS_B200_H
#define FLAGGEMS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FG_OK 0
#define FG_ERR_INVALID_ARGUMENT (-1)
#define FG_ERR_UNSUPPORTED (-2)
#define FG_ERR_CUDA (-3)
#define FG_ERR_DEVICE_STATUS (-4)

/* element type codes */
#define FG_DTYPE_BF16 0
#define FG_DTYPE_F16 1
#define FG_DTYPE_F32 2
#define FG_DTYPE_E4M3 3 /* output of fg_scaled_mm_fp8 only */

/* scale layout codes of fg_scaled_mm_fp8 / fg_moe_grouped_gemm_fp8 */
#define FG_SCALE_SCALAR 0 /* one fp32 value                        */
#define FG_SCALE_VECTOR 1 /* one value per row of A / column of C  */
#define FG_SCALE_BLOCK 2  /* 1x128 groups of A, 128x128 blocks of B */

int fg_version(void);
const char* fg_last_error(void);

/* Reads and clears the device-side status word of the current device (this call
 * synchronises the device).  *status is 0 when no kernel reported a problem; otherwise
 * (code << 16) | site of the first report: code 1 = a bounded wait ran out, code 2 = a row of
 * the expert-parallel exchange was addressed outside its buffer and was dropped.
 * Returns FG_OK, or FG_ERR_DEVICE_STATUS when *status != 0. */
int fg_device_status(unsigned int* status);

/* Failure-detection self-test (no counterpart in the reference): launches one thread that waits,
 * with the same bounded wait every kernel of this library uses, on a barrier that nothing will
 * ever complete.  The wait gives up after limit_ns (at most 100 ms), the kernel returns
 * normally and fg_device_status() then reports (1 << 16) | site.  The context stays usable. */
int fg_selftest_bounded_wait(int64_t limit_ns, int site, void* stream);

/* Number of kernel launches issued by this library in the calling process. */
uint64_t fg_launch_count(void);

/* ---- activation quantisation --------------------------------------------- */

/* act_quant_triton: src/flag_gems/fused/act_quant.py:111-174 (kernel :45-108).
 * x bf16 [M,N] (row stride ld_x), y e4m3 [M,N], s fp32 [M, N/block] (row stride
 * ld_s).  amax clamped to 1e-4, s = amax * fp32(1/448), round_pow2 != 0 rounds s
 * up to a power of two by the exponent/mantissa test (:22-41), y = x * (1/s). */
int fg_act_quant_bf16_e4m3(const void* x, void* y, float* s, int64_t M, int64_t N, int block,
                           int64_t ld_x, int64_t ld_y, int64_t ld_s, int round_pow2, void* stream);

/* per_token_group_quant_fp8: src/flag_gems/ops/per_token_group_quant_fp8.py:227-336
 * (kernels :34-216).  x [M,K] of x_dtype, q e4m3 [M,K] (row stride ld_q),
 * s[m*s_row_stride + g*s_col_stride] fp32 (any layout, column-major included).
 * s = max(amax, eps) / 448 (IEEE divide), ue8m0 != 0: s = 2^ceil(log2(max(|s|,1e-10))),
 * q = x / s. */
int fg_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K,
                                 int group, int64_t ld_x, int64_t ld_q, int64_t s_row_stride,
                                 int64_t s_col_stride, float eps, int ue8m0, void* stream);

/* Per-token branch of _fp8_quantize: src/flag_gems/fused/fused_moe.py:673-684.
 * s[m] = max(max(rowamax,1e-10)/448, 1/(448*512)), q = x / s.
 * row_index (nullable): when given, output row r reads input row row_index[r] / index_div
 * if row_index[r] < index_limit and is written as zeros otherwise (the gather of routed
 * rows into expert-sorted order); n_rows_dev (nullable) is a device int giving how many
 * output rows to produce (at most M). */
int fg_per_token_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K,
                           int64_t ld_x, int64_t ld_q, const int32_t* row_index, int32_t index_div,
                           int32_t index_limit, const int32_t* n_rows_dev, void* stream);

/* Per-token branch of _int8_quantize: src/flag_gems/fused/fused_moe.py:732-739.
 * s[m] = max(rowamax, 1e-10) / 127, q = clamp(round_half_even(x / s), -128, 127) as int8 bytes.
 * Row gather options as above. */
int fg_per_token_quant_int8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K,
                            int64_t ld_x, int64_t ld_q, const int32_t* row_index, int32_t index_div,
                            int32_t index_limit, const int32_t* n_rows_dev, void* stream);

/* Per-tensor branches of _fp8_quantize: src/flag_gems/fused/fused_moe.py:686-698.
 * dynamic == 0 (static scale given): q = x / scale_or_amax[0].
 * dynamic != 0: scale_or_amax[0] holds max|x| over the tensor (fg_abs_max); s = max(amax,1e-10)/448,
 * q = x * (1/s), and s is written to scale_out[0].  Row gather options as above. */
int fg_per_tensor_quant_fp8(const void* x, int x_dtype, void* q, const float* scale_or_amax, int dynamic,
                            float* scale_out, int64_t M, int64_t K, int64_t ld_x, int64_t ld_q,
                            const int32_t* row_index, int32_t index_div, int32_t index_limit,
                            const int32_t* n_rows_dev, void* stream);

/* max|x| over x[0:M, 0:K] into amax[0], which the caller has set to zero (the `A.abs().amax()` of
 * the same reference lines).  n_rows_dev (nullable): device-side row count. */
int fg_abs_max(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ld_x, const int32_t* n_rows_dev,
               float* amax, void* stream);

/* Same gather options for the per-group form (used by the block-FP8 MoE path;
 * src/flag_gems/fused/fused_moe.py:647-659 feeding :2016-2023). Scales are written
 * row-major [M, K/group]. */
int fg_per_token_group_quant_fp8_gather(const void* x, int x_dtype, void* q, float* s, int64_t M,
                                        int64_t K, int group, int64_t ld_x, int64_t ld_q,
                                        const int32_t* row_index, int32_t index_div,
                                        int32_t index_limit, const int32_t* n_rows_dev,
                                        void* stream);

/* ---- fused-MoE glue -------------------------------------------------------- */

/* moe_align_block_size / moe_align_block_size_triton:
 * src/flag_gems/fused/moe_align_block_size.py:789-820, :520-664 (stages :404-517).
 * topk_ids: numel route slots, int32 (ids_are_i64 == 0) or int64.  Writes
 * sorted_ids[max_pad] (route indices grouped by expert, ascending inside an expert,
 * each expert padded to block_size with the value numel), expert_ids[n_blocks]
 * (-1 past the used blocks) and num_post_pad[0].  expert_map (nullable, length
 * expert_map_len): every expert_ids entry v becomes expert_map[v] with Python
 * index semantics for v == -1 (:817-818). */
int fg_moe_align_block_size(const void* topk_ids, int ids_are_i64, int64_t numel, int num_experts,
                            int block_size, const int32_t* expert_map, int expert_map_len,
                            int32_t* sorted_ids, int64_t max_pad, int32_t* expert_ids,
                            int64_t n_blocks, int32_t* num_post_pad, void* stream);

/* Same kernel with three extras used by the expert-parallel layer (no counterpart in the
 * reference, which has no dispatch step): ids are read with a stride of ids_stride elements,
 * the bucket of a slot is id / id_div (id_div = experts per rank turns expert ids into
 * destination ranks), expert_counts (nullable) receives the unpadded rows per bucket, and
 * numel_dev (nullable) is a device-side slot count: numel is then only the capacity (and the
 * padding value), so a step needs no host round trip to learn how many rows arrived.
 * expert_ids may be NULL here when the caller only needs the order and the counts. */
int fg_moe_align_block_size_ex(const void* topk_ids, int ids_are_i64, int64_t numel, int num_experts,
                               int block_size, const int32_t* expert_map, int expert_map_len,
                               int32_t* sorted_ids, int64_t max_pad, int32_t* expert_ids,
                               int64_t n_blocks, int32_t* num_post_pad, int64_t ids_stride, int id_div,
                               int32_t* expert_counts, const int32_t* numel_dev, void* stream);

/* Same again for a slot range that is split into regions (no counterpart in the reference): the
 * numel slots are numel / region_rows regions of region_rows slots, and only the first
 * region_counts[s * region_stride] slots of region s hold rows (counts are clamped to
 * [0, region_rows]); the other slots are skipped without being read.  This is the receive buffer
 * of the expert-parallel layer, where every source rank owns one region.  region_rows == 0:
 * no regions. */
int fg_moe_align_block_size_regions(const void* topk_ids, int ids_are_i64, int64_t numel, int num_experts,
                                    int block_size, const int32_t* expert_map, int expert_map_len,
                                    int32_t* sorted_ids, int64_t max_pad, int32_t* expert_ids, int64_t n_blocks,
                                    int32_t* num_post_pad, int64_t ids_stride, int id_div, int32_t* expert_counts,
                                    const int32_t* numel_dev, int64_t region_rows, const int32_t* region_counts,
                                    int64_t region_stride, void* stream);

/* silu_and_mul_out / _silu_and_mul_kernel: src/flag_gems/fused/silu_and_mul.py:26-31,66-69,
 * src/flag_gems/fused/fused_moe.py:795-800.  out = dtype(x32/(1+exp(-x32)) * y32). */
int fg_silu_and_mul(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t ld_x,
                    int64_t ld_y, int64_t ld_out, int dtype, void* stream);

/* topk_softmax: src/flag_gems/fused/topk_softmax.py:84-137 (kernel :24-81); vLLM op
 * _moe_C::topk_softmax.  gating_output [T, E] (bf16/fp16/fp32, contiguous), softmax in fp32 with
 * 1e-8 added to the denominator, then topk rounds of arg-max (ties to the lower expert index).
 * topk_weights fp32 [T, topk]; topk_indices [T, topk] with index_kind 0 int32, 1 uint32, 2 int64;
 * token_expert_indices[t, k] = k * T + t.  renormalize divides by (sum of the topk + 1e-8).
 * topk <= 32 (assert of :94), E <= 1024 (block size cap of :107).  expert_counts: NULL, or
 * int32 [E] to which the number of route slots per expert is added (not in the reference: the
 * histogram an expert-parallel dispatch starts from). */
int fg_topk_softmax(float* topk_weights, void* topk_indices, int index_kind, int32_t* token_expert_indices,
                    const void* gating_output, int gating_dtype, int64_t num_tokens, int num_experts, int topk,
                    int renormalize, int32_t* expert_counts, void* stream);

/* grouped_topk: src/flag_gems/fused/grouped_topk.py:245-355 (kernels :24-243); vLLM op
 * _moe_C::grouped_topk.  scores [T, E] with row stride scores_stride, bias [E], both `dtype`.
 * scoring_func 1 applies sigmoid in fp32 and rounds to dtype (:291-294); group score = sum of
 * the two largest (score + bias) of the group (:24-76); the topk_group best groups, then topk
 * rounds of arg-max over (score + bias) inside them, ties to the lower index; weights are the
 * scores without bias times routed_scaling_factor, divided by (their sum + 1e-20) when
 * renormalize.  n_group <= 32, topk <= 32 (:262-265); num_experts <= 2048 (one row of scores per warp
 * in shared memory).  A token whose groups all score -inf gets weights 1/topk and experts 0..topk-1
 * (:221-227).  topk_values fp32, topk_indices int32, both [T, topk].  expert_counts as in
 * fg_topk_softmax. */
int fg_grouped_topk(float* topk_values, int32_t* topk_indices, const void* scores, const void* bias, int dtype,
                    int64_t num_tokens, int num_experts, int64_t scores_stride, int n_group, int topk_group, int topk,
                    int renormalize, float routed_scaling_factor, int scoring_func, int32_t* expert_counts,
                    void* stream);

/* moe_sum: src/flag_gems/fused/moe_sum.py:70-90 (kernel :24-67).
 * in [M, topk, K] contiguous, out [M, K]; fp32 sum in slot order. */
int fg_moe_sum(const void* in, void* out, int64_t M, int topk, int64_t K, int dtype, void* stream);

/* moe_sum with the rows of `in` addressed through row_index[m*topk + k] (negative = skip) and
 * an optional addend [M,K] joined in fp32 before the cast.  Combine step of the
 * expert-parallel layer: the top-k sum of src/flag_gems/fused/moe_sum.py:57-67 applied to
 * rows that came back from other ranks in dispatch order, plus the shared-expert output.
 * (The reference has no dispatch/combine; its own multi-GPU hook is expert_map.) */
int fg_moe_sum_indexed(const void* in, void* out, int64_t M, int topk, int64_t K, int dtype,
                       const int32_t* row_index, const void* addend, void* stream);

/* Copies FP8 rows [*, K] and their fp32 scale rows [*, s_cols] into a new row order:
 * output row r takes source row row_index[r] / index_div when 0 <= row_index[r] < index_limit,
 * else zeros (scales 1).  The A-operand gather the reference does inside fused_moe_kernel
 * (offs_token // top_k, src/flag_gems/fused/fused_moe.py:1101-1110), done ahead of the GEMM so
 * the GEMM reads contiguous tiles by TMA.  n_rows_dev (nullable): device count of rows. */
int fg_gather_rows_fp8(const void* src_q, const float* src_s, void* dst_q, float* dst_s, int64_t rows,
                       int64_t K, int64_t s_cols, int64_t src_q_stride, int64_t src_s_stride,
                       const int32_t* row_index, int32_t index_div, int32_t index_limit,
                       const int32_t* n_rows_dev, void* stream);

/* ---- expert-parallel dispatch format and one-call routed pipeline ------------------------
 * No counterpart in the reference (its multi-GPU hook is expert_map only); the per-row
 * arithmetic is that of fused_experts_impl, src/flag_gems/fused/fused_moe.py:1994-2183.
 *
 * Packed dispatch row (row_bytes, a multiple of 16, >= K + 4*K/128 + 16):
 *   [0, K) e4m3 | [K, K + 4*K/128) fp32 group scales | int32 local expert | fp32 router weight
 *   | int32 route slot at the home rank | int32 home rank. */

/* Quantises (1x128 groups) the tokens x [T,K] into packed rows in send order: output row p is
 * route slot order[p] (token order[p]/topk); its trailer gets topk_ids[slot] % experts_per_rank
 * and topk_w[slot]; inv[slot] = p (nullable). */
int fg_ep_pack_rows_fp8(const void* x, int x_dtype, int64_t T, int64_t K, int64_t ld_x,
                        const void* topk_ids, int ids_are_i64, const void* topk_w, int topk_w_dtype,
                        int topk, int experts_per_rank, int home_rank, const int32_t* order,
                        void* packed, int64_t row_bytes, int32_t* inv, void* stream);

/* Same, writing each packed row straight into the receive buffer of its destination rank over
 * NVLink peer memory (dispatch fused into the quantisation kernel).  send_counts[d] (device) is
 * the number of rows for rank d, rows being in send order with destinations ascending;
 * peer_rows[d] is rank d's receive buffer, in which this rank owns rows
 * [home_rank * region_rows, (home_rank + 1) * region_rows): the k-th row for rank d lands at row
 * home_rank * region_rows + k there, so a rank needs nobody else's counts to send.  A row that
 * would fall outside its region is not stored and the device status word is set (code 2).
 * send_counts == NULL: as above (rows go to `packed`).  With send_counts, a non-NULL `packed`
 * (at least T rows of row_bytes, 16-byte aligned) is a staging area: every token is quantised
 * once into it and its staged row is copied to each of its top-k destinations, instead of being
 * quantised once per route slot; same bytes either way. */
int fg_ep_pack_rows_fp8_peer(const void* x, int x_dtype, int64_t T, int64_t K, int64_t ld_x,
                             const void* topk_ids, int ids_are_i64, const void* topk_w,
                             int topk_w_dtype, int topk, int experts_per_rank, int home_rank,
                             const int32_t* order, void* packed, int64_t row_bytes, int32_t* inv,
                             const int32_t* send_counts, void* const* peer_rows, int world,
                             int64_t region_rows, void* stream);

/* Bytes of workspace the two functions below need for n_rows_in routed rows. */
int64_t fg_moe_routed_workspace_bytes(int64_t n_rows_in, int num_experts, int64_t H, int64_t I);

/* All experts local: y[T*topk, H] (route-slot order) = w2[e] . quant(silu_mul(w1[e] . quant(x)))
 * times the router weight, for every (token, slot).  Five launches (align, quantise+gather,
 * GEMM1+SiLU, quantise, GEMM2), no allocation: scratch is the caller's workspace (256-byte
 * aligned, fg_moe_routed_workspace_bytes(T*topk, ...)). */
int fg_moe_routed_block_fp8_local(void* y, const void* hidden, int hidden_dtype, const void* topk_ids,
                                  int ids_are_i64, const void* topk_w, int topk_w_dtype, int64_t T,
                                  int topk, const void* w1, const void* w2, const float* s1,
                                  const float* s2, int num_experts, int64_t H, int64_t I,
                                  void* workspace, int64_t workspace_bytes, void* stream);

/* fg_moe_routed_block_fp8_local for callers that must not allocate device memory and have no
 * workspace to lend.  It has no counterpart in the reference.  Think of a host that handed the
 * whole device to its own memory planner at start-up (a later cudaMalloc fails or fragments its
 * plan), of code that runs where an allocation would stall every stream of the device, or of a
 * plug-in whose contract leaves all memory management to the embedding process.  The scratch is
 * a fixed array of FG_NOALLOC_SCRATCH_BYTES inside the library image (each GPU that loads the
 * library holds it until the process ends).  Problems whose scratch need (the value
 * fg_moe_routed_workspace_bytes reports) exceeds it are refused with FG_ERR_UNSUPPORTED.
 * This function never calls cudaMalloc, cudaFree or any allocating routine.  Its first call on
 * a device looks up the array's device address (cudaGetSymbolAddress) and, like any first
 * launch, loads kernels: make that call before starting a stream capture.  All calls share the
 * one array and leave their intermediates in it; no part of it has to start at zero because a
 * call writes every element before reading it, but two calls whose kernels overlap on the GPU
 * (different streams, or graphs replayed concurrently) race on it: keep them on one stream. */
#define FG_NOALLOC_SCRATCH_BYTES (32u << 20)
int fg_moe_routed_block_fp8_local_noalloc(void* y, const void* hidden, int hidden_dtype,
                                          const void* topk_ids, int ids_are_i64, const void* topk_w,
                                          int topk_w_dtype, int64_t T, int topk, const void* w1,
                                          const void* w2, const float* s1, const float* s2,
                                          int num_experts, int64_t H, int64_t I, void* stream);

/* Same for R packed rows received from other ranks.  n_peers == 0: y[R, H] in arrival order
 * (to be returned by an all-to-all).  n_peers > 0 (y may be NULL): the combine is fused into
 * GEMM2's epilogue, which stores each result row straight into the home rank's buffer
 * peer_out[home rank] at row (route slot), over NVLink peer memory; the home rank may read its
 * buffer once every rank's call has completed (a stream-ordered barrier or collective).
 * peer_rows is the number of rows each peer_out buffer holds: a row whose trailer names a home
 * rank or slot outside the buffers is dropped and the device status word is set (code 2).
 * n_rows_dev (nullable): device-side row count; R is then the capacity of `rows`.
 * region_rows > 0: `rows` is split into R / region_rows regions as in
 * fg_moe_align_block_size_regions (region_counts, region_stride). */
int fg_moe_routed_block_fp8_packed(void* y, const void* rows, int64_t R, int64_t row_bytes,
                                   const void* w1, const void* w2, const float* s1, const float* s2,
                                   int num_experts, int64_t H, int64_t I, void* workspace,
                                   int64_t workspace_bytes, int out_dtype, void* const* peer_out,
                                   int n_peers, int64_t peer_rows, const int32_t* n_rows_dev,
                                   int64_t region_rows, const int32_t* region_counts,
                                   int64_t region_stride, void* stream);

/* fg_moe_grouped_gemm_fp8 with the peer scatter described above: with scatter != 0 and
 * n_peers > 0, row r (arrival index sid = sorted_ids[r]) goes to peer_out[dest[sid*dest_stride+1]]
 * at row dest[sid*dest_stride], provided that rank is below n_peers and the row below peer_rows
 * (otherwise the row is dropped and the device status word is set, code 2). */
int fg_moe_grouped_gemm_fp8_peer(void* c, const void* a, const void* w, const float* a_scale,
                                 const float* w_scale, const void* topk_weights, int topk_w_dtype,
                                 int64_t topk_w_stride, const int32_t* sorted_ids,
                                 const int32_t* expert_ids, const int32_t* num_post_pad,
                                 int64_t max_rows, int64_t numel, int num_experts, int64_t N,
                                 int64_t K, int64_t ld_a, int64_t ld_c, int block_rows,
                                 int scale_mode, int a_scale_per_row, int fuse_silu, int scatter,
                                 int mul_weight, int out_dtype, const int32_t* dest,
                                 int64_t dest_stride, void* const* peer_out, int n_peers,
                                 int64_t peer_rows, void* stream);

/* Buffers visible to every rank of one node (set-up time only; these four are the only entry
 * points that allocate or free device memory).  fg_symm_alloc: cudaMalloc + a 64-byte CUDA IPC
 * handle to pass to the other processes; fg_symm_open maps a peer's buffer (peer access is
 * enabled on first use); fg_symm_close / fg_symm_free undo them. */
int fg_symm_alloc(int64_t bytes, void** ptr, unsigned char* handle64);
int fg_symm_open(const unsigned char* handle64, void** ptr);
int fg_symm_close(void* ptr);
int fg_symm_free(void* ptr);

/* ---- scaled FP8 matrix products (tcgen05 / TMEM / TMA) ---------------------- */

/* cutlass_scaled_mm (scalar / per-token / per-channel scales):
 * src/flag_gems/fused/cutlass_scaled_mm.py:475-526, dispatch :371-431, kernel :207-314;
 * aten _scaled_mm: src/flag_gems/ops/scaled_mm.py:333-452 (bias_after_round = 0).
 * a e4m3 [M,K] row-major (ld_a), b e4m3 given as its [N,K] K-contiguous storage
 * (ld_b = elements between consecutive n, i.e. b.stride(1) of the column-major
 * [K,N] view), c [M,N] of out_dtype (ld_c).  c = out(sb[n] * (sa[m] * acc)) then
 * + bias in the output type (bias_after_round != 0) or + bias in fp32 before the
 * cast.  sa_mode/sb_mode: FG_SCALE_SCALAR or FG_SCALE_VECTOR.  K % 16 == 0.
 * out_dtype FG_DTYPE_E4M3 (the aten default, out_dtype=None -> the operands' type,
 * src/flag_gems/ops/scaled_mm.py:214-220): c holds e4m3 bytes, rounded to nearest even and
 * saturated at +-448; the bias is then fp32 and joins before the cast. */
int fg_scaled_mm_fp8(void* c, const void* a, const void* b, const float* sa, const float* sb,
                     const void* bias, int64_t M, int64_t N, int64_t K, int64_t ld_a, int64_t ld_b,
                     int64_t ld_c, int sa_mode, int sb_mode, int out_dtype, int bias_after_round,
                     void* stream);

/* w8a8_block_fp8_matmul / fp8_matmul / blockwise cutlass_scaled_mm:
 * src/flag_gems/ops/w8a8_block_fp8_matmul.py:173-232 (kernel :51-122),
 * src/flag_gems/ops/fp8_matmul.py:137-205,
 * src/flag_gems/fused/cutlass_scaled_mm.py:153-194.
 * a e4m3 [M,K], b e4m3 [N,K]; a_s[m*ld_as + kb*as_stride_k] fp32 (row-major [M, K/128] or the
 * column-major layout of column_major_scales, which the kernel reads coalesced);
 * b_s[nb*bs_stride_n + kb*bs_stride_k] fp32; block sizes fixed at 128x128.
 * C[m,n] = out(sum_kb (A_kb . B_kb) * a_s[m,kb] * b_s[n/128,kb]). */
int fg_block_scaled_mm_fp8(void* c, const void* a, const void* b, const float* a_s,
                           const float* b_s, int64_t M, int64_t N, int64_t K, int64_t ld_a,
                           int64_t ld_b, int64_t ld_c, int64_t ld_as, int64_t as_stride_k,
                           int64_t bs_stride_n, int64_t bs_stride_k, int out_dtype, void* stream);

/* Grouped expert GEMM of the fused MoE layer: fused_moe_kernel /
 * invoke_fused_moe_triton_kernel / dispatch_fused_moe_kernel,
 * src/flag_gems/fused/fused_moe.py:1015-1509, :1602-1727, :1730-1818.
 *
 * a: e4m3 [rows, K] already in expert-sorted padded order (row r belongs to route
 * slot sorted_ids[r]); w: e4m3 [E, N, K]; block b of block_rows sorted rows uses
 * expert expert_ids[b] (blocks with -1 produce zeros, :1350-1364); only rows below
 * num_post_pad[0] are processed.  scale_mode: FG_SCALE_SCALAR (per-tensor: a_scale[0]
 * or per-row when a_scale_per_row, w_scale[e]), FG_SCALE_VECTOR (a_scale[r] per
 * sorted row, w_scale[e*N + n]) or FG_SCALE_BLOCK (a_scale [rows, K/128],
 * w_scale [E, ceil(N/128), K/128]).
 * fuse_silu != 0: N = 2*I, output c[r, 0:I] = silu(gate) * up in sorted order
 * (FUSE_SILU branch :1186-1347); else c gets N columns.
 * scatter != 0: row r is written to c row sorted_ids[r] (skipped when
 * sorted_ids[r] >= numel) instead of row r; mul_weight != 0 multiplies by
 * topk_weights[sorted_ids[r] * topk_w_stride] in fp32 before the cast (:1485-1493). */
int fg_moe_grouped_gemm_fp8(void* c, const void* a, const void* w, const float* a_scale,
                            const float* w_scale, const void* topk_weights, int topk_w_dtype,
                            int64_t topk_w_stride, const int32_t* sorted_ids, const int32_t* expert_ids,
                            const int32_t* num_post_pad, int64_t max_rows, int64_t numel,
                            int num_experts, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c,
                            int block_rows, int scale_mode, int a_scale_per_row, int fuse_silu,
                            int scatter, int mul_weight, int out_dtype, void* stream);

/* The same grouped GEMM on signed 8-bit operands with 32-bit integer accumulation (tcgen05 kind::i8):
 * the int8 w8a8 branches of fused_moe_kernel, src/flag_gems/fused/fused_moe.py:1198-1347, :1466-1479.
 * a, w: int8; scale_mode FG_SCALE_SCALAR or FG_SCALE_VECTOR; everything else as above. */
int fg_moe_grouped_gemm_int8(void* c, const void* a, const void* w, const float* a_scale,
                             const float* w_scale, const void* topk_weights, int topk_w_dtype,
                             int64_t topk_w_stride, const int32_t* sorted_ids, const int32_t* expert_ids,
                             const int32_t* num_post_pad, int64_t max_rows, int64_t numel,
                             int num_experts, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c,
                             int block_rows, int scale_mode, int a_scale_per_row, int fuse_silu,
                             int scatter, int mul_weight, int out_dtype, void* stream);

/* The same grouped GEMM on bf16 or fp16 operands with fp32 accumulation (tcgen05 kind::f16): the
 * unquantised path of fused_moe_kernel (src/flag_gems/fused/fused_moe.py:1016, accumulate at :1468) and, with the
 * integer weights converted to the activation type and their per-channel scales passed as w_scale,
 * the weight-only int8 / int4 forms (:1976-1983).  a: [max_rows, K], w: [E, N, K], both of
 * operand_dtype, K a multiple of 8; scale_mode FG_SCALE_SCALAR (a_scale[0] or per row, w_scale[e]) or
 * FG_SCALE_VECTOR (a_scale[row], w_scale[e, n]); pass ones for an unscaled product. */
int fg_moe_grouped_gemm_16bit(void* c, const void* a, const void* w, const float* a_scale,
                              const float* w_scale, const void* topk_weights, int topk_w_dtype,
                              int64_t topk_w_stride, const int32_t* sorted_ids, const int32_t* expert_ids,
                              const int32_t* num_post_pad, int64_t max_rows, int64_t numel,
                              int num_experts, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c,
                              int block_rows, int scale_mode, int a_scale_per_row, int fuse_silu,
                              int scatter, int mul_weight, int operand_dtype, int out_dtype, void* stream);

/* ---- aten _scaled_grouped_mm ------------------------------------------------ */

/* scaled_grouped_mm, the "A 2-D, B 3-D" form: src/flag_gems/ops/scaled_grouped_mm.py:470-583 (kernel
 * :65-240).  a e4m3 [m_total, K] (row stride ld_a), rows [offs[g-1], offs[g]) belong to group g
 * (offs: device int32 [num_groups], ascending, offs[-1] <= m_total); b e4m3 [num_groups, N, K]
 * contiguous (the K-contiguous storage of the reference's [G, K, N] operand); scale_a fp32 [m_total],
 * scale_b fp32 [num_groups, N]; bias fp32, NULL, one row [N] (bias_stride_g = 0) or one row per
 * group (bias_stride_g = N).  c[m, n] = out((acc * scale_a[m]) * scale_b[g, n] + bias) (ld_c).
 * The other three forms of the reference op (both 3-D, B 2-D, both 2-D) are composed from this one by
 * the Python host.  Group ends are read on the device: no host synchronisation.  Scratch is the
 * caller's workspace of fg_scaled_grouped_mm_workspace_bytes(m_total, num_groups, K) bytes, 256-byte
 * aligned. */
int64_t fg_scaled_grouped_mm_workspace_bytes(int64_t m_total, int num_groups, int64_t K);
int fg_scaled_grouped_mm_fp8(void* c, const void* a, const void* b, const float* scale_a, const float* scale_b,
                             const float* bias, int64_t bias_stride_g, const int32_t* offs, int num_groups,
                             int64_t m_total, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c, int out_dtype,
                             void* workspace, int64_t workspace_bytes, void* stream);

/* Pieces of the above.  fg_group_ids_from_offsets: ids[r] = number of offsets <= r (the group of
 * row r; num_groups for rows past the last end).  fg_grouped_gemm_fp8_bias: the grouped GEMM of
 * fused_moe_kernel (src/flag_gems/fused/fused_moe.py:1015-1509) with per-row x per-column scales, rows
 * scattered back through sorted_ids, and an fp32 bias added before the cast. */
int fg_group_ids_from_offsets(const int32_t* offs, int num_groups, int64_t rows, int32_t* ids, void* stream);
int fg_grouped_gemm_fp8_bias(void* c, const void* a, const void* w, const float* a_scale, const float* w_scale,
                             const float* bias, int64_t bias_stride_g, const int32_t* sorted_ids,
                             const int32_t* expert_ids, const int32_t* num_post_pad, int64_t max_rows,
                             int64_t numel, int num_groups, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c,
                             int out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLAGGEMS_B200_H */
