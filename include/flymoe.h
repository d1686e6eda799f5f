/* flymoe_sm100 — C ABI of the B200 (sm_100a) FP8 block-scaled fused-MoE library.
 *
 * Every entry point takes raw device pointers, explicit sizes and a CUDA stream
 * (cudaStream_t passed as void*), enqueues work on that stream and returns
 * immediately: no host synchronisation and no allocation on the call path.  The
 * caller owns every buffer, including scratch.  Return value: 0 on success or a
 * negative FLYMOE_ERR_* code; flymoe_last_error() gives the text for the calling
 * thread.  No C++ exceptions cross this boundary.
 *
 * Each declaration cites the interface of the reference project (FlyDSL) that it
 * replaces, by file:line inside that project.
 */
#ifndef FLYMOE_H_
#define FLYMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLYMOE_ABI_VERSION 1

#define FLYMOE_OK 0
#define FLYMOE_ERR_INVALID_ARGUMENT (-1)
#define FLYMOE_ERR_CUDA (-2)
#define FLYMOE_ERR_UNSUPPORTED (-3)
#define FLYMOE_ERR_WORKSPACE (-4)
#define FLYMOE_ERR_DEVICE_TIMEOUT (-5)

/* element types */
#define FLYMOE_F32 0
#define FLYMOE_F16 1
#define FLYMOE_BF16 2
#define FLYMOE_E4M3 3
#define FLYMOE_I8 4

/* how the operands of a grouped GEMM are scaled */
#define FLYMOE_SCALE_BLOCK128 0  /* activations per (row, 128 K), weights per 128x128 block        */
#define FLYMOE_SCALE_PER_TOKEN 1 /* one scale per activation row, one per weight row (out column) */

/* values of the device status word (flymoe_device_status); 0 = healthy */
#define FLYMOE_STATUS_WAIT_FIRST 1        /* 1..7: a bounded wait of the grouped GEMM gave up (role)  */
#define FLYMOE_STATUS_WAIT_LAST 7
#define FLYMOE_STATUS_DISPATCH_OVERFLOW 16 /* flymoe_dispatch_rows dropped rows beyond pos_limit      */
#define FLYMOE_STATUS_ROW_DST_MISALIGNED 17 /* a per-row destination was not 16-byte aligned; dropped */
#define FLYMOE_STATUS_SELFTEST_TIMEOUT 99 /* flymoe_selftest_bounded_wait ran out, as it must        */

/* row layouts of an activation matrix that is indexed through the sorted-id list */
#define FLYMOE_ROWS_BY_TOKEN 0 /* row = token id                     (stage-1 input)   */
#define FLYMOE_ROWS_BY_PAIR 1  /* row = token*topk + slot            (reference layout) */
#define FLYMOE_ROWS_SORTED 2   /* row = position in the sorted list  (fused layer)      */
#define FLYMOE_ROWS_BY_SLOT 3  /* row = slot*num_tokens + token: the slot-major per-(token, slot) rows of the
                                  reference's "int8smooth" stage-1 input (kernels/moe_gemm_2stage.py:546-555) */

/* GEMM implementations */
#define FLYMOE_IMPL_TCGEN05 0 /* TMA + tcgen05.mma + TMEM (the product path)             */
#define FLYMOE_IMPL_SIMT 1    /* plain CUDA-core kernel, used to cross-check on the GPU */

int flymoe_abi_version(void);
const char* flymoe_error_string(int code);
const char* flymoe_last_error(void);

/* Reads (with a device synchronisation) and clears the device-side status word that
 * kernels set when a bounded wait gives up.  0 = no kernel reported a problem. */
int flymoe_device_status(int* status_out);

/* Top-k softmax gating.
 * Replaces kernels/topk_gating_softmax_kernel.py:54-59 (builder) and the launcher
 * :336-344 (GatingOutput, TopkWeights, TopkIndices, TokenExpertIndices, num_tokens, stream).
 * gating [T,E] of gating_dtype (F32/F16/BF16), row-major.  topk_weights f32 [T,k],
 * topk_indices i32 [T,k] (descending by logit, ties to the lower expert id),
 * token_expert_indices i32 [T,k] = k_idx*T + t. */
int flymoe_topk_gating_softmax(const void* gating, int gating_dtype, float* topk_weights,
                               int32_t* topk_indices, int32_t* token_expert_indices,
                               int num_tokens, int num_experts, int topk, int renormalize,
                               void* stream);

/* Scratch (int32 elements) flymoe_moe_sorting needs for this problem; 0 when the
 * single-block path is taken.  Replaces kernels/moe_sorting_kernel.py:1588-1598. */
int64_t flymoe_moe_sorting_workspace_elems(int num_tokens, int num_experts, int topk,
                                           int unit_size);

/* Token-to-expert counting sort with per-expert padding to unit_size rows.
 * Replaces kernels/moe_sorting_kernel.py:1628-1772 (moe_sorting_flydsl).
 * topk_ids i32 [T,k], topk_weights f32 [T,k]; outputs (caller-allocated):
 * sorted_ids i32 [T*k + E*unit - k] packed (slot<<24)|token with pad (k<<24)|T,
 * sorted_weights f32 (same length, pads 0), sorted_expert_ids i32 [ceil(len/unit)]
 * (local expert index under expert_mask, -1 beyond the valid blocks),
 * num_valid_ids i32 [2] = {padded row count, T}.  moe_buf (may be NULL) is zeroed
 * over moe_buf_bytes.  expert_mask i32 [E] or NULL.  workspace: int32 scratch of at
 * least flymoe_moe_sorting_workspace_elems() elements (may be NULL when that is 0). */
int flymoe_moe_sorting(const int32_t* topk_ids, const float* topk_weights, int32_t* sorted_ids,
                       float* sorted_weights, int32_t* sorted_expert_ids, int32_t* num_valid_ids,
                       void* moe_buf, int64_t moe_buf_bytes, const int32_t* expert_mask,
                       int32_t* workspace, int64_t workspace_elems, int num_tokens,
                       int num_experts, int topk, int unit_size, void* stream);

/* Same sort for callers that may not allocate device memory on their call path (a serving
 * loop whose memory pool owns the whole device heap, a plugin living inside another
 * framework's memory budget, code that must never reach the allocator because allocating
 * can synchronise the device).  No counterpart in the reference project.  The scratch the
 * multi-block path needs lives in a 4 MiB array inside the library (held by every GPU that
 * loads it, until exit): problems whose flymoe_moe_sorting_workspace_elems() exceeds
 * flymoe_moe_sorting_noalloc_max_elems() (2^20 int32) are rejected with
 * FLYMOE_ERR_WORKSPACE.  The call itself allocates nothing.  The first call on each
 * device looks up the array's device address; make that first call outside any stream
 * capture.  All calls share the one array: two calls whose kernels may overlap on the
 * GPU (different streams, no dependency between them) race on it. */
int64_t flymoe_moe_sorting_noalloc_max_elems(void);
int flymoe_moe_sorting_noalloc(const int32_t* topk_ids, const float* topk_weights,
                               int32_t* sorted_ids, float* sorted_weights,
                               int32_t* sorted_expert_ids, int32_t* num_valid_ids, void* moe_buf,
                               int64_t moe_buf_bytes, const int32_t* expert_mask, int num_tokens,
                               int num_experts, int topk, int unit_size, void* stream);

/* Copies rows of a one-byte-element matrix into sorted order: dst row r = src row
 * selected by sorted_ids[r] under src_layout (BY_TOKEN or BY_PAIR); pad rows are
 * zero-filled; rows at or beyond num_valid_ids[0] are left untouched.
 * A stand-alone version of the in-kernel gather of kernels/moe_blockscale_2stage.py:401-427 and
 * :1576-1590.  The GEMM stages below can do that gather themselves (x_layout / a_layout BY_TOKEN or
 * BY_PAIR), which is the better choice for row blocks of 16 or 32 rows; for 64 and 128 rows gathering
 * with this entry point first and passing the SORTED layout is faster. */
int flymoe_gather_rows(const void* src, void* dst, const int32_t* sorted_ids,
                       const int32_t* num_valid_ids, int num_tokens, int topk, int row_bytes,
                       int src_layout, int max_rows, void* stream);

/* Stage 1: gate/up grouped FP8 GEMM over sorted rows + SiLU(gate)*up.
 * Replaces kernels/moe_blockscale_2stage.py:70-84 (builder) and the launcher
 * :1142-1157.  x e4m3: [T,H] when x_layout==BY_TOKEN (each sorted row's activations are
 * fetched by token id inside the kernel, as the reference does, :401-427; meant for tile_m 16 or 32),
 * or the [rows,H] matrix already in sorted order (x_layout==SORTED, one TMA box per K block; see
 * flymoe_gather_rows).  scale_x f32, element
 * (kb, row) at kb*sx_stride + row*sx_row_stride: the reference's transposed layout
 * [H/128, rows] is (sx_stride = rows, sx_row_stride = 1), row-major [rows, H/128] is
 * (1, H/128); row = token (x_scale_layout BY_TOKEN) or sorted row.
 * w e4m3 [E,2I,H] row-major (gate rows first), scale_w f32 [E,2I/128,H/128].
 * out: out_dtype F16/BF16 -> [rows,I] values; E4M3 -> codes [rows,I] plus
 * out_scale f32 [I/128, out_scale_stride] (the per-1x128 requantisation that the
 * reference performs outside the kernel, tests/kernels/test_moe_blockscale.py:447-452).
 * out_layout BY_PAIR (reference) or SORTED.  tile_m = sort unit (16/32/64/128). */
int flymoe_moe_gemm1(void* out, float* out_scale, int64_t out_scale_stride, const void* x,
                     const float* scale_x, int64_t sx_stride, int64_t sx_row_stride, const void* w,
                     const float* scale_w,
                     const int32_t* sorted_ids, const int32_t* sorted_expert_ids,
                     const float* sorted_weights, const int32_t* num_valid_ids, int num_tokens,
                     int inter_dim, int model_dim, int size_expert_ids, int experts, int topk,
                     int tile_m, int doweight, int out_dtype, int x_layout, int x_scale_layout,
                     int out_layout, int impl, void* stream);

/* Stage 2: down-projection grouped FP8 GEMM + top-k-weighted scatter-reduce.
 * Replaces kernels/moe_blockscale_2stage.py:1189-1207 (builder) and the launcher
 * :2335-2350.  a2 e4m3 [rows,I] under a_layout (BY_PAIR: row t*topk+s, fetched by index inside the
 * kernel as the reference does, :1576-1590; or SORTED);
 * scale_a f32 [I/128, sa_stride] indexed under a_scale_layout (BY_PAIR or SORTED).
 * w e4m3 [E,H,I], scale_w f32 [E,H/128,I/128].  accumulate!=0: out [T,H] of
 * out_dtype (F16/BF16/F32), pre-zeroed, receives atomic adds; accumulate==0: out
 * [T*k,H] rows t*k+s receive plain stores (F16/BF16 only). */
int flymoe_moe_gemm2(void* out, const void* a2, const float* scale_a, int64_t sa_stride,
                     const void* w, const float* scale_w, const int32_t* sorted_ids,
                     const int32_t* sorted_expert_ids, const float* sorted_weights,
                     const int32_t* num_valid_ids, int num_tokens, int model_dim, int inter_dim,
                     int size_expert_ids, int experts, int topk, int tile_m, int doweight,
                     int out_dtype, int accumulate, int a_layout, int a_scale_layout, int impl,
                     void* stream);

/* The two stages with ONE scale per activation row and ONE per weight row (output column)
 * instead of 128-wide blocks: the per-token / per-channel family.
 * Replace kernels/moe_gemm_2stage.py:90-108 (compile_moe_gemm1, launcher :1730-1745) and
 * :1780-1796 (compile_moe_gemm2, launcher :3151-3166) for in_dtype "fp8", "int8", "int8smooth",
 * "fp16" and "bf16".  in_dtype E4M3, I8 (signed 8-bit operands, exact int32 accumulation), or
 * F16 / BF16 (16-bit operands and weights, tcgen05 kernel only; their scale pointers may be null,
 * which means every scale is 1, as in the reference where these variants carry no scales).
 * Stage 1: x [T,H] (x_layout BY_TOKEN), [k*T,H] slot-major (BY_SLOT: "int8smooth"), [T*k,H] (BY_PAIR)
 * or rows already in sorted order (SORTED); scale_x f32 [T] (x_scale_layout BY_TOKEN), [k*T] (BY_SLOT), [T*k] (BY_PAIR)
 * or per sorted row; w [E,2I,H] row-major, scale_w f32 [E*2I]; out F16/BF16 [T*k,I]
 * (out_layout BY_PAIR) or sorted rows; or out_dtype F32 (tcgen05 kernel, BY_PAIR): the scaled gate and
 * up sums themselves are ADDED to out [T*k, 2I] (gate columns first), without activation or routing
 * weight -- the output contract of the reference's split-K launches (k_batch > 1,
 * kernels/moe_gemm_2stage.py:121-122), which finish SiLU(gate)*up outside the kernel.  Stage 2: a2 [T*k,I] / sorted rows, scale_a f32 [T*k] /
 * per sorted row, w [E,H,I], scale_w f32 [E*H]; out as flymoe_moe_gemm2.  The K range is
 * accumulated in TMEM and each tile is scaled once: out = (sum_k a*w) * scale_a[row] * scale_w[col].
 * scale_w must be 16-byte aligned. */
int flymoe_moe_gemm1_pertoken(void* out, const void* x, const float* scale_x, const void* w,
                              const float* scale_w, const int32_t* sorted_ids,
                              const int32_t* sorted_expert_ids, const float* sorted_weights,
                              const int32_t* num_valid_ids, int num_tokens, int inter_dim,
                              int model_dim, int size_expert_ids, int experts, int topk, int tile_m,
                              int doweight, int in_dtype, int out_dtype, int x_layout,
                              int x_scale_layout, int out_layout, int impl, void* stream);
int flymoe_moe_gemm2_pertoken(void* out, const void* a2, const float* scale_a, const void* w,
                              const float* scale_w, const int32_t* sorted_ids,
                              const int32_t* sorted_expert_ids, const float* sorted_weights,
                              const int32_t* num_valid_ids, int num_tokens, int model_dim,
                              int inter_dim, int size_expert_ids, int experts, int topk, int tile_m,
                              int doweight, int in_dtype, int out_dtype, int accumulate, int a_layout,
                              int a_scale_layout, int impl, void* stream);

/* Stage 2 with a caller-given destination per output row: row_dst[t*topk+s] is the byte
 * address the H out_dtype (F16/BF16) values of that (token, slot) row are stored to, 0 drops
 * the row.  Addresses must be 16-byte aligned (a misaligned one drops the row and sets the
 * device status word to FLYMOE_STATUS_ROW_DST_MISALIGNED) and may lie in another GPU's memory that is
 * mapped into this process with peer access: in the expert-parallel layer each rank
 * stores its expert outputs straight into the buffers of the ranks that own the tokens, so
 * the combine transfer rides on stage 2's epilogue instead of a separate all-to-all.
 * No accumulation, no routing weight unless doweight; tensor-core kernel only.  The
 * reference has no counterpart (it has no dispatch/combine; its stage 2 writes out[t] or
 * out[t*k+s], kernels/moe_blockscale_2stage.py:2335-2350). */
int flymoe_moe_gemm2_scatter_rows(const uint64_t* row_dst, const void* a2, const float* scale_a,
                                  int64_t sa_stride, const void* w, const float* scale_w,
                                  const int32_t* sorted_ids, const int32_t* sorted_expert_ids,
                                  const float* sorted_weights, const int32_t* num_valid_ids,
                                  int num_tokens, int model_dim, int inter_dim,
                                  int size_expert_ids, int experts, int topk, int tile_m,
                                  int doweight, int out_dtype, int a_layout, int a_scale_layout,
                                  void* stream);

/* Expert-parallel dispatch by direct stores.  For every (token, slot) row r of this rank's
 * expert-sorted order (sorted_ids / sorted_expert_ids of a unit-1 sort, one expert id per
 * row): the token's e4m3 row (model_dim bytes) is stored to dst_x[e] + r*model_dim and its
 * model_dim/128 fp32 scales (x_scale row-major [T, model_dim/128]) to
 * dst_scale[e] + r*(model_dim/128)*4, e being the row's expert.  The two tables hold one
 * byte address per expert, usually in the memory of the GPU that owns the expert (mapped
 * into this process, peer access enabled), chosen so that a row lands at its final position
 * of the receiver's block-padded sorted layout; dst_x addresses must be 16-byte aligned (rows of an
 * expert whose address is not are dropped and the status word reads FLYMOE_STATUS_ROW_DST_MISALIGNED).
 * Rows with ids outside [0, T) x [0, topk) or experts outside [0, experts) are skipped.
 * Optional bound for callers that size nothing on the host: with pos_base != NULL, row r
 * of expert e is dropped -- and the device status word set to 16
 * (flymoe_device_status) -- when pos_base[e] + r >= pos_limit, i.e. when it would fall
 * outside the receiver's buffer of pos_limit rows.
 * The reference has no counterpart (no dispatch/combine). */
int flymoe_dispatch_rows(const void* x, const float* x_scale, const int32_t* sorted_ids,
                         const int32_t* sorted_expert_ids, const int32_t* num_valid_ids,
                         const int64_t* dst_x, const int64_t* dst_scale, const int64_t* pos_base,
                         int64_t pos_limit, int num_tokens, int topk, int model_dim, int experts,
                         int max_rows, void* stream);

/* Expert-parallel step planning on the device (no reference counterpart: the reference has no
 * dispatch/combine).  flymoe_expert_counts: counts[e] = rows of the ascending per-row expert list
 * (the sorted_expert_ids of a unit-1 sort) that belong to expert e.  flymoe_ep_plan_direct: from the
 * rows-per-(rank, expert) matrix counts [world, experts] (every rank's flymoe_expert_counts,
 * all-gathered) it writes what rank `rank` needs for a step whose dispatch and combine are peer stores:
 * pos_base / dst_x / dst_scale [experts] for flymoe_dispatch_rows (each rank's operand buffer holds its
 * local experts in ascending order, every expert padded to a multiple of `unit` rows, sources in rank
 * order inside an expert; peer_base[r] + off_x / off_scale is where rank r's operand rows / scales
 * start), and for the rows this rank receives: sorted_ids [cap_rows] (row index, or the pad id
 * (1<<24)|cap_rows), sorted_expert_ids [cap_rows/unit] (local expert of each row block), num_valid_ids
 * {extent, extent} and row_dst [cap_rows] (peer_base[source] + off_back + source_row * model_dim * 2,
 * 0 for pad rows) for flymoe_moe_gemm2_scatter_rows.  Rows beyond cap_rows are not planned; the
 * dispatch kernel drops them and reports FLYMOE_STATUS_DISPATCH_OVERFLOW.  world <= 8, experts <= 1024;
 * workspace: flymoe_ep_plan_workspace_elems(world, experts) int32. */
int flymoe_expert_counts(const int32_t* row_expert, const int32_t* num_valid_ids, int64_t* counts,
                         int experts, int max_rows, void* stream);
int64_t flymoe_ep_plan_workspace_elems(int world, int experts);
int flymoe_ep_plan_direct(const int64_t* counts, const int64_t* peer_base, int64_t off_x,
                          int64_t off_scale, int64_t off_back, int64_t* dst_x, int64_t* dst_scale,
                          int64_t* pos_base, int32_t* sorted_ids, int32_t* sorted_expert_ids,
                          int32_t* num_valid_ids, int64_t* row_dst, int32_t* workspace,
                          int64_t workspace_elems, int world, int rank, int experts, int unit,
                          int model_dim, int64_t cap_rows, void* stream);

/* Dense block-scaled FP8 GEMM  c[M,N] = (a . b^T) with per-1x128 activation scales and
 * per-128x128 weight scales -- the stage-2 kernel run with one expert and identity routing.
 * Replaces kernels/blockscale_preshuffle_gemm.py:32-45 (builder) and the launcher :865-901.
 * a e4m3 [M,K]; scale_a f32 [K/128, sa_stride] (the reference's transposed layout,
 * sa_stride >= M); b e4m3 [N,K] row-major; scale_b f32 [ceil(N/128), K/128]; c [M,N] of
 * out_dtype (F16/BF16).  K must be a multiple of 128, N a multiple of 64.
 * workspace: flymoe_blockscale_gemm_workspace_elems(M, tile_m) int32, rewritten by every
 * call (the routing arrays of the grouped kernel); tile_m 16/32/64/128. */
int64_t flymoe_blockscale_gemm_workspace_elems(int m, int tile_m);
int flymoe_blockscale_gemm(void* c, const void* a, const float* scale_a, int64_t sa_stride,
                           const void* b, const float* scale_b, int32_t* workspace,
                           int64_t workspace_elems, int m, int n, int k, int tile_m, int out_dtype,
                           void* stream);

/* Test hook for the bounded waits: launches one thread that waits, with the same bounded
 * wait every kernel of the library uses, on a barrier nobody arrives at.  After limit_ns
 * nanoseconds (at most 1e8) the wait gives up, the kernel returns normally and the device
 * status word reads FLYMOE_STATUS_SELFTEST_TIMEOUT once.  Nothing faults or hangs; the
 * context stays usable.  The reference spins without a bound
 * (kernels/custom_all_reduce_kernel.py:236-246) and has no counterpart. */
int flymoe_selftest_bounded_wait(int64_t limit_ns, void* stream);

/* Caps the persistent grid of the two GEMM stages at max_ctas CTAs (0 restores one CTA per SM).
 * Process-wide.  For callers that run communication kernels next to the GEMMs (the
 * expert-parallel layer); the reference has no counterpart (its grid is one CTA per tile,
 * kernels/moe_blockscale_2stage.py:1165-1183). */
int flymoe_set_gemm_cta_limit(int max_ctas);

/* Y[t,:] = sum_s w[t,s] * X[row(t,s),:] with fp32 accumulation; row(t,s) = t*k+s, or
 * row_index[t*k+s] when row_index is given (negative entries are skipped); optional u8
 * valid_mask [T,k] and optional f32 weights [T,k] (NULL = 1).
 * Replaces kernels/moe_blockscale_2stage.py:2383-2589. */
int flymoe_moe_reduce(const void* x, void* y, const uint8_t* valid_mask, const float* weights,
                      const int32_t* row_index, int num_tokens, int topk, int model_dim, int dtype,
                      void* stream);

/* inverse[t*k+s] = position r of pair (t,s) in sorted_ids[0, num_valid_ids[0]); pairs that
 * do not appear keep -1.  Used by the expert-parallel combine to read returned rows in
 * (token, slot) order; the reference has no dispatch/combine, so this has no counterpart
 * there beyond the packed-id format of kernels/moe_sorting_kernel.py:17-20. */
int flymoe_sorted_inverse(const int32_t* sorted_ids, const int32_t* num_valid_ids, int32_t* inverse,
                          int num_tokens, int topk, int max_rows, void* stream);

/* Per-row, per-128-column FP8 quantiser: x [R,K] F16/BF16/F32 -> q e4m3 [R,K] and
 * scale f32 stored transposed [K/128, scale_stride] (scale = amax/448, 0 -> 1).
 * Replaces the test-side quantiser tests/utils.py:29-73 as used at
 * tests/kernels/test_moe_blockscale.py:354-367. */
int flymoe_quant_act_1x128(const void* x, int x_dtype, void* q, float* scale, int64_t scale_stride,
                           int rows, int cols, void* stream);

/* Converts weights between the reference's 16x16 preshuffle order
 * (tests/utils.py:76-96; kernels/mfma_preshuffle_pipeline.py:168-225) and plain
 * row-major [E*N, K]; to_plain!=0 undoes the shuffle.  src != dst. */
int flymoe_shuffle_weight(const void* src, void* dst, int64_t rows, int cols, int to_plain,
                          void* stream);
/* The same for elements of elem_bytes (1 or 2) bytes: the reference's order keeps 16 bytes of one row
 * together, i.e. 16 one-byte or 8 two-byte elements (tests/utils.py:84), cols counts elements. */
int flymoe_shuffle_weight_elems(const void* src, void* dst, int64_t rows, int cols, int elem_bytes,
                                int to_plain, void* stream);

/* Unpacks the reference's packed-int4 weights (tests/kernels/test_moe_gemm.py:49-65: signed 4-bit
 * values of the 16x16-preshuffled one-byte layout, eight per four bytes, b_i = (v_{i+4} << 4) | v_i)
 * to row-major [rows, cols] I8 or BF16, which the per-token-scale stages take as their weight
 * operand ("int4": W4A8 with int8 activations; "int4_bf16": W4A16 with bf16 activations).
 * packed holds rows * cols / 2 bytes. */
int flymoe_unpack_int4_weight(const void* packed, void* dst, int64_t rows, int cols, int out_dtype,
                              void* stream);
/* The same with group-wise weight scales folded in (W4A16 with group_size 32,
 * kernels/moe_gemm_2stage.py:90-108 `group_size`; scale layout tests/utils.py:99-129): BF16 output
 * = bf16(value * scale[e][k/32][n]), rows = E * rows_per_expert.  group_scale is F32 [E, cols/32,
 * rows_per_expert] or BF16 [E, cols/64, rows_per_expert, 2]; null = no scaling. */
int flymoe_unpack_int4_weight_grouped(const void* packed, void* dst, int64_t rows, int cols, int out_dtype,
                                      const void* group_scale, int group_scale_dtype, int group_size,
                                      int rows_per_expert, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLYMOE_H_ */
