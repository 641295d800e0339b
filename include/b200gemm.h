/*
 * b200gemm -- C ABI of the B200 (sm_100a) grouped-GEMM / per-block-quantiser library.
 *
 * The reference project (DeepLink-org/Triton_Grouped_GEMM) has no C interface: its kernels
 * are Triton JIT functions launched from Python.  Each entry point below replaces the Triton
 * launch made by one reference Python function (cited per function, paths relative to the
 * reference's root); the Python package triton_grouped_gemm_b200 binds them with ctypes.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the comment says "host".
 *   - Every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream), never synchronises the host, and allocates nothing.
 *   - Return value: 0 = ok, negative = rejected on the host (B200GEMM_ERR_*);
 *     b200gemm_last_error() then holds a message (thread local).
 *   - Errors detected on the device (a bounded wait that ran out) are OR-ed into a
 *     per-device status word, read with b200gemm_device_status().
 *   - Group sizes always stay on the device; `sizes_is_i64` selects int64_t / int32_t.
 *   - dtype codes: 0 = bfloat16, 1 = float16.  fp8 format codes: 0 = e4m3, 1 = e5m2.
 */
#ifndef B200GEMM_H_
#define B200GEMM_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200GEMM_OK 0
#define B200GEMM_ERR_INVALID_ARGUMENT (-1)
#define B200GEMM_ERR_UNSUPPORTED (-2)
#define B200GEMM_ERR_CUDA (-3)
#define B200GEMM_ERR_DRIVER_ENTRY (-4)

/* bits of the device status word */
#define B200GEMM_DEV_TIMEOUT_PRODUCER 0x1u
#define B200GEMM_DEV_TIMEOUT_MMA 0x2u
#define B200GEMM_DEV_TIMEOUT_EPILOGUE 0x4u
#define B200GEMM_DEV_TIMEOUT_PROMOTE 0x8u
/* the group sizes of an M-grouped call added up to more rows than m_rows: the excess rows were
 * neither read nor written (the call computed the groups that fit) */
#define B200GEMM_DEV_BAD_GROUP_SIZE 0x10u
/* a row mover was given a rank, a destination row or a source row outside its buffers: that row
 * was skipped */
#define B200GEMM_DEV_BAD_ROW_INDEX 0x20u

/* ---- library services (no reference counterpart: the reference reports errors with Python
 *      assert / ValueError and lets a wedged kernel hang) -------------------------------- */
int b200gemm_version(void);
const char* b200gemm_last_error(void);
/* Waits for all work on the current device (cudaDeviceSynchronize, so kernels on non-blocking
 * streams are covered), then copies its status word to *out_status (host pointer).
 * clear != 0 resets it afterwards. */
int b200gemm_device_status(unsigned* out_status, int clear);
int b200gemm_sm_count(void);
/* Tuning override for the 16-bit M-grouped kernels: 0 = pick the tile width (64 / 128 / 256
 * output columns) from the problem size, otherwise force that width.  Process-wide. */
int b200gemm_set_block_n(int block_n);
/* Tuning override: the M-grouped kernels, and the K-grouped kernels when they run with a
 * workspace, exist in a single-CTA form (128-row tiles) and a CTA-pair form (two SMs share a
 * 256 x 256 tile).  -1 = choose by problem size, 0 = never use the pair form, 1 = use it
 * whenever it is implemented for the call.  Process-wide. */
int b200gemm_set_cta_pair(int mode);
/* Number of CTAs (2 per cluster) a persistent launch of the CTA-pair kernel keeps resident on
 * the current device; 0 if it cannot be determined. */
int b200gemm_cta_pair_grid(void);

/* ---- BF16 / FP16 grouped GEMMs ------------------------------------------------------- */

/* M-grouped GEMM: C[rows of g, :] = A[rows of g, :] * B_g, fp32 accumulate, one rounding.
 * Replaces _m_grouped_gemm_launch + m_grouped_gemm_b{K,N}major_kernel + the host metadata
 * build (gemm/BF16/m_grouped_gemm_TMA.py:73-268, 297-326, 329-432; sm_80 twin
 * gemm/BF16/m_grouped_gemm.py:43-292).
 *   A [m_rows, k] row-major, compact (no padding rows); C [m_rows, n] row-major.
 *   trans_b != 0: B [G, n, k];  trans_b == 0: B [G, k, n].
 *   sizes [G]: rows per group, sum <= m_rows.  The kernels enforce that bound themselves (the
 *   sizes live on the device, the host cannot check them without a synchronisation): a group
 *   that would run past row m_rows is cut off there, later groups get no rows, nothing at or
 *   beyond row m_rows of A, C or the row scales is touched, and B200GEMM_DEV_BAD_GROUP_SIZE is
 *   raised in the status word.  The same holds for every M-grouped entry point below.
 *   Requires k % 8 == 0, n % 8 == 0, 16-byte aligned base pointers.  num_sms <= 0 = all SMs. */
int b200gemm_m_grouped(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                       int num_groups, int64_t m_rows, int n, int k, int trans_b, int dtype, int num_sms,
                       void* stream);

/* Same product for the padded row layout of DeepGEMM's "contiguous" grouped GEMM, which the
 * reference reaches through gemm/deep_gemm_ops.py:24-57: A and C hold each group's rows
 * rounded up to a multiple of 128 (m_rows = sum of padded sizes); padding rows are neither
 * read for results nor written. */
int b200gemm_m_grouped_padded(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                              int num_groups, int64_t m_rows, int n, int k, int trans_b, int dtype, int num_sms,
                              void* stream);

/* Masked M-grouped GEMM: for each g, rows [g*expected_m, g*expected_m + masked_m[g]) of
 * out = same rows of lhs * rhs[g]^T; other rows of out are left untouched.
 * Replaces m_grouped_gemm_masked + m_grouped_gemm_masked_kernel
 * (gemm/BF16/m_grouped_gemm_masked_TMA.py:54-250).  lhs [G*expected_m, k], rhs [G, n, k]
 * (trans_b != 0) or [G, k, n], out [G*expected_m, n].  masked_m[g] is clamped to
 * [0, expected_m].  Runs on `stream` (the reference uses a private side stream). */
int b200gemm_m_grouped_masked(const void* lhs, const void* rhs, void* out, const void* masked_m,
                              int sizes_is_i64, int num_groups, int expected_m, int n, int k, int trans_b,
                              int dtype, int num_sms, void* stream);

/* K-grouped GEMM (expert weight gradient): C[g] = A[gs:ge, :]^T * B[gs:ge, :], fp32
 * accumulate, one rounding; an empty group yields zeros.  Replaces k_grouped_gemm +
 * k_grouped_gemm_kernel (gemm/BF16/k_grouped_gemm_TMA.py:71-294; sm_80 twin
 * gemm/BF16/k_grouped_gemm.py:62-216).
 *   A [k_total, m_dim], B [k_total, n_dim] row-major; C [G, m_dim, n_dim].
 *   Token ranges: group_start/group_end (int32 [G], both or neither) if given, else the
 *   running prefix of sizes [G].  Requires m_dim % 8 == 0, n_dim % 8 == 0.
 *   workspace: optional device scratch of b200gemm_k_grouped_workspace_bytes(G) bytes (contents
 *   need no initialisation).  With it, tiles are claimed dynamically, groups with the most
 *   tokens first (tile cost varies with the group's token count); NULL = fixed round-robin
 *   assignment.  Two calls that overlap on the GPU must not share one workspace. */
long long b200gemm_k_grouped_workspace_bytes(int num_groups);
int b200gemm_k_grouped(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                       const int* group_start, const int* group_end, int num_groups, int64_t k_total, int m_dim,
                       int n_dim, int dtype, void* workspace, int64_t workspace_bytes, int num_sms, void* stream);

/* The balanced K-grouped GEMM for callers that cannot supply device memory.  It has no
 * counterpart in the reference.  Written for hosts that may not allocate on the GPU: a runtime
 * that gave all of HBM to its own pools (a later cudaMalloc fails or is against its rules), or a
 * latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc implies,
 * reached from C where no framework allocator is at hand.  Same arguments and results as
 * b200gemm_k_grouped without the workspace pair: the scheduler's scratch is a fixed array inside
 * the library (12.5 KB held by every GPU that loads it, for the life of the process).
 *   - At most 1024 groups; more are rejected with B200GEMM_ERR_INVALID_ARGUMENT.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address (once, cached); make
 *     that first call before starting any stream capture on that device.
 *   - All calls on a device share the one array.  Nothing needs clearing between calls (each
 *     call rewrites what it reads), but two calls whose kernels overlap on the GPU - different
 *     streams, or different host threads - race on it and compute garbage: serialise them. */
int b200gemm_k_grouped_static_scratch(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                                      const int* group_start, const int* group_end, int num_groups, int64_t k_total,
                                      int m_dim, int n_dim, int dtype, int num_sms, void* stream);

/* ---- FP8 grouped GEMMs with per-row x per-channel scales ------------------------------- */

/* FP8 M-grouped GEMM: C[m, n] = (sum_k A[m,k] * B[g,n,k])_fp32 * a_scale[m] * b_scale[g*n_dim+n].
 * Replaces gmm_fp8_act_per_channel_w_per_expert + its Triton kernel
 * (gemm/FP8/m_grouped_gemm_channel_expert.py:64-198).  A [m_rows, k] fp8 (fmt_a), a_scale
 * [m_rows] fp32, B [G, n, k] fp8 (fmt_b), b_scale [G*n] fp32, C [m_rows, n] of out_dtype
 * (0 = bf16, 1 = fp16).  Requires k % 16 == 0, n % 8 == 0. */
int b200gemm_fp8_m_grouped_rowcol(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                                  const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int n, int k,
                                  int fmt_a, int fmt_b, int out_dtype, int num_sms, void* stream);

/* FP8 K-grouped GEMM: out[g, m, n] = (sum_{k in group g} X[m,k] * Y[n,k])_fp32 *
 * x_scale[g*m_dim+m] * y_scale[g*n_dim+n] -> bf16.  Replaces matmul + gemm_kernel_tma
 * (gemm/FP8/k_grouped_gemm_channel_expert.py:64-181).  X [m_dim, k_total], Y [n_dim, k_total]
 * fp8, K-major; the scales are group-major in memory; tokens_per_expert[g] must be a multiple
 * of 128 with zero-padded data, as in the reference.  out [G, m_dim, n_dim] bf16.  workspace: as for
 * b200gemm_k_grouped. */
int b200gemm_fp8_k_grouped_rowcol(const void* x, const float* x_scale, const void* y, const float* y_scale, void* out,
                                  const void* tokens_per_expert, int sizes_is_i64, int num_groups, int64_t k_total,
                                  int m_dim, int n_dim, int fmt_x, int fmt_y, void* workspace, int64_t workspace_bytes,
                                  int num_sms, void* stream);

/* ---- FP8 grouped GEMMs with 1x128 / 128x128 block scales -------------------------------- */

/* Block-scaled FP8 M-grouped GEMM:
 *   C[m,n] = sum_kb (sum_{k in kb} a[m,k] * b[g,n,k]) * a_scale[m,kb] * b_scale[g, n/128, kb] -> bf16.
 * The reference has no kernel of its own for this: gemm/deep_gemm_ops.py:60-100 forwards to the
 * external DeepGEMM package; this entry point takes over that call with fp32 scales as produced
 * by per_token_cast_to_fp8 / per_block_cast_to_fp8
 * (gemm/FP8/m_grouped_gemm_channel_expert.py:217-245).
 *   a [m_rows, k] e4m3, a_scale [m_rows, ceil(k/128)] fp32 (row-major);
 *   b [G, n, k] e4m3, b_scale [G, ceil(n/128), ceil(k/128)] fp32; c [m_rows, n] bf16.
 *   rows_padded == 0: a / c rows are compact; != 0: each group's rows are padded to 128 (the
 *   layout gemm/deep_gemm_ops.py:87-89 requires).  Requires k % 16 == 0, n % 8 == 0. */
int b200gemm_fp8_m_grouped_block(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                                 const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int n, int k,
                                 int rows_padded, int num_sms, void* stream);

/* Same GEMM with an indirection from row groups to weight matrices: group g (its
 * size_per_group[g] rows, compact) is multiplied by b[group_to_b[g]], b holding num_b matrices.
 * An expert-parallel layer uses it to consume rows in the order an all-to-all delivers them
 * ([source rank][local expert] blocks, each its own group) without permuting them into
 * expert-major order first.  group_to_b: int32 [num_groups] on the device, values in
 * [0, num_b) (clamped).  No counterpart in the reference (it has no multi-GPU path). */
int b200gemm_fp8_m_grouped_block_mapped(const void* a, const float* a_scale, const void* b, const float* b_scale,
                                        void* c, const void* sizes, int sizes_is_i64, int num_groups,
                                        const int* group_to_b, int num_b, int64_t m_rows, int n, int k, int num_sms,
                                        void* stream);

/* Gate+up projection of a SwiGLU feed-forward with the activation and its 1x128 quantisation in
 * the epilogue.  b [num_b or G, n, k] holds gate and up weight rows interleaved in 128-row blocks
 * (rows [256 t, 256 t + 128) = gate rows [128 t, +128), rows [256 t + 128, +128) = up rows
 * [128 t, +128)), b_scale likewise; n = 2 x intermediate size, a multiple of 256.  Writes
 * act [m_rows, n/2] e4m3 = quantised bf16(silu(bf16(gate)) * bf16(up)) and act_scale [m_rows, n/256]
 * fp32: bit for bit what b200gemm_fp8_m_grouped_block followed by b200quant_swiglu_act_1x128
 * produce from the un-interleaved weights, without storing the bf16 product.  group_to_b may be
 * NULL (group g uses b[g]); masked_stride > 0 selects the masked row layout (rows g*stride ...),
 * 0 the compact one.  No counterpart in the reference. */
int b200gemm_fp8_m_grouped_block_swiglu(const void* a, const float* a_scale, const void* b, const float* b_scale,
                                        void* act, float* act_scale, const void* sizes, int sizes_is_i64,
                                        int num_groups, const int* group_to_b, int num_b, int64_t m_rows,
                                        int masked_stride, int n, int k, int num_sms, void* stream);

/* Masked-layout twin (decode): rows [g*expected_m, g*expected_m + masked_m[g]) of out.  No
 * reference counterpart as a kernel; it combines the masked layout of
 * gemm/BF16/m_grouped_gemm_masked_TMA.py:164-250 with the block-scaled contract above. */
int b200gemm_fp8_m_grouped_masked_block(const void* a, const float* a_scale, const void* b, const float* b_scale,
                                        void* out, const void* masked_m, int sizes_is_i64, int num_groups,
                                        int expected_m, int n, int k, int num_sms, void* stream);

/* Block-scaled FP8 K-grouped GEMM: the expert weight gradient from two outputs of the transposing
 * 128x128 quantiser (b200quant_trans_expand_128x below).
 *   out[g, m, n] = sum_{kb in group g} (sum_{t in kb} x8[m,t] * y8[n,t]) * x_scale[m/128, kb] * y_scale[n/128, kb] -> bf16
 *   x8 [m_dim, m_expand], y8 [n_dim, m_expand] e4m3 (tokens along the inner axis, each expert's
 *   tokens padded to a multiple of 128); x_scale [m_dim/128, m_expand/128], y_scale
 *   [n_dim/128, m_expand/128] fp32; padded_sizes [G]: padded token count of each expert (the
 *   quantiser's third output), k-blocks of group g = the running prefix / 128; out [G, m_dim, n_dim]
 *   bf16, an expert without tokens gives zeros.  m_dim, n_dim, m_expand multiples of 128.
 *   workspace: optional device scratch of b200gemm_k_grouped_workspace_bytes(G) bytes (contents need
 *   no initialisation); with it the tiles are handed out in order of falling token count, which
 *   balances the CTAs when the experts' token counts differ; NULL = tiles in expert order.
 * The reference ships the quantiser that produces this layout
 * (quant/trans_per_block_quant_expand_128x.py:135-208) but no kernel that consumes it; the
 * skeleton (K-major operands, 128-token blocks, tile -> (group, m tile, n tile)) is that of its
 * per-channel kernel gemm/FP8/k_grouped_gemm_channel_expert.py:64-140. */
int b200gemm_fp8_k_grouped_block(const void* x8, const float* x_scale, const void* y8, const float* y_scale, void* out,
                                 const void* padded_sizes, int sizes_is_i64, int num_groups, int64_t m_expand,
                                 int m_dim, int n_dim, void* workspace, int64_t workspace_bytes, int num_sms,
                                 void* stream);

/* ---- per-block FP8 (e4m3) quantisers: bytes and fp32 scales identical to the reference's
 *      torch functions ------------------------------------------------------------------ */

/* 1x128 activation quantiser.  Replaces per_token_cast_to_fp8
 * (gemm/FP8/m_grouped_gemm_channel_expert.py:217-222).  x [rows, k] 16-bit, k % 128 == 0;
 * q [rows, k] bytes; scales [rows, k/128] fp32. */
int b200quant_act_1x128(const void* x, void* q, float* scales, int64_t rows, int64_t k, int dtype, void* stream);

/* SwiGLU fused with the 1x128 quantiser, for the step between an expert's gate+up and down
 * GEMMs: h [rows, 2*inter] bf16 (gate | up) -> act = bf16(silu(gate) * up), quantised as by
 * b200quant_act_1x128.  q [rows, inter] bytes, scales [rows, inter/128].  The reference keeps
 * this as separate torch steps (README.md:175-179); fusing it saves one HBM round trip of act. */
int b200quant_swiglu_act_1x128(const void* h, void* q, float* scales, int64_t rows, int64_t inter, void* stream);

/* 128x128 weight quantiser, batched over experts.  Replaces per_block_cast_to_fp8
 * (gemm/FP8/m_grouped_gemm_channel_expert.py:237-245) applied to each x[e].
 * x [batch, rows, cols] 16-bit; q same shape, bytes; scales [batch, ceil(rows/128),
 * ceil(cols/128)] fp32. */
int b200quant_w_128x128(const void* x, void* q, float* scales, int64_t batch, int rows, int cols, int dtype,
                        void* stream);

/* Transposing 128x128 quantiser with per-expert expansion.  Replaces
 * trans_per_block_quant_expand_128x + its Triton kernel
 * (quant/trans_per_block_quant_expand_128x.py:42-208); results equal the torch function
 * per_block_trans_quant_expand_torch (same file :253-273).
 * x [m_rows, n] 16-bit (n % 128 == 0), sizes [G] rows per expert;
 * q [n, m_expand] bytes, scales [n/128, m_expand/128] fp32, padded_sizes_out [G] int64
 * (may be NULL).  m_expand = m_rows + 128*G - m_rows % 128 (computed by the caller). */
int b200quant_trans_expand_128x(const void* x, const void* sizes, int sizes_is_i64, int num_groups, void* q,
                                float* scales, int64_t* padded_sizes_out, int64_t m_rows, int n, int64_t m_expand,
                                int dtype, void* stream);

/* ---- row movement around the expert GEMMs (expert-parallel MoE layer) --------------------- */

/* dst[i, :] = src[idx[i], :] for i < rows (rows of row_bytes bytes, a multiple of 16; idx int64).
 * The dispatch-side gather into expert-major order; the reference has this only in its vendored
 * baseline extension (grouped_gemm/csrc/permute.cu:40-297, moe_permute_topK_kernel).  src holds
 * src_rows rows: an index outside [0, src_rows) (such as the -1 of a rejected routing pair) is
 * skipped - dst[i] keeps its contents - and B200GEMM_DEV_BAD_ROW_INDEX is raised. */
int b200moe_gather_rows(const void* src, const int64_t* idx, void* dst, int64_t rows, int64_t row_bytes,
                        int64_t src_rows, void* stream);

/* out[t, :] = bf16(sum_k weights[t,k] * y[pos[t,k], :]), fp32 accumulation: the combine-side
 * weighted sum of a token's top-k expert outputs (baseline counterpart:
 * grouped_gemm/csrc/permute.cu, moe_recover_topK_kernel).  y [y_rows, hidden], out bf16.  A pos
 * outside [0, y_rows) contributes nothing and raises B200GEMM_DEV_BAD_ROW_INDEX. */
int b200moe_combine_topk(const void* y, const int64_t* pos, const float* weights, void* out, int64_t tokens, int top_k,
                         int hidden, int64_t y_rows, void* stream);

/* Routing plan of an MoE step: counting sort of the (token, k) pairs by expert.
 * expert int64 [n] with values in [0, num_experts), num_experts <= 1024.  counts int32 [E]: pairs
 * per expert; cursor int32 [E]: scratch (ends as the END of each expert's range); order int64 [n]:
 * pair indices grouped by expert (expert e's pairs at [sum(counts[:e]), +counts[e]), order inside
 * a range unspecified); pos int64 [n] = order^-1.  A pair whose expert id lies outside the range
 * (a dropped token's -1) is counted nowhere, raises B200GEMM_DEV_BAD_ROW_INDEX, gets pos = -1,
 * and leaves one slot at the end of order at -1; the row movers skip such indices.  The role of
 * the sort in the vendored baseline's permute (grouped_gemm/csrc/permute.cu:504-690), without a
 * comparison sort. */
int b200moe_route_plan(const int64_t* expert, int64_t n, int num_experts, int* counts, int* cursor, int64_t* order,
                       int64_t* pos, void* stream);

/* The same counting sort on a permutation of the expert ids: the sort key of expert e is
 * key_table[e] (int64 [num_experts], a permutation of 0 .. num_experts-1), counts / cursor / order
 * are in key order.  An expert-parallel layer uses it to send its pairs chunk by chunk.
 * No counterpart in the reference. */
int b200moe_route_plan_mapped(const int64_t* expert, int64_t n, int num_experts, const int64_t* key_table, int* counts,
                              int* cursor, int64_t* order, int64_t* pos, void* stream);

/* Plan of the peer-memory exchange, on the device (no counterpart in the reference).  Given the
 * all-gathered pair counts of every rank in key order (counts_all int32 [world, num_experts]), the
 * permutation in both directions (expert_of_key int32, key_of_expert int64) and this rank's send
 * order (order, from b200moe_route_plan_mapped) over its routing (expert int64 [n], n = tokens *
 * top_k), it writes for the buffers laid out [local expert][source rank] on every rank:
 *   dst_start / send_start int64 [num_experts] (scratch: first row of this rank's pairs of a key in
 *   the owner's buffers / first position of the key in this rank's send order),
 *   size_per_group int64 [num_experts / world]: rows of each local expert here,
 *   token_of_pair int64 [n], dst_rank int32 [n], dst_row int64 [n]: per position of the send order
 *   (-1 for a slot of a rejected pair). */
int b200moe_peer_plan(const int* counts_all, const int* expert_of_key, const int64_t* key_of_expert, int world, int me,
                      int num_experts, const int64_t* order, const int64_t* expert, int64_t n, int top_k,
                      int64_t* dst_start, int64_t* send_start, int64_t* size_per_group, int64_t* token_of_pair,
                      int* dst_rank, int64_t* dst_row, void* stream);

/* The same row movers over the buffers of several ranks (peer memory mapped into this process):
 * dst_bases[dst_rank[i]][dst_row[i], :] = src[src_idx[i], :], and
 * out[t, :] = bf16(sum_k weights[t,k] * src_bases[pair_rank[t,k]][pair_row[t,k], :]).
 * dst_bases / src_bases: HOST arrays of `world` (<= 16) device pointers, each buffer holding
 * capacity_rows rows; src holds src_rows rows.  Ranks, destination rows and source rows are
 * bounds-checked on the device (a bad index raises B200GEMM_DEV_BAD_ROW_INDEX and is skipped).
 * They replace the all-to-alls of an expert-parallel layer: the caller synchronises the ranks
 * between writing and reading (e.g. a barrier collective).
 * blocks > 0: the mover runs as that many 1024-thread blocks (one per SM at most) instead of
 * filling the GPU, for running beside a persistent GEMM that was given the other SMs (num_sms);
 * <= 0: fill the GPU.  No counterpart in the reference. */
int b200moe_scatter_rows_multi(const void* src, const int64_t* src_idx, void* const* dst_bases, const int* dst_rank,
                               const int64_t* dst_row, int64_t rows, int64_t row_bytes, int world,
                               int64_t capacity_rows, int64_t src_rows, int blocks, void* stream);
int b200moe_combine_topk_multi(const void* const* src_bases, const int* pair_rank, const int64_t* pair_row,
                               const float* weights, void* out, int64_t tokens, int top_k, int hidden, int world,
                               int64_t capacity_rows, void* stream);

/* Quantise-on-dispatch.  For the pairs i in [first_pair, first_pair + num_pairs) of a step's send
 * order: the 16-bit row x[token_of_pair[i], :] (x [tokens, hidden], hidden % 128 == 0, <= 8192) is
 * quantised 1x128 - bytes and scales identical to b200quant_act_1x128 - and stored at row
 * dst_row[i] of rank dst_rank[i]: the e4m3 row into row_bases (hidden bytes per row), its
 * hidden/128 fp32 scales into scale_bases, and the pair's return address (int64 i, int64
 * my_rank) into meta_bases (16 bytes per row).  One kernel instead of the activation quantiser
 * plus one scatter per payload, and the fp8 copy of x never goes through HBM.  Bounds checks and
 * `blocks` as above.  No counterpart in the reference. */
int b200moe_dispatch_quant_rows_multi(const void* x, const int64_t* token_of_pair, void* const* row_bases,
                                      void* const* scale_bases, void* const* meta_bases, const int* dst_rank,
                                      const int64_t* dst_row, int64_t first_pair, int64_t num_pairs, int64_t tokens,
                                      int hidden, int dtype, int world, int64_t capacity_rows, int my_rank, int blocks,
                                      void* stream);
/* Quantise-and-permute on one GPU: row t of x [tokens, hidden] (bf16 / fp16, hidden % 128 == 0,
 * <= 8192) is quantised 1x128 once - bytes and scales identical to b200quant_act_1x128 - and
 * written to row pos[t * top_k + j] of dst8 [dst_rows, hidden] (e4m3 bytes) and dst_scales
 * [dst_rows, hidden/128] for every j < top_k: the activation quantiser and the token permute
 * (baseline counterpart of the latter: grouped_gemm/csrc/permute.cu, moe_permute_topK_kernel) in
 * one pass.  A pos outside [0, dst_rows) - the -1 of a rejected pair - is skipped and raises
 * B200GEMM_DEV_BAD_ROW_INDEX.  No counterpart in the reference's Triton path. */
int b200moe_quant_scatter_rows(const void* x, int dtype, int64_t tokens, int hidden, const int64_t* pos, int top_k,
                               void* dst8, float* dst_scales, int64_t dst_rows, void* stream);
/* The same dispatch for rows that are already quantised: x8 [tokens, hidden] e4m3 bytes and
 * x_scales [tokens, hidden/128] fp32 (as b200quant_act_1x128 writes them) are copied to the
 * pair's row of the owner's buffers together with the return address - one launch per chunk
 * instead of one scatter per payload.  Cheaper than quantising per pair when few SMs run the
 * mover beside a GEMM (a token's row is quantised once, not once per expert it goes to).
 * No counterpart in the reference. */
int b200moe_dispatch_rows_multi(const void* x8, const float* x_scales, const int64_t* token_of_pair,
                                void* const* row_bases, void* const* scale_bases, void* const* meta_bases,
                                const int* dst_rank, const int64_t* dst_row, int64_t first_pair, int64_t num_pairs,
                                int64_t tokens, int hidden, int world, int64_t capacity_rows, int my_rank, int blocks,
                                void* stream);
/* The way back: dst_bases[meta[r][1]][meta[r][0], :] = src[r, :] for r < rows, meta [rows, 2] int64
 * being the return addresses left by b200moe_dispatch_quant_rows_multi beside the rows
 * (capacity_rows = rows of each return buffer).  No counterpart in the reference. */
int b200moe_return_rows_multi(const void* src, const int64_t* meta, void* const* dst_bases, int64_t rows,
                              int64_t row_bytes, int world, int64_t capacity_rows, int blocks, void* stream);

/* Buffers other processes of the node can address, for the peer-memory row movers above.
 * alloc: cudaMalloc on the current device, zero-filled.  export: 64-byte CUDA IPC handle of a
 * buffer from alloc.  open: maps another process's buffer for the CURRENT device of the calling
 * process (peer access to the owning device is enabled); the returned pointer is valid in kernels
 * of that device.  close / free undo open / alloc.  No counterpart in the reference. */
int b200ipc_alloc(int64_t bytes, void** out);
int b200ipc_free(void* p);
int b200ipc_export(const void* p, void* handle64);
int b200ipc_open(const void* handle64, void** out);
int b200ipc_close(void* p);
/* n contiguous device-to-device copies queued on `stream`, each its own copy-engine transfer
 * (dst / src / bytes: HOST arrays of n entries; either side may be a buffer from b200ipc_open).
 * An expert-parallel layer returns each (expert, source rank) block of results with one such
 * copy: contiguous on both sides, so no kernel and no SM is needed for the way back.
 * No counterpart in the reference. */
int b200ipc_copy_many_async(int n, void* const* dst, const void* const* src, const int64_t* bytes, void* stream);

/* ---- integer layouts on the device ------------------------------------------------------- */

/* gemm/layout.py:61-71 make_group_starts: exclusive prefix of the group sizes (padded != 0: of the
 * sizes rounded up to block_m).  sizes int32/int64 [num_groups] on the device -> out int32. */
int b200layout_group_starts(const void* sizes, int sizes_is_i64, int num_groups, int padded, int block_m, int* out,
                            void* stream);
/* gemm/layout.py:100-120 make_deep_gemm_psum_layout: per group the end offset of its real rows in
 * padded-row coordinates. */
int b200layout_psum(const void* sizes, int sizes_is_i64, int num_groups, int block_m, int* out, void* stream);
/* gemm/layout.py:73-98 make_deep_gemm_grouped_layout: one int32 per padded row, the group id on
 * real rows and -1 on padding rows.  out holds total_padded_rows entries (the caller computes
 * that sum; rows beyond it are not written). */
int b200layout_grouped_rows(const void* sizes, int sizes_is_i64, int num_groups, int block_m, int* out,
                            int64_t total_padded_rows, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* B200GEMM_H_ */
