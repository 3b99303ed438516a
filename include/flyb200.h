/* C ABI of libflyb200: the B200 (sm_100a) implementation of the quantised
 * A8W8 "preshuffle" GEMM operator of ROCm/FlyDSL.
 *
 * Every entry point takes plain pointers and sizes, launches asynchronously on
 * the given CUDA stream (a cudaStream_t passed as void*; NULL = default stream),
 * allocates nothing and never synchronises, so calls can be captured into a CUDA
 * graph.  All pointers are device pointers on the current device unless stated
 * otherwise.  Return value: 0 on success, else one of the FLYB200_E_* codes
 * (flyb200_strerror() gives text).  Reference citations below are paths inside
 * the FlyDSL project.
 */
#ifndef FLYB200_H_
#define FLYB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define FLYB200_OK 0
#define FLYB200_E_BAD_ARG 1     /* inconsistent sizes, null pointers, unknown enum */
#define FLYB200_E_BAD_ALIGN 2   /* a pointer is not 16-byte aligned */
#define FLYB200_E_CUDA 3        /* a CUDA runtime/driver call failed (see flyb200_last_cuda_error) */
#define FLYB200_E_TIMEOUT 4     /* a bounded device-side wait expired (read via flyb200_read_status) */
#define FLYB200_E_UNSUPPORTED 5 /* shape or dtype outside what the kernels cover */
#define FLYB200_E_SMEM_ALIGN 6  /* device reported misaligned shared memory (read via flyb200_read_status) */
#define FLYB200_E_WORKSPACE 7   /* workspace missing or too small for the requested split */
#define FLYB200_E_SCRATCH_LIMIT 8 /* flyb200_gemm_a8w8_static_scratch: needs more than the built-in array */

/* in_dtype: element type of A and of the preshuffled weights
 * (compile_preshuffle_gemm(in_dtype=...), kernels/gemm/preshuffle_gemm.py:117,129-130) */
#define FLYB200_DT_FP8 0  /* float8 e4m3fn */
#define FLYB200_DT_INT8 1
#define FLYB200_DT_FP16 2
#define FLYB200_DT_BF16 3

/* out_dtype (kernels/gemm/preshuffle_gemm.py:118,168) */
#define FLYB200_OUT_BF16 0
#define FLYB200_OUT_FP16 1

/* epilogue (kernels/gemm/preshuffle_gemm.py:119,133-134,672-692) */
#define FLYB200_EPI_NONE 0
#define FLYB200_EPI_BIAS 1
#define FLYB200_EPI_BIAS_RELU 2
#define FLYB200_EPI_BIAS_SILU 3
#define FLYB200_EPI_BIAS_GELU 4

/* source layouts accepted by flyb200_shuffle_weight */
#define FLYB200_SRC_ROW_MAJOR 0 /* plain [N, K] */
#define FLYB200_SRC_MFMA_16x16 1 /* already permuted by the reference's shuffle_weight(layout=(16,16)) */

/* variant_hint: 0 = choose automatically.  Otherwise a bit field used for
 * tuning sweeps (each field: 0 = automatic):
 *   bits 0-7   small-M kernel: split-K factor; large-M kernel (one CTA per
 *              tile, kernels 2 and 6): tile width in units of 32 output channels
 *              (1..8, i.e. 128 x 32 ... 128 x 256 tiles; 256 rows for kernel 6).  Automatic for the large-M kernel:
 *              the width whose tiles fill the SMs in the fewest, fullest rounds.
 *   bits 8-11  kernel: 1 = small-M weight-stationary kernel (M <= 1024: up to 256
 *              tokens per CTA, more as token blocks of 256 in grid.z),
 *              2 = large-M persistent kernel, one CTA per 128 x (32..256) tile,
 *              3 = large-M persistent kernel, CTA pairs on 256x256 tiles
 *              4 = small-M kernel with 64-channel weight tiles and no K split
 *              (M <= 64 per token block; twice the CTAs, no reduction step)
 *              5 = small-M kernel as CTA pairs (tcgen05 cta_group::2: 256 channels
 *              per pair, each CTA stages half of the token tile; token tiles of
 *              64..256, an even number of 128-channel tiles, K splits <= 4 inside
 *              the pair's cluster)
 *              6 = large-M persistent kernel, one CTA per 256 x (32..256) tile (two
 *              accumulators that share every weight block; three-stage ring)
 *              (automatic: M <= 256 -> 1 [5 when FLYB200_DECODE_PAIR=1 and the shape
 *              allows it; 4 when FLYB200_DECODE_W64=1 and the N/64 tiles fill
 *              75-100 % of the SMs], except for outputs so wide that the small-M
 *              kernel would run in several rounds of CTAs: with S SMs and
 *              T = ceil(N/128) > S, M > 64, or M >= 32 when the rounds are less than
 *              70 % full, or M > 16 (M = 16 with K >= 8192 bytes) when T >= 3 S, go to 2;
 *              256 < M <= 1024 -> 1 when 2 * T * ceil(M/256) <= S and K spans at
 *              least 32 blocks of 128 bytes; else M > 256 -> 2, or 3 when FLYB200_ROWS_2SM=1, or 6
 *              when FLYB200_ROWS_TALL=1 or when ceil(M/256) * ceil(N/256) tiles
 *              cover the output in one round that fills at least 80 % of the SMs)
 *   bits 12-15 how K splits are combined: 1 = global workspace + ticket,
 *              2 = thread-block cluster + distributed shared memory (split <= 8)
 *   bits 16-23 rasterisation group (row tiles per group, large-M kernel)
 *   bits 24-27 depth of the shared-memory ring of the small-M kernel (an odd
 *              depth becomes the next even one, or the one below when that
 *              does not fit into shared memory)
 *   bits 28-29 programmatic dependent launch (small-M kernel; large-M kernels when
 *              the launch has at most two rounds of tiles): 1 = on (its
 *              set-up overlaps the tail of the previous kernel on the stream; no
 *              global memory is touched before that kernel has completed),
 *              3 = on, and additionally the first weight loads are issued before
 *              the previous kernel has completed (only valid when no kernel on
 *              the stream writes the weights), 2 = off.  Automatic: the first
 *              form, unless the environment variable FLYB200_PDL says 0 (off)
 *              or 2 (the second form).
 *   bits 30-31 token blocks of the small-M kernel (CTAs per channel tile that
 *              each take a block of the tokens over the whole K range; no
 *              reduction step, but every weight block is fetched once per token
 *              block): 1 = one block, 2 = two, 3 = four.  Automatic: one. */

/* The GEMM: c[M,N] = epilogue((a[M,K] . w[N,K]^T) * scale_a[m] * scale_b[n]).
 * Replaces the launcher returned by compile_preshuffle_gemm and the kernel
 * behind it (kernels/gemm/preshuffle_gemm.py:717-806 launch_gemm,
 * :220-714 kernel_gemm; call convention pinned by
 * tests/kernels/test_preshuffle_gemm.py:240-256).
 *   c        [>=M, N] row-major, out_dtype; rows >= M are never written
 *   a        [M, K] row-major, in_dtype
 *   w_shuf   weights [N, K] in the layout written by flyb200_shuffle_weight
 *   scale_a  [M] fp32 per-token scale, scale_b [N] fp32 per-channel scale; both
 *            NULL for FP16/BF16 inputs (no scaling)
 *   bias     [N] in out_dtype; NULL when epilogue == FLYB200_EPI_NONE
 *   workspace/workspace_bytes  scratch for the split-K variant that reduces
 *            through global memory, sized by flyb200_workspace_bytes(); its
 *            first 16 KiB must be zero before the first use and are left zero by
 *            every completed call; may be NULL (the automatic choice then keeps
 *            partial sums on chip).  Two calls that overlap on the GPU must not
 *            share a workspace.  A call whose kernel gave up on a bounded wait
 *            (flyb200_read_status() != 0) may leave counters non-zero: zero the
 *            first 16 KiB again before the workspace is reused.
 * Requirements: N % 16 == 0, K * elem_bytes % 128 == 0, pointers 16-byte aligned. */
int flyb200_gemm_a8w8(void* c, const void* a, const void* w_shuf, const float* scale_a, const float* scale_b,
                      const void* bias, int M, int N, int K, int in_dtype, int out_dtype, int epilogue,
                      int variant_hint, void* workspace, size_t workspace_bytes, void* stream);

/* Raw 32-bit accumulators acc[M,N] (int32 for INT8, fp32 bit patterns for FP8)
 * before any scaling: what the reference holds in its MFMA accumulators at
 * kernels/gemm/preshuffle_gemm.py:538,699-702.  Used to prove the INT8 path
 * bit-exact.  Same kernels, same dispatch as flyb200_gemm_a8w8. */
int flyb200_gemm_a8w8_acc(void* acc, const void* a, const void* w_shuf, int M, int N, int K, int in_dtype,
                          int variant_hint, void* workspace, size_t workspace_bytes, void* stream);

/* The small-M GEMM (M <= 256) for callers that cannot hand the library a
 * workspace because they are not able to allocate device memory at the point
 * of the call: a plug-in running inside a host application that has already
 * claimed the device's memory for its own pool, code on a latency-critical
 * path where cudaMalloc's implicit device-wide synchronisation is not
 * acceptable, or a component whose allocator simply is not reachable from
 * where the GEMM is issued.  It has no counterpart in the reference.
 *
 * Same arguments and result as flyb200_gemm_a8w8, except that the split-K
 * partial sums go to an 8 MiB array that is part of the library's device image
 * (flyb200_static_scratch_bytes(); every GPU that has loaded the library holds
 * it until the process exits).  The call itself performs no cudaMalloc/cudaFree
 * and uses no allocating library routine.
 *   split_k  number of K splits, 0 = choose automatically (the largest useful
 *            factor whose partial sums fit).  An explicit factor whose partial
 *            sums (split_k * ceil(N/128) * BN * 512 bytes, BN = M rounded up
 *            to 16/32/64/128/256, plus 16 KiB of counters) exceed the array is
 *            rejected with FLYB200_E_SCRATCH_LIMIT; nothing is launched.
 * The first call on each device looks up the array's device address; make that
 * first call with the device current and before starting any stream capture.
 * All calls on a device share the one array, which keeps the previous call's
 * contents: the counters that must start at zero are cleared on `stream` before
 * the kernel runs, and two calls that may overlap on the GPU (different
 * streams, or different host threads on the same device) race on it and must
 * be serialised by the caller. */
int flyb200_gemm_a8w8_static_scratch(void* c, const void* a, const void* w_shuf, const float* scale_a,
                                     const float* scale_b, const void* bias, int M, int N, int K, int in_dtype,
                                     int out_dtype, int epilogue, int split_k, void* stream);
size_t flyb200_static_scratch_bytes(void);

/* The large-M GEMM with its output tiles stored into the same window of several
 * buffers at once: window = columns [c_col_offset, c_col_offset + N) of row-major
 * matrices with c_pitch elements per row.  This is the column-parallel form of
 * the operator fused with the all-gather of its output shards: rank r of a group
 * of n_bufs GPUs passes the (peer-mapped) full-width output buffers of all ranks
 * and c_col_offset = r * N, and every 128 x 256 tile leaves the kernel through
 * TMA stores to each buffer, so the transfer over NVLink overlaps the math tile
 * by tile.  Plain per-CTA stores; no multicast, no loads from peer memory.  The
 * reference has no multi-GPU form of this operator (its only matching
 * collective is the all_gather_into_tensor fallback of
 * kernels/comm/custom_all_reduce.py:929-938).
 *   c_bufs     host array of n_bufs (1..8) device pointers, each 16-byte aligned
 *              and writable from the current device
 *   first_buf  index of the buffer stored to first (use the caller's rank)
 *   c_pitch, c_col_offset  in elements; both multiples of 8
 * The caller orders the kernel against readers on other GPUs (a barrier across
 * the group after the call) and against the next overwrite of the buffers. */
int flyb200_gemm_a8w8_scatter(void* const* c_bufs, int n_bufs, int first_buf, long long c_pitch, long long c_col_offset,
                              const void* a, const void* w_shuf, const float* scale_a, const float* scale_b,
                              const void* bias, int M, int N, int K, int in_dtype, int out_dtype, int epilogue,
                              int variant_hint, void* stream);

/* Weight preshuffle: dst = B200 image of the [N, K] matrix src.  Replaces
 * shuffle_weight (tests/utils.py:76-96) and the layout it encodes
 * (kernels/gemm/preshuffle_gemm.py:765-780).  dst and src must not overlap;
 * both hold N*K*elem_bytes bytes.  Image: [K*elem_bytes/128][N][128 bytes] with
 * the 16-byte chunks of each row XOR-ed by (row % 8). */
int flyb200_shuffle_weight(void* dst, const void* src, int N, int K, int elem_bytes, int src_layout, void* stream);

/* Inverse of flyb200_shuffle_weight: row-major [N, K] from the B200 image. */
int flyb200_unshuffle_weight(void* dst, const void* src, int N, int K, int elem_bytes, void* stream);

/* Per-token quantiser on the GPU: y[rows, K] (fp8 e4m3fn or int8) and
 * scale[rows] (fp32) from x[rows, K] (x_dtype: 0 = fp32, 1 = fp16, 2 = bf16).
 * Same arithmetic, bit for bit, as pertoken_quant (tests/utils.py:29-73)
 * evaluated by torch on a GPU: scale = rowmax|x| * (1/qmax) with 0 -> 1 (qmax
 * 448 / 127), y = x / scale converted with round-to-nearest-even (fp8) or
 * truncation toward zero (int8), NaN -> 0 and +-Inf -> +-qmax beforehand.  The
 * reference's own device kernel for this step is tests/kernels/test_quant.py:82-275.
 * Requirements: K a multiple of 4 (fp32) or 8 (16-bit input), x 16-byte aligned. */
int flyb200_pertoken_quant(void* y, float* scale, const void* x, int rows, int K, int x_dtype, int quant_dtype,
                           void* stream);

/* 1 when (N, K, elem_bytes) can be preshuffled into the B200 image, else 0.
 * A pure function of its arguments: the helper and the GEMM evaluate the same
 * predicate because the `is_shuffled` attribute does not survive the flat views
 * the call convention uses (tests/kernels/test_preshuffle_gemm.py:234-245). */
int flyb200_layout_kind(int N, int K, int elem_bytes);

/* Bytes of workspace flyb200_gemm_a8w8 needs for this shape and variant_hint on
 * the current device (0 when the chosen variant keeps its partial sums on chip). */
size_t flyb200_workspace_bytes(int M, int N, int K, int in_dtype, int variant_hint);

/* Which kernel variant flyb200_gemm_a8w8 would run for this problem on a GPU with
 * sm_count SMs (pure host function, no CUDA call): out8 = { kernel (1 small-M,
 * 2 large-M, 3 large-M as CTA pairs), tile width on the UMMA N side, split-K
 * factor, k-blocks per split, reduction (0 none, 1 workspace, 2 cluster), ring
 * depth, dependent-launch mode, token blocks }.  The B200 counterpart of the
 * per-tile table _TILE_PRELOAD_TABLE / tile arguments the reference's callers
 * tune by hand (kernels/gemm/preshuffle_gemm.py:19-105). */
int flyb200_describe_plan(int M, int N, int K, int in_dtype, int variant_hint, int sm_count, int* out8);

/* Device-side status word of the current device (0 = no failure since the last
 * read).  Synchronises the device; not for the launch path.  The reference only
 * prints runtime errors (lib/Runtime/ROCm/FlyRocmRuntimeWrappers.cpp:23-31). */
int flyb200_read_status(int* out_status);

/* Failure-path self test: launches one tiny kernel whose bounded wait (the one
 * every GEMM kernel uses) can never be satisfied and must give up after
 * limit_us microseconds (1..100000), set the status word to FLYB200_E_TIMEOUT
 * and return; the device stays usable.  Read the result with
 * flyb200_read_status.  The reference has no device-side failure reporting
 * (lib/Runtime/ROCm/FlyRocmRuntimeWrappers.cpp:23-31 prints host errors only). */
int flyb200_selftest_bounded_wait(unsigned int limit_us, void* stream);

/* ---- Grouped (mixture-of-experts) two-stage GEMM on the same weight image ----
 * Replaces the launchers returned by compile_moe_gemm1 / compile_moe_gemm2 and
 * compile_moe_reduction (kernels/moe/moe_gemm_2stage/gemm1.py:366-580,
 * gemm2.py:350-643, moe_reduce.py:164-205; call convention pinned by
 * tests/kernels/test_moe_gemm_2stage.py:161-193).  Routing input is what the
 * reference's moe_sorting produces (tests/kernels/test_moe_gemm_2stage.py:99-137):
 *   sorted_ids[P]      (slot << 24) | token per sorted row, every expert's rows
 *                      padded to a multiple of tile_m with token >= tokens
 *   expert_ids[blocks] expert of each block of tile_m sorted rows (-1: none)
 *   sorted_weights[P]  routed weight per sorted row
 *   num_valid_ids[1]   sorted rows in use
 * Weights: one image per expert (flyb200_shuffle_weight applied to each
 * [rows_per_expert, K] matrix), stored back to back in expert order. */
#define FLYB200_OUT_F32 2 /* flyb200_moe_gemm stage 2 with accumulate only */

/* Activation rows and their scales gathered into sorted order (the A-gather the
 * reference does inside its kernels, gemm1.py:403-460 / gemm2.py:374-380):
 *   dst[p, :] = src[r, :], dst_scale[p] = src_scale[r], r = token (by_slot = 0,
 *   stage 1), token * topk + slot (by_slot = 1, stage 2) or slot * tokens + token
 *   (by_slot = 2: slot-major per-route activations, the reference's
 *   in_dtype="int8smooth" in stage 1, gemm1.py:36-39,321-333); padding rows and rows
 *   >= num_valid_ids[0] become zero with scale zero.  rows = blocks * tile_m,
 *   row_bytes a multiple of 16. */
int flyb200_moe_gather_rows(void* dst, float* dst_scale, const void* src, const float* src_scale, const int* sorted_ids,
                            const int* num_valid_ids, int tokens, int topk, int by_slot, int row_bytes, int rows,
                            void* stream);

/* stage 1: out[token, slot, inter_dim] = silu(g) * u [* routed weight],
 *          g/u = (x . W1[e, gate/up rows]^T) * scale_w * scale_x
 * stage 2: accumulate = 1: out[token, model_dim] += y (atomic adds; the caller zeroes out),
 *          accumulate = 0: out[token * topk + slot, model_dim] = y,
 *          y = (a2 . W2[e]^T) * scale_w * scale_x [* routed weight]
 *   a_sorted        [blocks * tile_m, K] activations in sorted order (flyb200_moe_gather_rows)
 *   scale_a_sorted  [blocks * tile_m] their scales
 *   w_shuf          per-expert images of [2 * inter_dim, model_dim] (stage 1, gate rows
 *                   first) or [model_dim, inter_dim] (stage 2)
 *   scale_w         one fp32 per weight row
 *   in_dtype        FLYB200_DT_FP8 or FLYB200_DT_INT8; out_dtype FLYB200_OUT_BF16 /
 *                   _FP16, or FLYB200_OUT_F32 for stage 2 with accumulate
 *   after_gather    1: this call directly follows, on the same stream, the
 *                   flyb200_moe_gather_rows call that writes a_sorted and
 *                   scale_a_sorted, and no kernel on the stream writes the weights:
 *                   the GEMM is then launched as a programmatic dependent of the
 *                   gather pass and streams its first weight tiles while that pass
 *                   still runs (it reads the gathered rows only after the pass has
 *                   completed).  0: plain stream order.
 * Requirements: K (model_dim in stage 1, inter_dim in stage 2) a multiple of
 * 128, output row length a multiple of 16, tile_m a multiple of 16 in [16, 256]. */
int flyb200_moe_gemm(int stage, void* out, const void* a_sorted, const void* w_shuf, const float* scale_a_sorted,
                     const float* scale_w, const int* sorted_ids, const int* expert_ids, const float* sorted_weights,
                     const int* num_valid_ids, int tokens, int topk, int experts, int model_dim, int inter_dim,
                     int tile_m, int blocks, int in_dtype, int out_dtype, int doweight, int accumulate, int after_gather,
                     void* stream);

/* Routing table from the router's choice: the device form of the reference's
 * moe_sorting (layout stated in tests/kernels/test_moe_gemm_2stage.py:99-137; the
 * reference's own device kernel is kernels/moe/moe_sorting_kernel.py).  A stable
 * counting sort of the (token, slot) pairs by expert; three small launches on
 * the stream, no host synchronisation, so the whole MoE layer can be captured.
 *   topk_ids[tokens, topk] int32, topk_weights[tokens, topk] fp32
 *   sorted_ids / sorted_weights  [tokens * topk + experts * block_size - topk]
 *   sorted_expert_ids            [ceil(that / block_size)]
 *   num_tokens_post_pad          [2] = { sorted rows in use, tokens }
 *   counts_scratch               [experts] int32 (contents irrelevant on entry) */
int flyb200_moe_sorting(const int* topk_ids, const float* topk_weights, int tokens, int topk, int experts, int block_size,
                        int* sorted_ids, float* sorted_weights, int* sorted_expert_ids, int* num_tokens_post_pad,
                        int* counts_scratch, void* stream);

/* y[token, dim] = sum over slots of x[token, slot, dim] (fp32 sum, one rounding);
 * dtype FLYB200_OUT_BF16 or FLYB200_OUT_FP16, dim even.  With expert_mask
 * (int32[num_experts], else NULL) slot k of token t counts only if
 * expert_mask[topk_ids[t, k]] != 0 — the expert-parallel validity mask of the
 * reference's reduction (kernels/moe/moe_gemm_2stage/moe_reduce.py:3-7,100-150);
 * rows of masked routes are never read.  topk_ids: int32[tokens, topk]. */
int flyb200_moe_reduce(void* y, const void* x, int tokens, int topk, int dim, int dtype, const int* expert_mask,
                       const int* topk_ids, int num_experts, void* stream);

/* ---- MXFP8: E4M3 codes with one E8M0 scale per 32 elements of K on both operands ----
 * Replaces the MXFP8 x MXFP8 configuration of the reference's block-scaled
 * preshuffle GEMM (kernels/gemm/mxfp4_preshuffle.py launch_gemm with a_dtype =
 * b_dtype = "fp8"; call convention and data recipe pinned by
 * tests/kernels/test_preshuffle_gemm.py:602-700 test_mfma_a8w8_preshuffle):
 *   c[M, N] = sum_k a[m,k] * 2^(sa[m, k/32] - 127) * w[n,k] * 2^(sw[n, k/32] - 127)
 * computed with tcgen05.mma kind::mxf8f6f4.block_scale, scale factors in TMEM.
 *   a              [M, K] E4M3 codes, row-major
 *   w_shuf         [N, K] E4M3 codes in the image of flyb200_shuffle_weight
 *   scale_a_image, scale_w_image   the operands' E8M0 scales [rows, K/32] rearranged by
 *                  flyb200_mx_scale_image (the counterpart of the reference's
 *                  shuffle_scale_w4, tests/kernels/utils/gemm_common_utils.py:645-672):
 *                  [K/128][ceil(rows/128)][512 bytes], byte (r % 32) * 16 + (r / 32) * 4 + j of
 *                  an atom = scale of row r of the 128-row tile for the j-th 32-element
 *                  block of the 128-element k-block; rows past the end are zero
 *   out_dtype      FLYB200_OUT_BF16 or FLYB200_OUT_FP16
 * Requirements: K % 128 == 0, N % 128 == 0, pointers 16-byte aligned. */
int flyb200_gemm_mxfp8(void* c, const void* a, const void* w_shuf, const void* scale_a_image, const void* scale_w_image,
                       int M, int N, int K, int out_dtype, void* stream);

/* ---- MXFP4: E2M1 codes (two per byte) with one E8M0 scale per 32 elements of K on both operands ----
 * Replaces the MXFP4 x MXFP4 configuration of the same reference kernel
 * (kernels/gemm/mxfp4_preshuffle.py launch_gemm with a_dtype = b_dtype = "fp4",
 * :72-74,99-133; call convention and data recipe pinned by
 * tests/kernels/test_preshuffle_gemm.py:343-466 test_mfma_w4_flyc_preshuffle):
 *   c[M, N] = sum_k fp4(a[m,k]) * 2^(sa[m, k/32] - 127) * fp4(w[n,k]) * 2^(sw[n, k/32] - 127)
 * computed with tcgen05.mma kind::mxf4.block_scale.scale_vec::2X (64 elements of
 * K and two scale blocks per instruction), scale factors in TMEM.
 *   a              [M, K/2] bytes, row-major; element 2i of a row in the low nibble of byte i
 *   w_shuf         the [N, K/2] byte matrix of weight codes in the image of
 *                  flyb200_shuffle_weight (elem_bytes = 1, K/2 bytes per row); takes the
 *                  place of shuffle_weight_w4 (tests/kernels/utils/gemm_common_utils.py:607-642)
 *   scale_a_image, scale_w_image   as for flyb200_gemm_mxfp8: flyb200_mx_scale_image of the
 *                  [rows, K/32] scales with K counted in ELEMENTS
 * K is the number of elements.  Requirements: K % 256 == 0, N % 128 == 0, pointers
 * 16-byte aligned.  The reference's mixed configurations (fp8 or fp6 activations
 * with fp4 weights) are not built: kind::mxf8f6f4 wants 4- and 6-bit operands
 * padded to 8 bits in shared memory, which forfeits the smaller weight stream. */
int flyb200_gemm_mxfp4(void* c, const void* a, const void* w_shuf, const void* scale_a_image, const void* scale_w_image,
                       int M, int N, int K, int out_dtype, void* stream);

/* ---- mixed block-scaled kinds: 8-, 6- and 4-bit codes in byte containers ----
 * Replaces the configurations of the same reference kernel whose operands
 * differ in width: MXFP6 (E2M3) activations x MXFP4 (E2M1) weights
 * (kernels/gemm/mxfp4_preshuffle.py a_dtype = "fp6", b_dtype = "fp4"; pinned by
 * tests/kernels/test_preshuffle_gemm.py:472-587 test_mfma_a6w4_preshuffle) and
 * MXFP8 activations x MXFP4 weights (a_dtype = "fp8"; the reference's test
 * skips it).  Computed with tcgen05.mma kind::mxf8f6f4.block_scale, which takes
 * sub-byte codes only in byte-sized containers: every 16 consecutive codes of a
 * row occupy 16 bytes - 16 E4M3 bytes, or 12 bytes of 6-bit codes (code i in
 * bits [6i, 6i+6) of the little-endian bit stream) followed by 4 bytes of
 * padding, or 8 bytes of 4-bit codes (code i in nibble i, low nibble first)
 * followed by 8 bytes of padding.  Both operands are passed in that form, so
 * the weight stream has the size of FP8's: the memory saving of 4-bit weights
 * is realised by flyb200_gemm_mxfp4 (both operands 4-bit), not here.
 *   a              [M, K] bytes, row-major, codes in containers as above
 *   w_shuf         the [N, K] byte matrix of weight containers in the image of
 *                  flyb200_shuffle_weight (elem_bytes = 1)
 *   scale images   as for flyb200_gemm_mxfp8 (K counted in elements)
 *   a_format, w_format   FLYB200_MXFMT_* below
 * Requirements: K % 128 == 0, N % 128 == 0, pointers 16-byte aligned. */
#define FLYB200_MXFMT_E4M3 0
#define FLYB200_MXFMT_E5M2 1
#define FLYB200_MXFMT_E2M3 3
#define FLYB200_MXFMT_E3M2 4
#define FLYB200_MXFMT_E2M1 5
int flyb200_gemm_mx_mixed(void* c, const void* a, const void* w_shuf, const void* scale_a_image, const void* scale_w_image,
                          int M, int N, int K, int a_format, int w_format, int out_dtype, void* stream);
int flyb200_mx_scale_image(void* dst, const void* src, int rows, int K, void* stream);
size_t flyb200_mx_scale_image_bytes(int rows, int K);

const char* flyb200_strerror(int code);
const char* flyb200_last_cuda_error(void);
int flyb200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FLYB200_H_ */
