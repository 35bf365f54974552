/*
 * gridbook_b200 -- C ABI of the sm_100a codebook-decode linear / routed-MoE kernels.
 *
 * One shared library (libgridbook_b200.so) replaces the reference's JIT-built
 * pybind11 modules (gridbook/cuda_ext.py:344-354 `_EXT_SYMBOLS`, :446-451
 * `_V2_SYMBOLS`, :1370-1377, :1087-1095, :2011-2033).  Conventions, all taken from the
 * reference's bindings (gridbook/csrc/cb_gemv.cu:658-712):
 *   - every pointer is a DEVICE pointer on the current device unless it says host;
 *   - work is enqueued on the caller's stream, nothing synchronises, nothing allocates;
 *   - outputs are caller-owned; scratch is passed in as `workspace`;
 *   - the return value is 0 on success, otherwise a GB_E* code, and
 *     gb_last_error() returns a thread-local description (the reference raises
 *     RuntimeError from TORCH_CHECK);
 *   - bf16 tensors are row-major and contiguous, index vectors are int32.
 */
#ifndef GRIDBOOK_B200_H_
#define GRIDBOOK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GB_ABI_VERSION 3
#define GB_API __attribute__((visibility("default")))

enum { GB_OK = 0, GB_EINVAL = 1, GB_ECUDA = 2, GB_EUNSUPPORTED = 3, GB_EWORKSPACE = 4 };

enum { GB_GRID_FP4 = 0, GB_GRID_FP8 = 1 };
/* index-encoding modes of docs/SPEC.md:94-128 */
enum { GB_MODE_PRODUCT = 0, GB_MODE_SIGNED = 1, GB_MODE_FULL = 2 };
/* docs/SPEC.md:130-177: none (fp8), v1 = 16 E4M3 bytes, v2 = super byte + 16 nibbles */
enum { GB_SCALE_NONE = 0, GB_SCALE_V1 = 1, GB_SCALE_V2 = 2 };
/* how `amax / c` is evaluated in the activation buckets: the fp32 reciprocal
 * multiply of torch-on-CUDA that the reference kernels reproduce
 * (gridbook/csrc/cb_gemv.cu:88-91,485-511), or a true division (torch-on-CPU) */
enum { GB_SCALE_RULE_RECIP = 0, GB_SCALE_RULE_DIV = 1 };
enum { GB_ACT_NONE = 0, GB_ACT_FP4_GROUP16 = 1, GB_ACT_FP8_TOKEN = 2 };

/* One packed format (the `scheme` dict of gridbook/config.py:803-957). */
typedef struct gb_format {
  int32_t grid;         /* GB_GRID_*  */
  int32_t mode;         /* GB_MODE_*  */
  int32_t k_bits;       /* bits per 8-weight codeword */
  int32_t n_sub;        /* product mode: sub-indices per codeword (2 or 4); else 1 */
  int32_t type_size;    /* bytes per 256-weight superblock */
  int32_t scale_coding; /* GB_SCALE_* */
} gb_format;

/* A packed weight matrix as the kernels see it.  Mirrors the tensors the
 * reference's linear method keeps resident (gridbook/linear.py:374-680). */
typedef struct gb_weight {
  const uint8_t* qw;            /* [rows, row_stride] packed superblocks; readable up to
                                   the next 16-byte boundary past the last row */
  int64_t row_stride;           /* bytes between rows (>= K/256*type_size) */
  const void* codebook;         /* flat codebook: bf16 (fp4 grid) or E4M3 bytes (fp8 grid),
                                   gridbook/codec.py:146-167 */
  const int32_t* cb_row_offset; /* [rows] element offset of each row's codebook block, or NULL = 0
                                   (gridbook/linear.py:419-459) */
  const float* compose;         /* [256*16] two-tier table, v2 only (gridbook/codec.py:170-183) */
  const float* weight_scale;    /* [rows] fp8 grid per-row scale, else NULL */
  float global_scale;           /* epilogue multiplier (1.0f = none); no reference counterpart */
  int64_t rows;                 /* N */
  int64_t K;
  gb_format fmt;
} gb_weight;

/* The version a binding compares with GB_ABI_VERSION before its first call: with the binding's
 * list of required symbols this replaces the strict symbol tuples the reference checks when it
 * loads a native module (gridbook/cuda_ext.py:344-365,446-451), so a stale library fails at load. */
GB_API int gb_abi_version(void);
/* Text of the calling thread's last non-zero status; replaces the message of the RuntimeError a
 * TORCH_CHECK raises in the reference's bindings (gridbook/csrc/cb_gemv.cu:658-712). */
GB_API const char* gb_last_error(void);

/* Per-device one-time set-up (function attributes, SM count).  Call at model load,
 * before any stream capture; replaces the `*_prepare` entries of
 * gridbook/csrc/cb_gemv_v2.cu:495-548. */
GB_API int gb_prepare(int device);

/* Device error word written by kernels whose bounded waits ran out; 0 when healthy.  No counterpart
 * in the reference, whose kernels do not wait on one another. */
GB_API int gb_device_status(int device, int* status_out);

/* Clears the device error word (after the cause has been dealt with). */
GB_API int gb_device_status_reset(int device);
/* How long a device-side wait of the exchange kernels and of gb_gemv_tab may spin before it gives
 * up and raises the status word: `ms` milliseconds, 0 = the default of two seconds.  Host-side
 * setting read at launch; meant for tests that make a wait run out on purpose. */
GB_API int gb_set_wait_limit_ms(int ms);

/* ---- activation buckets ---------------------------------------------------- */
/* replaces fp8_act_qdq (gridbook/csrc/cb_gemv.cu:135-172, gridbook/ops.py:441-447) */
GB_API int gb_fp8_act_qdq(const void* x_bf16, void* out_bf16, int64_t M, int64_t K,
                   int scale_rule, void* stream);
/* replaces fp4_act_qdq (gridbook/csrc/cb_gemv.cu:532-570, gridbook/ops.py:454-460) */
GB_API int gb_fp4_act_qdq(const void* x_bf16, void* out_bf16, int64_t M, int64_t K,
                   int scale_rule, void* stream);

/* ---- decoded tiles (bit-exact gates) ---------------------------------------- */
/* replaces cb_expand_fp8 (gridbook/csrc/cb_gemv.cu:2168-2280, gridbook/ops.py:96-116):
 * rows [row0, row0+nrows) -> [nrows, K] E4M3 bytes */
GB_API int gb_expand_fp8(const gb_weight* w, int64_t row0, int64_t nrows, void* out_e4m3,
                  void* stream);
/* The served fp8-grid weight of rows [row0, row0+nrows): -> [nrows, K] bf16 =
 * bf16(value * weight_scale[row]), the per-weight rounding of the decode contract
 * (gridbook/csrc/cb_gemv.cu:20-27,219-228), for bf16 tensor-core routes that must keep it. */
GB_API int gb_expand_fp8_bf16(const gb_weight* w, int64_t row0, int64_t nrows, void* out_bf16,
                              void* stream);
/* replaces cb_expand_v2 (gridbook/csrc/cb_gemv_v2.cu:374-439,802-863, gridbook/ops.py:119-134)
 * for every fp4 mode and scale coding: -> [nrows, K] bf16 = bf16(value * group scale) */
GB_API int gb_expand_fp4_bf16(const gb_weight* w, int64_t row0, int64_t nrows, void* out_bf16,
                       void* stream);
/* native NVFP4 tile (docs/SPEC.md:30-39; the operand of the reference's block-scaled
 * GEMM, gridbook/csrc/cb_fused_fp4_gemm.cu:25-60): packed E2M1 [nrows, K/2] (even element
 * in the low nibble) and E4M3 group scales, either row-major [nrows, K/16]
 * (sf_swizzled = 0) or in the 128x4 atom layout of gridbook/codec.py:353-374
 * (sf_swizzled = 1, plane padded to 128 rows x 4 groups, caller zero-fills).  sf_swizzled = 2:
 * the same atom layout in the operand form of the block-scaled MMA, whose UE4M3 scale factors
 * carry no sign - a negative group scale moves its sign into the group's sixteen values. */
GB_API int gb_expand_fp4_nvfp4(const gb_weight* w, int64_t row0, int64_t nrows, void* out_packed,
                        void* out_sf, int sf_swizzled, void* stream);

/* ---- decode-batch linear (M <= 16; up to gb_gemv_row_batch_max rows where that is larger) ---- */
/* replaces cb_gemv_fp8 / cb_gemv_fp4_v2 (gridbook/csrc/cb_gemv.cu:658-712,1138-1198;
 * gridbook/ops.py:52-93).  y[M,N] = bucket(x)[M,K] . W^T, fp32 accumulate, one bf16
 * rounding.  `act` selects a fused activation bucket applied to x first (GB_ACT_NONE
 * when x is already bucketed).  workspace: gb_gemv_workspace_bytes() bytes.
 * Three formats - the literal one (fp4 grid, full mode, k = 8, v1 scales), the two-tier product
 * format fp4 k = 16 with its superblocks padded to 80 bytes (fmt.type_size = 80: the 73 shipped
 * bytes, then 7 ignored ones), and the fp8 product format k = 32 - with one codebook, K >= 1024,
 * N >= 128 and 16-byte aligned rows are also served, up to gb_gemv_row_batch_max() rows, by a
 * kernel that decodes the packed rows into TENSOR MEMORY and multiplies on the tensor cores
 * (tcgen05, weights on the M side, no decoded copy anywhere) - the decode-in-mainloop band of
 * the reference (gridbook/csrc/cb_fused_fp4v2_gemm.cu, M <= 128) with the decode contract kept.
 * The literal format takes it from gb_set_row_routes' `umma_min` rows on (its table kernels are
 * faster below), the other two from one row on.  Other formats return GB_EUNSUPPORTED past 16
 * rows and take the expand + gb_gemm_tn route. */
GB_API int64_t gb_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K);
GB_API int gb_gemv(const void* x_bf16, int64_t M, const gb_weight* w, int act, int scale_rule,
            void* y_bf16, void* workspace, int64_t workspace_bytes, void* stream);
/* Most rows gb_gemv takes for this weight: 16, or what the tensor-core decode kernel serves for its
 * format and layout (up to 128).  No counterpart in the reference. */
GB_API int gb_gemv_row_batch_max(const gb_weight* w);

/* Row counts at which gb_gemv changes kernel for the literal format: up to `dot_rows` rows run one
 * inner-product-table GEMV per row (default 4, at most 8), from `umma_min` rows on the tensor-core
 * decode kernel (default 5; 129 switches that kernel off for every format).  0 restores a default.  Process-wide; for tests and tuning.  No
 * counterpart in the reference, whose lane selection is a set of environment flags. */
GB_API int gb_set_row_routes(int dot_rows, int umma_min);

/* Same computation as gb_gemv for callers that are not allowed to allocate device memory
 * and have no workspace to hand over: a runtime that has already given every byte of the
 * device to its own pools, a serving loop whose allocator is frozen once graphs are being
 * recorded, or a host binding whose ABI simply has no place for a scratch buffer.  The
 * scratch is a fixed array of GB_GEMV_STATIC_SCRATCH_BYTES inside the library, resident on
 * every device that loads it for the life of the process.
 *   - Shapes whose scratch (gb_gemv_workspace_bytes) exceeds the array are refused with
 *     GB_EINVAL and a message naming both sizes; use gb_gemv for those.
 *   - The first call on a device looks up the array's device address; make that call during
 *     set-up, before any stream capture starts on that device.
 *   - All calls share the one array, which keeps whatever the previous call left; the part
 *     that must start from zero is cleared on the caller's stream every time.  Two calls that
 *     may overlap on the GPU (different streams, no dependency) race on it: serialise them.
 *   - No cudaMalloc, cudaFree or allocating library routine is called.
 * This entry point has no counterpart in the reference. */
#define GB_GEMV_STATIC_SCRATCH_BYTES (4u << 20)
GB_API int gb_gemv_static(const void* x_bf16, int64_t M, const gb_weight* w, int act, int scale_rule,
                          void* y_bf16, void* stream);

/* One activation row of the literal format (fp4 grid, full mode, k = 8, v1 scales, one codebook
 * per matrix, 16-byte aligned rows, >= 64 rows) against n_weights <= 4 matrices that read the SAME
 * row - q and kv, gate and up - in one launch: y[i][N_i] = bucket(x)[K] . W_i^T.  Replaces the
 * same reference entries as gb_gemv (gridbook/csrc/cb_gemv.cu:1138-1198) for M = 1, one launch
 * where gb_gemv needs two per matrix.  The K-slice partial sums travel through `slots`, an
 * "armed" buffer of gb_gemv_tab_slots_bytes() bytes (256-byte aligned): every byte must read 0xFF
 * before the first call (gb_gemv_tab_arm), and every call leaves it in that state again, so one
 * buffer serves any number of consecutive calls, of any shapes it is large enough for, on one
 * stream.  Calls that may overlap on the GPU need a buffer each.  A buffer that was never armed
 * raises the device status word (24); after any non-zero status, arm the buffer again.
 * act: GB_ACT_NONE or GB_ACT_FP4_GROUP16.  Returns GB_EUNSUPPORTED for other formats or layouts
 * and for K so wide that one wave of CTAs cannot hold every K slice (use gb_gemv). */
GB_API int64_t gb_gemv_tab_slots_bytes(const gb_weight* const* w, int n_weights);
GB_API int gb_gemv_tab_arm(void* slots, int64_t bytes, void* stream);
GB_API int gb_gemv_tab(const void* x_bf16, const gb_weight* const* w, void* const* y_bf16, int n_weights,
                       int act, int scale_rule, void* slots, int64_t slots_bytes, void* stream);

/* ---- prefill (M > 16): tensor-core GEMM over decoded tiles --------------------------- */
enum { GB_GEMM_BF16 = 0, GB_GEMM_E4M3 = 1 };
/* Per-token dynamic E4M3 quantisation of bf16 activations: q[M,K] bytes and scale[M] with
 * x ~ q * scale; replaces the reference's use of vLLM's dynamic_per_token_scaled_fp8_quant
 * (gridbook/native_cutlass.py:158-168; arithmetic of gridbook/codec.py:428-437). */
GB_API int gb_fp8_quantize_rows(const void* x_bf16, void* q_e4m3, float* scale, int64_t M, int64_t K,
                                int scale_rule, void* stream);
/* D[M,N] bf16 = bf16( global_scale * a_scale[m] * b_scale[n] * sum_k A[m,k] B[n,k] ), A [M,K] and
 * B [N,K] row-major in bf16 (GB_GEMM_BF16) or E4M3 bytes (GB_GEMM_E4M3); scale vectors may be
 * NULL.  K*elem_size must be a multiple of 128 bytes, pointers 16-byte aligned.  tcgen05
 * kind::f16 / kind::f8f6f4 with the accumulator in tensor memory.  With B = gb_expand_fp8 /
 * gb_expand_fp4_bf16 of a layer this replaces the reference's expand + GEMM prefill routes and
 * the scaled epilogue of its fused FP8 lane (gridbook/linear.py:1146-1152,1255-1264;
 * gridbook/csrc/cb_fused_gemm.cu:476-486). */
GB_API int gb_gemm_tn(const void* A, const void* B, void* D_bf16, int64_t M, int64_t N, int64_t K, int kind,
                      const float* a_scale, const float* b_scale, float global_scale, void* stream);
/* ---- prefill on the block-scaled FP4 tensor cores ----------------------------------- */
/* Bytes of a scale-factor plane in the 128 x 4 atom layout for `rows` rows of K elements
 * (rows padded to 128, groups of sixteen padded to four). */
GB_API int64_t gb_nvfp4_sf_bytes(int64_t rows, int64_t K);
/* Native NVFP4 quantisation of bf16 activation rows with one scale per row, chosen so that the
 * row's largest group scale is `range` (<= 448): packed E2M1 [M, K/2] (even element in the low
 * nibble), UE4M3 group-of-16 scale factors in the atom layout (gb_nvfp4_sf_bytes(M, K) bytes,
 * the padding rows of the last tile are cleared), a_scale[M] with x ~ a_scale * SF * code.
 * Replaces cb_nvfp4_quantize_rows (gridbook/csrc/cb_fused_fp4_gemm.cu:291-450,459-479) with
 * the exactly rounded arithmetic of its torch statement (gridbook/codec.py:377-425). */
GB_API int gb_nvfp4_quantize_rows(const void* x_bf16, int64_t M, int64_t K, float range, void* packed,
                                  void* sf, float* a_scale, void* stream);
/* D[M,N] bf16 = bf16(global_scale * a_scale[m] * sum_k (A SFA)[m,k] (B SFB)[n,k]): A [M,K/2] and
 * B [N,K/2] packed E2M1, SFA / SFB their scale-factor planes in the atom layout, K a multiple of
 * 256.  tcgen05 kind::mxf4nvf4 (block16, UE4M3 scale factors in tensor memory), fp32 accumulate.
 * With B, SFB = gb_expand_fp4_nvfp4(.., sf_swizzled = 2) of a layer and A, SFA, a_scale =
 * gb_nvfp4_quantize_rows this replaces the reference's block-scaled prefill
 * (gridbook/csrc/cb_fused_fp4_gemm.cu:758-903; mainloop
 * gridbook/csrc/cutlass_fork/sm120_cb_fused_fp4_mma.hpp:661-805). */
GB_API int gb_gemm_fp4(const void* A, const void* sfa, const void* B, const void* sfb, void* D_bf16, int64_t M,
                       int64_t N, int64_t K, const float* a_scale, float global_scale, void* stream);

/* The same GEMM over expert segments (routed prefill): A [P,K] holds the routed rows sorted by
 * expert, expert e owning rows [seg_offsets[e], seg_offsets[e+1]) (gb_moe_route's offsets, read
 * on the device: no host read); B [E*N,K] is the decoded stack (gb_expand_* over all E*N rows);
 * sorted row j of expert e gets D[r, n] = global_scale * a_scale[j] * b_scale[e*N+n] * <A[j], B[e*N+n]>
 * with r = row_map[j] (row_map = gb_moe_route's order puts the result in pair order) or r = j
 * when row_map is NULL.  Rows at or past seg_offsets[E] are neither read into a result nor
 * written.  E <= 1024.  Replaces the grouped bf16 GEMM over expert segments and the grouped
 * decode-in-mainloop prefill (gridbook/ops.py:137-306,309-428;
 * gridbook/csrc/cb_bf16_grouped_gemm.cu:228-245,547-610;
 * gridbook/csrc/cb_moe_persistent_b.cu:1645-1960). */
GB_API int gb_gemm_tn_grouped(const void* A, const void* B, void* D_bf16, int64_t P, int64_t N, int64_t K, int kind,
                              int64_t E, const int32_t* seg_offsets, const int32_t* row_map, const float* a_scale,
                              const float* b_scale, float global_scale, void* stream);
/* out[j, :] = x[x_row[order[j]], :] (x[order[j]] when x_row is NULL) for the sorted rows
 * j < seg_offsets[E]: the routed rows of a [T,K] bf16 batch in expert order (the reference sorts
 * with torch indexing, gridbook/moe.py:1609-1625).  K a multiple of 8. */
GB_API int gb_moe_gather_rows(const void* x_bf16, const int32_t* x_row, const int32_t* order,
                              const int32_t* seg_offsets, int64_t E, int64_t P, int64_t K, void* out_bf16,
                              void* stream);
/* out[j, c] = bf16(bf16(silu(h[j, c])) * h[j, inter + c]) for the sorted rows j < seg_offsets[E];
 * h [P, 2*inter] bf16 (the chain of tests/test_cuda_gemv.py:336-338).  inter a multiple of 8.
 * act = GB_ACT_FP4_GROUP16 also applies the next projection's fp4 group-16 bucket to the result
 * (same bits as gb_fp4_act_qdq on it; inter a multiple of 16), GB_ACT_NONE leaves it as it is. */
GB_API int gb_moe_swiglu_rows(const void* h_bf16, const int32_t* seg_offsets, int64_t E, int64_t P, int64_t inter,
                              int act, int scale_rule, void* out_bf16, void* stream);

/* ---- routed MoE -------------------------------------------------------------- */
/* Device-side histogram + exclusive scan + stable expert-major permutation of the
 * P = T*topk routed pairs; replaces the torch chain of gridbook/moe.py:1609-1625 and
 * gridbook/moe_routing.py:99-207.  ids < 0 (vLLM's padding sentinel,
 * gridbook/ops.py:764-784) are dropped from every expert.
 *   counts [E], offsets [E+1] (exclusive scan, offsets[E] = routed pairs kept),
 *   order [P]: sorted position -> flat pair index t*topk+slot (token-ascending per expert).
 * Optional (both or neither): topk_weights [P] fp32 in, pair_w [P] fp32 out = the combine
 * weight of every pair, i.e. the router weight rounded to bf16 (gridbook/moe.py:2407-2408)
 * and zero for a dropped pair (gridbook/ops.py:764-784), so no separate masking pass runs.
 * expert_base: the experts held here are the global ids [expert_base, expert_base + E); ids
 * outside that range are dropped like padding (expert parallelism; 0 on one GPU). */
GB_API int gb_moe_route(const int32_t* topk_ids, int64_t T, int64_t topk, int64_t E, int64_t expert_base,
                 int32_t* counts, int32_t* offsets, int32_t* order,
                 const float* topk_weights, float* pair_w, void* stream);
/* The same with a workspace of gb_moe_route_workspace_bytes(T, topk, E) bytes (0 below 4096
 * pairs or above 256 experts: one CTA does it all).  With the workspace the routing of a large
 * batch runs as three launches over tiles of 1024 pairs that use the whole GPU (per-tile
 * histograms, scan, placement) instead of one CTA; same outputs, same stable order.
 * workspace = NULL: gb_moe_route. */
GB_API int64_t gb_moe_route_workspace_bytes(int64_t T, int64_t topk, int64_t E);
GB_API int gb_moe_route_ws(const int32_t* topk_ids, int64_t T, int64_t topk, int64_t E, int64_t expert_base,
                           int32_t* counts, int32_t* offsets, int32_t* order, const float* topk_weights,
                           float* pair_w, void* workspace, int64_t ws_bytes, void* stream);

/* Grouped GEMV over routed pairs; replaces cb_moe_gemv_fp8 / cb_moe_gemv_fp4_v2 /
 * cb_moe_gemv_v2 (gridbook/csrc/cb_gemv.cu:1210-1681,1873-2138; gridbook/csrc/cb_gemv_v2.cu:233-366).
 * `w` describes ONE expert's matrix; expert e starts at qw + e*expert_stride bytes and
 * weight_scale + e*rows.  Pairs come grouped by expert through (offsets, order); pair p
 * reads activation row x_row[p] (NULL = p) and writes y[p].  When `swiglu` is set the
 * kernel's output is silu(gate)*up of rows [0,rows/2) and [rows/2,rows) -> y[P, rows/2]
 * (replaces native_moe_activation, gridbook/native_cutlass.py:129-155).
 * act: GB_ACT_NONE, or GB_ACT_FP4_GROUP16 to apply the fp4 activation bucket (scale_rule as
 * in gb_fp4_act_qdq) while the rows are staged, which saves the separate bucket launch; every
 * row tile of an expert buckets its rows again, so it pays for small batches only.
 * y_rows (optional, not with swiglu): instead of y_bf16, pair p's output row goes to
 * y_rows->base[p / rows_per_rank] + (p % rows_per_rank) * rows * 2 bytes, i.e. straight into
 * the buffer of the rank the pair came from (expert-parallel combine over peer memory). */
typedef struct gb_peer_rows {
  void* base[8];
  int64_t rows_per_rank;
} gb_peer_rows;
GB_API int64_t gb_moe_gemv_workspace_bytes(int64_t P, int64_t rows);
GB_API int gb_moe_gemv(const void* x_bf16, const int32_t* x_row, const gb_weight* w,
                int64_t expert_stride, int64_t E, const int32_t* offsets,
                const int32_t* order, int64_t P, int swiglu, int act, int scale_rule,
                void* y_bf16, const gb_peer_rows* y_rows, void* workspace,
                int64_t workspace_bytes, void* stream);

/* Grouped linear over rows ALREADY in expert order (gb_moe_gather_rows), for batches between the
 * decode kernels and the grouped GEMM: x_sorted [P,K] bf16 (bucketed), expert e owns rows
 * [seg_offsets[e], seg_offsets[e+1]); y[r, :] = x_sorted[j] . W_e^T with r = row_map[j] (or j).
 * Every (expert, 128-row tile) CTA decodes its packed rows into shared memory and multiplies on
 * the tensor cores (tcgen05, weights on the M side), 64 routed rows per pass; experts without rows
 * cost nothing.  Literal fp4 format, contiguous stack (expert_stride = rows * row_stride), rows a
 * multiple of 128; GB_EUNSUPPORTED otherwise.  y_rows (optional): row r goes to its home rank's
 * buffer base[r / rows_per_rank] + (r % rows_per_rank) * rows instead of y_bf16, as in gb_moe_gemv.  Replaces the grouped decode-in-mainloop kernels of
 * the reference for mid-size batches (gridbook/csrc/cb_moe_persistent_b.cu:1645-1960). */
GB_API int gb_moe_gemv_sorted(const void* x_sorted_bf16, const gb_weight* w, int64_t expert_stride, int64_t E,
                              const int32_t* seg_offsets, const int32_t* row_map, int64_t P, void* y_bf16,
                              const gb_peer_rows* y_rows, void* stream);

/* The same routed projection for SMALL batches of the literal format (fp4 grid, full mode,
 * k = 8, E4M3-direct scales, one codebook per stack): every routed pair p is its own M = 1 linear
 * through the inner-product-table kernel, y[p] = W[pair_expert[p]] . x[x_row[p]] (NULL x_row:
 * row p).  No routing tables are needed; pairs whose expert lies outside
 * [expert_base, expert_base + E) are skipped.  An expert's weights stream once per pair, as in
 * the reference's grouped GEMV (gridbook/csrc/cb_gemv.cu:1220-1233), so this pays while few
 * pairs share an expert; pairs_expected (0 = P) sizes the grid for the pairs expected to be
 * live on this rank.  Returns GB_EUNSUPPORTED for any other format (use gb_moe_gemv).
 * swiglu / act / y_rows as in gb_moe_gemv. */
GB_API int64_t gb_moe_gemv_pairs_workspace_bytes(int64_t P, int64_t rows, int64_t K);
GB_API int gb_moe_gemv_pairs(const void* x_bf16, const int32_t* x_row, const gb_weight* w,
                int64_t expert_stride, int64_t E, int64_t expert_base, const int32_t* pair_expert,
                int64_t P, int64_t pairs_expected, int swiglu, int act, int scale_rule, void* y_bf16,
                const gb_peer_rows* y_rows, void* workspace, int64_t workspace_bytes, void* stream);

/* Both projections of the routed MLP through gb_moe_gemv_pairs' kernels in TWO launches: the
 * gate/up GEMVs leave their K-slice partial sums in the workspace, and the down projection sums
 * them, applies SwiGLU and the activation bucket while it stages each pair's row (replaces
 * cb_moe_gemv_* + native_moe_activation + the second bucket of gridbook/moe.py:2388-2504 for
 * small batches).  w13: one expert's [2*inter, hidden] matrix, w2: [hidden, inter]. */
GB_API int64_t gb_moe_mlp_pairs_workspace_bytes(int64_t P, int64_t hidden, int64_t inter);
GB_API int gb_moe_mlp_pairs(const void* x_bf16, const int32_t* x_row, const gb_weight* w13, int64_t stride13,
                const gb_weight* w2, int64_t stride2, int64_t E, int64_t expert_base,
                const int32_t* pair_expert, int64_t P, int64_t pairs_expected, int act, int scale_rule,
                void* y_bf16, const gb_peer_rows* y_rows, void* workspace, int64_t workspace_bytes,
                void* stream);

/* out[t] = sum over the token's topk pairs of w[p] * y[p], fp32 accumulate, one bf16
 * rounding; replaces cb_moe_combine (gridbook/csrc/cb_gemv.cu:1853-1871,2140-2158).
 * pair p = t*topk + slot.  topk_ids (optional, with E): pairs whose id lies outside [0, E)
 * were dropped by gb_moe_route and have no row in y; they are skipped, so y needs no
 * clearing beforehand.
 * round_weights: pair_w holds raw router weights; round each to bf16 first
 * (gridbook/moe.py:2407-2408), for callers that did not get them from gb_moe_route. */
GB_API int gb_moe_combine(const void* y_bf16, const float* pair_w, const int32_t* topk_ids,
                   int64_t E, int64_t T, int64_t topk, int64_t H, int round_weights,
                   void* out_bf16, void* stream);

/* Kernel launches this library has issued in this process so far (launches recorded into a
 * CUDA graph count once, at capture).  No reference counterpart; used by the benchmark to
 * report how many of its own kernels a step runs. */
GB_API int64_t gb_launch_count(void);

/* ---- peer-memory exchange on one NVSwitch node ------------------------------- */
/* None of this has a counterpart in the reference, which runs on one GPU
 * (gridbook/config.py:565-576).  One process per GPU; a buffer from gb_peer_alloc is exported
 * as a 64-byte handle, sent to the other ranks by any host channel, and mapped there with
 * gb_peer_open.  The allocation, export and mapping calls are setup-time only. */
#define GB_PEER_MAX 8
#define GB_PEER_HANDLE_BYTES 64
#define GB_PEER_FLAG_BYTES 128
GB_API int gb_peer_alloc(int64_t bytes, void** ptr);          /* zero-filled device buffer */
GB_API int gb_peer_free(void* ptr);
GB_API int gb_peer_export(void* ptr, void* handle64);
GB_API int gb_peer_open(const void* handle64, void** ptr);
GB_API int gb_peer_close(void* ptr);

typedef struct gb_peer_group {
  int32_t rank, world;              /* world <= GB_PEER_MAX */
  void* flags[GB_PEER_MAX];         /* flags[r]: rank r's GB_PEER_FLAG_BYTES block (own: gb_peer_alloc; others: mapped) */
} gb_peer_group;

typedef struct gb_peer_piece {
  const void* src;                  /* this rank's piece, rows x row_bytes at src_pitch */
  void* dst[GB_PEER_MAX];           /* where the piece goes inside rank r's buffer (dst_pitch between rows) */
  int64_t rows, row_bytes, src_pitch, dst_pitch;
} gb_peer_piece;

/* All-gather by peer stores: every rank copies its pieces (up to four) into every rank's
 * buffer, between a "buffers are free" and a "stores are visible" exchange of flags, in one
 * launch.  Every rank must make the same sequence of gb_peer_allgather / gb_peer_barrier calls.
 * A peer that does not show up within two seconds raises gb_device_status (3); nothing hangs. */
GB_API int gb_peer_allgather(const gb_peer_group* g, const gb_peer_piece* pieces, int n_pieces, void* stream);
GB_API int gb_peer_barrier(const gb_peer_group* g, void* stream);   /* "my stores before this call are visible" */
/* gb_moe_combine that first does gb_peer_barrier's exchange inside the same launch: the rows of
 * y were stored by the peers' down projections (gb_moe_gemv / gb_moe_gemv_pairs with y_rows).
 * Counts as one exchange in the ranks' common call sequence. */
GB_API int gb_moe_combine_peer(const void* y_bf16, const float* pair_w, const int32_t* topk_ids,
                   int64_t E, int64_t T, int64_t topk, int64_t H, int round_weights,
                   void* out_bf16, const gb_peer_group* g, void* stream);

/* The same all-gather for small pieces, flag-in-data: every 4-byte word is sent as an 8-byte
 * {word, exchange number} store into a staging buffer of the receiver (ll[r]: rank r's buffer of
 * ll_bytes, zero at first use, mapped here), who unpacks it into its own memory.  One one-way
 * trip instead of two flag round trips.  dst_local[s] says where rank s's piece lands in THIS
 * rank's buffer.  All pieces of a call together must fit ll_bytes / (16 * world) words. */
typedef struct gb_peer_ll_piece {
  const void* src;
  void* dst_local[GB_PEER_MAX];
  int64_t rows, row_bytes, src_pitch, dst_pitch;
} gb_peer_ll_piece;
GB_API int gb_peer_allgather_ll(const gb_peer_group* g, void* const* ll, int64_t ll_bytes,
                                const gb_peer_ll_piece* pieces, int n_pieces, void* stream);

/* Column-parallel decode linear, compute and collective in one pass: this rank's row shard of a
 * fused module (an equal slice of every role) times ONE activation row through the
 * inner-product-table kernel, then a single launch that adds the K slices, rounds to bf16 and
 * all-gathers the shards flag-in-data (as gb_peer_allgather_ll) into every rank's full output
 * row y_full [N].  layout: per role the first column of the slice inside the shard (lcol), the
 * global column of rank 0's slice (gcol0) and the slice width; rank s's slice of role r lands at
 * gcol0[r] + s * width[r].  Returns GB_EUNSUPPORTED for formats/shapes without the table kernel:
 * run gb_gemv and gb_peer_allgather_ll instead (every rank gets the same answer, the format is
 * the same everywhere).  Counts as one exchange in the ranks' common call sequence. */
typedef struct gb_gather_layout {
  int32_t n_roles;
  int64_t lcol[4], gcol0[4], width[4];
} gb_gather_layout;
GB_API int gb_gemv_allgather(const void* x_bf16, const gb_weight* w, int act, int scale_rule,
                             const gb_peer_group* g, void* const* ll, int64_t ll_bytes,
                             const gb_gather_layout* layout, void* y_full_bf16, void* workspace,
                             int64_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GRIDBOOK_B200_H_ */
