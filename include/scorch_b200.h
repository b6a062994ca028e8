/*
 * scorch_b200 — C ABI of the B200 (sm_100a) sparse kernels that replace the CPU/OpenMP kernels
 * behind scorch.matmul / scorch.einsum.
 *
 * Conventions
 *   - Every pointer argument is a DEVICE pointer unless its name ends in "_host".
 *   - Index arrays are int32, values are 1-D, dense operands are row-major with an explicit
 *     leading dimension (elements), exactly the arrays the reference hands to its kernels
 *     (reference: src/scorch/prebuilt_kernels.py:211-218, src/scorch/storage.py:46-51).
 *   - Sizes are 64-bit.  Where the reference keeps a size in a 32-bit int (csrc/spmm.h:113,
 *     csrc/kernels.h:110,520) and the value would not fit, the call returns SB_ERR_OVERFLOW
 *     instead of wrapping.
 *   - `stream` is a cudaStream_t passed as void*.  Calls are asynchronous on that stream unless
 *     stated otherwise.  Nothing here allocates device memory: outputs and workspaces are the
 *     caller's, sized with the *_bytes() queries.
 *   - Return value: 0 (SB_OK) or an SB_ERR_* code; sb_last_error() gives the message of the
 *     last failing call on the calling thread.  No call throws, none falls back to the CPU.
 *
 * Reference-side binding: each entry point names the reference function it replaces
 * (path:line inside the reference project).
 */
#ifndef SCORCH_B200_H_
#define SCORCH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SB_API __attribute__((visibility("default")))
#else
#define SB_API
#endif

enum {
  SB_OK = 0,
  SB_ERR_INVALID_ARG = 1, /* null pointer, negative size, misaligned or inconsistent shapes */
  SB_ERR_CUDA = 2,        /* a CUDA runtime call or launch failed; see sb_last_error() */
  SB_ERR_OVERFLOW = 3,    /* a quantity the reference stores as int32 does not fit */
  SB_ERR_WORKSPACE = 4,   /* workspace/scratch smaller than the matching *_bytes() query */
  SB_ERR_UNSUPPORTED = 5  /* dtype or shape outside what the kernels implement */
};

/* value dtypes of the typed entry points; suffixes follow csrc/prebuilt_types.h:36-62 */
enum { SB_F32 = 0, SB_F64 = 1, SB_I32 = 2, SB_I64 = 3 };

SB_API int sb_abi_version(void);
SB_API const char* sb_status_string(int status);
SB_API const char* sb_last_error(void);

/* --------------------------------------------------------------------------------------------
 * Row plan: the nnz-balanced split of a CSR matrix that SpMM uses.  Rows with more than
 * SB_HEAVY_ROW_NNZ stored entries ("heavy" rows, e.g. hubs of a power-law graph) are cut into
 * segments of SB_HEAVY_ROW_NNZ entries; one CTA sums one segment in shared memory and a
 * fixed-order second stage adds the segment sums, so results do not depend on scheduling.
 * The plan depends only on `pos`; build it once per matrix and reuse it.
 * Replaces: the atomic work-stealing row loop of csrc/spmm.h:2032-2046 and the
 * schedule(dynamic,16) loop of csrc/spmm.h:121.
 * -------------------------------------------------------------------------------------------- */
#define SB_HEAVY_ROW_NNZ 1024

/* bytes of device memory a plan for (m rows, nnz entries) needs (worst case over all patterns) */
SB_API size_t sb_csr_plan_bytes(int64_t m, int64_t nnz);
/* upper bound on the number of heavy-row segments of any matrix with nnz entries */
SB_API int64_t sb_csr_plan_max_segments(int64_t nnz);
/* asynchronous; `plan` must hold sb_csr_plan_bytes(m, nnz) bytes and be 16-byte aligned */
SB_API int sb_csr_plan_build(int64_t m, int64_t nnz, const int32_t* pos, void* plan,
                             size_t plan_bytes, void* stream);
/* synchronises `stream`; returns the exact counts so callers can size scratch tightly */
SB_API int sb_csr_plan_counts(const void* plan, int64_t* heavy_rows_host, int64_t* segments_host,
                              void* stream);

/* nnz-balanced contiguous row blocks for sharding one matrix over `parts` GPUs:
 * bounds[g] = first row of block g (bounds[parts] = m); block g starts at the first row whose
 * pos[] reaches g*nnz/parts.  `bounds` is a DEVICE array of parts+1 int64.  No reference
 * counterpart: the reference is single-process. */
SB_API int sb_partition_rows_by_nnz(int64_t m, const int32_t* pos, int parts, int64_t* bounds,
                                    void* stream);

/* --------------------------------------------------------------------------------------------
 * CSR x dense SpMM, fp32, with optional fused bias and ReLU:
 *     C[i, 0:k] = act( bias[0:k] + sum_p val[p] * B[crd[p], 0:k] ),  p in [pos[i], pos[i+1])
 * Rows without entries give act(bias) (zeros when bias is NULL).
 * Replaces: spmm_csr_float_v2 csrc/spmm.h:2007-2089, spmm_csr_typed<float> csrc/spmm.h:91-150,
 *           spmm_csr_bias_act<float,relu> csrc/spmm.h:28-89 (bias != NULL; relu = 0/1), and the
 *           compiler-emitted SpMM loop (src/scorch/compiler/cin_lowerer.py:3616-3667).
 * `plan` may be NULL (every row is then handled by one warp).  `plan_segments` is the number of
 * heavy segments to launch for: the exact count from sb_csr_plan_counts(), or -1 for the
 * worst-case bound.  `scratch` must hold sb_spmm_csr_scratch_bytes(plan_segments or bound, k).
 * ldb/ldc are in elements; B, C, bias must be 16-byte aligned and ldb, ldc multiples of 4 for
 * the vector path (other layouts take a scalar path).  `batch` independent products with the
 * same sparsity structure: val/B/C advance by their strides (elements) per batch item;
 * stride_val may be 0 to share the values.
 * -------------------------------------------------------------------------------------------- */
SB_API size_t sb_spmm_csr_scratch_bytes(int64_t segments, int64_t k, int64_t batch);
SB_API int sb_spmm_csr_f32(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                           const int32_t* crd, const float* val, const float* B, int64_t ldb,
                           const float* bias, int relu, float* C, int64_t ldc, int64_t batch,
                           int64_t stride_val, int64_t stride_b, int64_t stride_c,
                           const void* plan, int64_t plan_segments, void* scratch,
                           size_t scratch_bytes, void* stream);

/* Accumulating form:  C[i, 0:k] = act( bias + C[i, 0:k] + sum_p ... ), same arguments.  A product
 * whose dense operand arrives in pieces (row chunks of B, each with the matrix entries whose
 * columns fall in it) is the first piece through sb_spmm_csr_f32 and the others through this
 * call, bias / ReLU on the last one only.  Vector layout only (SB_ERR_UNSUPPORTED otherwise).
 * Replaces: the same loops as sb_spmm_csr_f32; spmm_csr_typed (csrc/spmm.h:117-139) and the
 *           compiler-emitted loop accumulate straight into the output array in the same way. */
SB_API int sb_spmm_csr_acc_f32(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                               const int32_t* crd, const float* val, const float* B, int64_t ldb,
                               const float* bias, int relu, float* C, int64_t ldc, int64_t batch,
                               int64_t stride_val, int64_t stride_b, int64_t stride_c,
                               const void* plan, int64_t plan_segments, void* scratch,
                               size_t scratch_bytes, void* stream);

/* Wide dense operands (k >= 512, one matrix, no heavy rows) have a second kernel: operand rows
 * staged through shared memory by 1-D bulk copies (cp.async.bulk + mbarrier) instead of gathers
 * through L1 and registers.  sb_spmm_wide_select(1 | 0) picks the bulk-copy / the gather kernel
 * for later sb_spmm_csr_f32 calls of this process and returns the previous choice (any other
 * argument only queries); the first choice comes from the environment variable
 * SCORCH_B200_SPMM_WIDE = "tma" | "gather", else it is the one measured faster on B200.  All waits
 * in that kernel are bounded; sb_spmm_wide_status() (synchronises) returns 0, or 1 / 2 when a
 * producer / consumer wait ever gave up, or -1 when the status could not be read.
 * sb_probe_l2_gather launches a measurement kernel: `warps` warps (multiple of 8) each read
 * `gathers_per_warp` (multiple of 4) pseudo-random 1 KB rows of the `rows` x 256 fp32 `panel`
 * (rows < 2^24) — the load pattern of such a product with nothing else on the critical path;
 * timed by the caller, it gives the L2 gather rate a wide SpMM can at best reach.  `out`: one
 * float per warp.  No reference counterpart (measurement aid). */
SB_API int sb_spmm_wide_select(int mode);
SB_API int sb_spmm_wide_status(void);
SB_API int sb_probe_l2_gather(const float* panel, int64_t rows, int64_t gathers_per_warp, int64_t warps,
                              float* out, void* stream);

/* Same product for the other registry dtypes (SB_F64, SB_I32, SB_I64; SB_F32 also accepted).
 * Integer products wrap like the reference's C++ arithmetic.
 * Replaces: prebuilt_spmm_csr_{f64,i32,i64}, spmm_csr_double (csrc/ops.cpp:91-116). */
SB_API int sb_spmm_csr_typed(int dtype, int64_t m, int64_t n, int64_t k, int64_t nnz,
                             const int32_t* pos, const int32_t* crd, const void* val,
                             const void* B, int64_t ldb, void* C, int64_t ldc, void* stream);

/* --------------------------------------------------------------------------------------------
 * CSR SpMV: y[i] = sum_p val[p] * x[crd[p]].  Every y[i] is written.
 * Replaces: spmv_csr<T> csrc/kernels.h:12-49 (prebuilt_spmv_csr_{f32,f64,i32,i64}) and the
 *           compiler-emitted loop of scorch.ops.spmv (src/scorch/ops.py:48-136).
 * The fp32 entry cuts the entry arrays into tiles (balanced by stored entries, so power-law rows
 * need no special case) and takes a scratch of sb_spmv_csr_scratch_bytes(nnz) for the partial
 * sums of rows cut by tile borders; they are added in tile order (bitwise reproducible).
 * -------------------------------------------------------------------------------------------- */
SB_API size_t sb_spmv_csr_scratch_bytes(int64_t nnz);
SB_API int sb_spmv_csr_f32(int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                           const int32_t* crd, const float* val, const float* x, float* y,
                           void* scratch, size_t scratch_bytes, void* stream);
SB_API int sb_spmv_csr_typed(int dtype, int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                             const int32_t* crd, const void* val, const void* x, void* y,
                             void* stream);

/* SpMV that allocates nothing and asks the caller for no workspace.  (No counterpart in the
 * reference: its kernels malloc freely on the host.)  For callers that cannot call cudaMalloc —
 * a plugin living inside another runtime's device-memory arena, or a service that must not touch
 * the allocator after start-up.  Same result as sb_spmv_csr_f32; the scratch for the partial sums
 * lives in an array of SB_STATIC_SCRATCH_BYTES that is part of the library image, so each GPU
 * that loads the library holds that much memory until the process exits.
 *   - nnz above SB_STATIC_SPMV_MAX_NNZ is rejected with SB_ERR_UNSUPPORTED.
 *   - The first call on a device resolves the array's device address and keeps it for the life
 *     of the process; make that call outside of any stream capture, and do not use this entry
 *     again after a cudaDeviceReset in the same process (the kept address is then stale).
 *   - All calls share the array: calls that overlap on one GPU (other streams, other threads)
 *     race.  Serialise them, or use sb_spmv_csr_f32 with buffers of your own. */
#define SB_STATIC_SPMV_MAX_NNZ (1LL << 26)
#define SB_STATIC_SCRATCH_BYTES (512 << 10)
SB_API int sb_spmv_csr_f32_static(int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                                  const int32_t* crd, const float* val, const float* x, float* y,
                                  void* stream);

/* --------------------------------------------------------------------------------------------
 * SDDMM: out_val[p] = mask_val[p] * dot(Q[i_p, 0:d], K[j_p, 0:d]) for every stored (i_p, j_p) of
 * the mask, in the mask's entry order.  mask_val may be NULL (all ones).  K is (n, d) row-major,
 * i.e. the "ij,ik,jk->ij" operand; for "ij,ik,kj->ij" the reference transposes K first
 * (src/scorch/ops.py:534-540) and so does the host shim.
 * CSR mask  — replaces the compiler-emitted scalar-accumulator loop (generator:
 *             src/scorch/ops.py:638-664, src/scorch/compiler/iter_lattice.py:1011-1098,
 *             src/scorch/compiler/cin_lowerer.py:2286-2326); like it, writes fresh int32
 *             coordinate arrays out_row/out_col when they are non-NULL.
 * COO mask  — replaces sddmm_coo_float_prebuilt csrc/kernels.h:508-570 (output shares the
 *             input's coordinate arrays, so none are written).
 * `batch` independent (Q, K) pairs share the mask: Q/K/out_val advance by their strides
 * (elements); mask_val is shared.
 * -------------------------------------------------------------------------------------------- */
SB_API int sb_sddmm_csr_f32(int64_t m, int64_t n, int64_t d, int64_t nnz, const int32_t* pos,
                            const int32_t* crd, const float* mask_val, const float* Q,
                            int64_t ldq, const float* K, int64_t ldk, float* out_val,
                            int32_t* out_row, int32_t* out_col, int64_t batch, int64_t stride_q,
                            int64_t stride_k, int64_t stride_out, void* stream);
SB_API int sb_sddmm_coo_f32(int64_t m, int64_t n, int64_t d, int64_t nnz, const int32_t* row,
                            const int32_t* col, const float* mask_val, const float* Q,
                            int64_t ldq, const float* K, int64_t ldk, float* out_val,
                            int64_t batch, int64_t stride_q, int64_t stride_k,
                            int64_t stride_out, void* stream);

/* --------------------------------------------------------------------------------------------
 * Dense-block path (tensor cores) for patterns that contain dense aligned 16x16 blocks, e.g.
 * banded attention masks.  A block plan splits the pattern once into its fully stored 16x16
 * blocks and a CSR list of the remaining entries; the blocked SDDMM / SpMM run a TF32x3
 * tensor-core kernel (fp32-level accuracy) over the blocks and the gather kernels over the rest.
 * Results are identical in layout to the unblocked entry points (same entry order, same C).
 * No counterpart in the reference: it has no block level type (src/scorch/format.py:7-11).
 *   sb_block_plan_build : synchronises; returns the number of dense blocks and of remaining
 *                         entries (blocks*256 + rem_nnz == nnz), which the blocked calls take back.
 *   sb_sddmm_csr_blocked_f32 : d in {16, 32, 64, 128}; Q/K 16-byte aligned, pitches % 4 == 0;
 *                              writes values only (no coordinate arrays).
 *   sb_spmm_csr_blocked_f32  : k in {32, 64, 128}; for matrices without heavy rows.
 * -------------------------------------------------------------------------------------------- */
SB_API size_t sb_block_plan_bytes(int64_t m, int64_t nnz);
SB_API int sb_block_plan_build(int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                               const int32_t* crd, void* plan, size_t plan_bytes,
                               int64_t* blocks_host, int64_t* rem_nnz_host, void* stream);
SB_API int sb_sddmm_csr_blocked_f32(int64_t m, int64_t n, int64_t d, int64_t nnz,
                                    const int32_t* pos, const int32_t* crd, const float* mask_val,
                                    const float* Q, int64_t ldq, const float* K, int64_t ldk,
                                    float* out_val, int64_t batch, int64_t stride_q,
                                    int64_t stride_k, int64_t stride_out, const void* block_plan,
                                    int64_t blocks, int64_t rem_nnz, void* stream);
SB_API int sb_spmm_csr_blocked_f32(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                                   const int32_t* crd, const float* val, const float* B,
                                   int64_t ldb, const float* bias, int relu, float* C, int64_t ldc,
                                   int64_t batch, int64_t stride_val, int64_t stride_b,
                                   int64_t stride_c, const void* block_plan, int64_t blocks,
                                   int64_t rem_nnz, void* stream);

/* --------------------------------------------------------------------------------------------
 * Row softmax over the stored entries of a CSR matrix: out[p] = exp(scale*v[p] - max_row) / sum.
 * Rows without entries are untouched.  in == out is allowed.
 * Replaces: the caller-side torch scatter code between SDDMM and SpMM,
 *           bench/bench_sparse_transformer.py:277-297 (scale = 1) and its `values * scale`
 *           pre-multiplication (bench/bench_sparse_transformer.py:363-366).
 * -------------------------------------------------------------------------------------------- */
SB_API int sb_csr_row_softmax_f32(int64_t m, int64_t nnz, const int32_t* pos, const float* in,
                                  float* out, float scale, int64_t batch, int64_t stride,
                                  void* stream);

/* --------------------------------------------------------------------------------------------
 * Sparse attention over a CSR mask, scores never written out:
 *   O = softmax_rows(scale * mask_val .* (Q K^T) on the stored entries) V      per batch item.
 * Replaces: the operator sequence of the reference's sparse-transformer caller,
 *           bench/bench_sparse_transformer.py:304-382 (SDDMM, `values * scale`, row softmax over
 *           the stored entries, SpMM with V, per head), i.e. sb_sddmm_csr_f32 ->
 *           sb_csr_row_softmax_f32 -> sb_spmm_csr_f32 in one call.  Rows without stored entries
 *           give zero rows of O.
 * An attention plan splits the mask once into the aligned 16x16 blocks that hold at least
 * SB_ATTN_MIN_BLOCK_ENTRIES stored entries (with a mask of the stored columns per row) and a
 * CSR list of the remaining (scattered) entries.  A call runs two kernels: a gather kernel over
 * the scattered entries that keeps a running row softmax and leaves, per row, the unnormalised
 * output in O and (maximum, sum) in `scratch`; then the block kernel, which continues from those
 * on the tensor cores (TF32x3, fp32-level accuracy) over the row's blocks and writes O / sum.
 *   sb_attn_plan_build   : synchronises; returns the number of blocks and of remaining entries,
 *                          which the attention call takes back.  A mask without blocks is valid
 *                          (everything is "remaining").
 *   sb_sparse_attention_csr_f32 : d (head dimension of Q, K and V) in {32, 64}; Q/K/V 32-byte
 *                          aligned with row pitches and batch strides multiples of 8, O 16-byte
 *                          aligned with pitch and stride multiples of 4; scratch of
 *                          sb_sparse_attention_scratch_bytes(m, rem_nnz, batch) bytes.
 *                          `stages` is SB_ATTN_ALL_STAGES, or one of the two kernels for callers
 *                          that time or schedule them one by one: they must run in the order
 *                          scattered entries -> blocks, with the same arguments, O and scratch.
 * -------------------------------------------------------------------------------------------- */
#define SB_ATTN_MIN_BLOCK_ENTRIES 64
#define SB_ATTN_STAGE_SCATTERED 1
#define SB_ATTN_STAGE_BLOCKS 2
#define SB_ATTN_ALL_STAGES 3
SB_API size_t sb_attn_plan_bytes(int64_t m, int64_t nnz);
SB_API int sb_attn_plan_build(int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                              const int32_t* crd, void* plan, size_t plan_bytes,
                              int64_t* blocks_host, int64_t* rem_nnz_host, void* stream);
SB_API size_t sb_sparse_attention_scratch_bytes(int64_t m, int64_t rem_nnz, int64_t batch);
SB_API int sb_sparse_attention_csr_f32(int64_t m, int64_t n, int64_t d, int64_t nnz,
                                       const int32_t* pos, const int32_t* crd,
                                       const float* mask_val, const float* Q, int64_t ldq,
                                       const float* K, int64_t ldk, const float* V, int64_t ldv,
                                       float scale, float* O, int64_t ldo, int64_t batch,
                                       int64_t stride_q, int64_t stride_k, int64_t stride_v,
                                       int64_t stride_o, const void* attn_plan, int64_t blocks,
                                       int64_t rem_nnz, void* scratch, size_t scratch_bytes,
                                       int stages, void* stream);

/* --------------------------------------------------------------------------------------------
 * CSR input validation (no counterpart in the reference, whose loops trust their inputs like the
 * kernels here: csrc/spmm.h:2035-2077 never checks crd against the operand's height).  Finds the
 * first entry that would make a kernel of this library read or write outside its arrays, reading
 * nothing outside pos[0..m] and crd[0..nnz): row pointers first, then — only if those are valid —
 * the columns of every row.  report_host[0] = one of the codes below (0: valid), [1] = row,
 * [2] = entry index (column checks), [3] = the offending value; the smallest (row, entry) is
 * reported whatever the scheduling.  sorted_unique != 0 also requires strictly ascending columns
 * per row (SpGEMM, the element-wise kernels, the attention plans and the transposes rely on it).
 * Synchronises the stream.  `ws`: sb_csr_validate_workspace_bytes() bytes, 16-byte aligned.
 * The Python layer runs it on every CSR operand when SCORCH_B200_VALIDATE=1.
 * -------------------------------------------------------------------------------------------- */
#define SB_CSR_BAD_FIRST_POS 1
#define SB_CSR_BAD_LAST_POS 2
#define SB_CSR_POS_OUT_OF_RANGE 3
#define SB_CSR_POS_DECREASES 4
#define SB_CSR_COLUMN_OUT_OF_RANGE 5
#define SB_CSR_COLUMNS_NOT_ASCENDING 6
SB_API size_t sb_csr_validate_workspace_bytes(void);
SB_API int sb_csr_validate(int64_t m, int64_t n, int64_t nnz, const int32_t* pos, const int32_t* crd,
                           int sorted_unique, int32_t* report_host, void* ws, size_t ws_bytes,
                           void* stream);

/* --------------------------------------------------------------------------------------------
 * The same sparse attention for banded masks on the tcgen05 tensor cores (head dimension 64).
 * Replaces: the same operator sequence (bench/bench_sparse_transformer.py:304-382).
 * A band plan cuts the mask rows into tiles of SB_ATTN_BAND_ROWS rows and gives tile t the window
 * of SB_ATTN_BAND_COLS columns that starts at clamp(t * ROWS - (COLS - ROWS) / 2, 0, n - COLS);
 * per row it holds the stored columns inside the window as bits and the index of the row's first
 * entry there; entries outside the windows go to a CSR remainder list (the scattered entries).
 * Columns must be ascending and unique per row (the reference's CSR).
 *   sb_attn_band_plan_build : synchronises; *inside_host = entries inside the windows,
 *                          *rem_nnz_host = entries outside (inside + outside = nnz).  Worth using
 *                          when most entries are inside; any mask gives correct results.
 *   sb_sparse_attention_band_f32 : same arguments, alignment rules, scratch and stages as
 *                          sb_sparse_attention_csr_f32; the scattered entries first (the same
 *                          gather kernel), then one CTA per (tile, batch item): S = Q K^T and
 *                          O += P V as tcgen05.mma kind::tf32 with the TF32x3 split, S, P and O in
 *                          tensor memory.  Every wait on the tensor cores is bounded; when one runs
 *                          out the CTA gives up and sb_attn_band_status (synchronises the device)
 *                          returns non-zero afterwards, else 0.
 *   sb_attn_band_probe   : self-test of the tensor-core path on one tile with every window column
 *                          counted as stored and scale 1: `raw_scores` receives the 128 x 384
 *                          products Q K^T; `tmem_image` (may be null) the tile's 128 x 512
 *                          tensor-memory cells at the end: columns [0,384) the hi parts of
 *                          P = exp2(log2(e) S - row max), [384,448) the unnormalised O = P V,
 *                          [448,512) the lo parts of P's last 64 columns; `phase_clocks` (may be
 *                          null, 36 values; the scores are then not copied out) the SM clock at the kernel's phase boundaries (scores
 *                          staged and issued piece by piece, row maxima, the six rounds of
 *                          O += P V, end).  O is not written.
 * -------------------------------------------------------------------------------------------- */
#define SB_ATTN_BAND_ROWS 128
#define SB_ATTN_BAND_COLS 384
SB_API size_t sb_attn_band_plan_bytes(int64_t m, int64_t nnz);
SB_API int sb_attn_band_plan_build(int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                                   const int32_t* crd, void* plan, size_t plan_bytes,
                                   int64_t* inside_host, int64_t* rem_nnz_host, void* stream);
SB_API int sb_sparse_attention_band_f32(int64_t m, int64_t n, int64_t d, int64_t nnz,
                                        const int32_t* pos, const int32_t* crd,
                                        const float* mask_val, const float* Q, int64_t ldq,
                                        const float* K, int64_t ldk, const float* V, int64_t ldv,
                                        float scale, float* O, int64_t ldo, int64_t batch,
                                        int64_t stride_q, int64_t stride_k, int64_t stride_v,
                                        int64_t stride_o, const void* band_plan, int64_t rem_nnz,
                                        void* scratch, size_t scratch_bytes, int stages,
                                        void* stream);
SB_API int sb_attn_band_probe(int64_t m, int64_t n, int64_t d, int64_t tile, const float* Q,
                              int64_t ldq, const float* K, int64_t ldk, const float* V, int64_t ldv,
                              float* raw_scores, float* tmem_image, long long* phase_clocks,
                              void* stream);
SB_API int sb_attn_band_status(void);

/* --------------------------------------------------------------------------------------------
 * CSR x CSR SpGEMM (Gustavson), two phases.  Output rows have strictly ascending, unique
 * columns; the structure is the symbolic union (entries whose products cancel are kept).
 * Replaces: spmspm_csr<T> csrc/kernels.h:51-202 (prebuilt_spmspm_csr_{f32,f64,i32,i64},
 *           spmspm_csr_float) and the compiler-emitted two-phase code
 *           (src/scorch/compiler/cin_lowerer.py:2683+).
 *   symbolic: fills Cpos[0..m] (int32) and returns the total in *total_nnz_host; SYNCHRONISES the
 *             stream (the caller must size Ccrd/Cval).  SB_ERR_OVERFLOW when total >= 2^31.
 *   numeric : fills Ccrd/Cval for the Cpos of the symbolic call; `ws` must be the SAME,
 *             unmodified workspace (it carries the row bins).
 * A has m rows; B has `kb` rows and n columns.
 * -------------------------------------------------------------------------------------------- */
SB_API size_t sb_spgemm_workspace_bytes(int64_t m, int64_t n, int dtype);
SB_API int sb_spgemm_symbolic(int64_t m, int64_t kb, int64_t n, const int32_t* Apos,
                              const int32_t* Acrd, const int32_t* Bpos, const int32_t* Bcrd,
                              int32_t* Cpos, int64_t* total_nnz_host, void* ws, size_t ws_bytes,
                              void* stream);
SB_API int sb_spgemm_numeric(int dtype, int64_t m, int64_t kb, int64_t n, const int32_t* Apos,
                             const int32_t* Acrd, const void* Aval, const int32_t* Bpos,
                             const int32_t* Bcrd, const void* Bval, const int32_t* Cpos,
                             int32_t* Ccrd, void* Cval, void* ws, size_t ws_bytes, void* stream);

/* --------------------------------------------------------------------------------------------
 * Element-wise product / sum of two CSR matrices of the same shape, CSR out with ascending columns:
 *   SB_EWISE_MUL  C = A .* B, stored where both operands store an entry;
 *   SB_EWISE_ADD  C = A + B,  stored where either operand stores an entry.
 * The structure is symbolic (a result that happens to be zero stays stored).  Two calls, like
 * SpGEMM: _symbolic writes Cpos[0..m] and returns the number of stored entries (synchronises), the
 * caller allocates Ccrd / Cval, _numeric fills them.  `ws`: sb_csr_ewise_workspace_bytes(m) bytes.
 * Replaces: the loops the reference's compiler emits for einsum("ij,ij->ij", A, B) and A + B over
 *           compressed operands (src/scorch/ops.py:375-819; covered by
 *           tests/test_scorch/test_kernels_comprehensive.py:119-200).
 * -------------------------------------------------------------------------------------------- */
enum { SB_EWISE_MUL = 0, SB_EWISE_ADD = 1 };
SB_API size_t sb_csr_ewise_workspace_bytes(int64_t m);
SB_API int sb_csr_ewise_symbolic(int op, int64_t m, const int32_t* Apos, const int32_t* Acrd,
                                 const int32_t* Bpos, const int32_t* Bcrd, int32_t* Cpos,
                                 int64_t* nnz_host, void* ws, size_t ws_bytes, void* stream);
SB_API int sb_csr_ewise_numeric(int op, int dtype, int64_t m, const int32_t* Apos, const int32_t* Acrd,
                                const void* Aval, const int32_t* Bpos, const int32_t* Bcrd,
                                const void* Bval, const int32_t* Cpos, int32_t* Ccrd, void* Cval,
                                void* stream);

/* --------------------------------------------------------------------------------------------
 * Format plumbing on the device (the reference does these with torch ops before dispatch,
 * src/scorch/stensor.py:785-896): sorted COO rows -> CSR row pointers, CSR row pointers -> row
 * ids.
 * -------------------------------------------------------------------------------------------- */
SB_API int sb_coo_rows_to_csr_pos(int64_t m, int64_t nnz, const int32_t* row_sorted,
                                  int32_t* pos, void* stream);
SB_API int sb_csr_pos_to_coo_rows(int64_t m, int64_t nnz, const int32_t* pos, int32_t* row,
                                  void* stream);

/* --------------------------------------------------------------------------------------------
 * More format plumbing, so that whole pipelines stay on the device.
 *   dense -> CSR : the non-zero entries of a row-major fp32 matrix (what the reference's callers
 *                  get from torch's to_sparse_csr(), bench/bench_sparse_autoencoder.py:233,261;
 *                  -0.0 is dropped, NaN kept).  Two calls because the output size is data
 *                  dependent: _count writes pos[0..m] and returns the number of stored entries
 *                  (synchronises), the caller allocates crd / val, _fill writes them in ascending
 *                  column order.  `ws`: sb_dense_to_csr_workspace_bytes(m) bytes.
 *   sb_csr_sym_normalize_f32 : val[p] = d_i^-1/2 * d_j^-1/2 for the entry p = (i, j) of a square
 *                  pattern, d = stored entries per row (pattern of A + I; rows without entries
 *                  give 0).  Replaces: compute_normalized_adj, bench/bench_gcn.py:233-267.
 * -------------------------------------------------------------------------------------------- */
SB_API size_t sb_dense_to_csr_workspace_bytes(int64_t m);
SB_API int sb_dense_to_csr_count(int64_t m, int64_t n, const float* A, int64_t lda, int32_t* pos,
                                 int64_t* nnz_host, void* ws, size_t ws_bytes, void* stream);
SB_API int sb_dense_to_csr_fill(int64_t m, int64_t n, const float* A, int64_t lda,
                                const int32_t* pos, int32_t* crd, float* val, void* stream);
/* CSR transpose: (tpos, tcrd, tval) = CSR of the transpose of the m x n matrix (pos, crd, val), i.e.
 * its CSC form; output rows hold their entries in ascending source-row order.  `val` / `tval` may
 * both be NULL (pattern only); otherwise `dtype` (SB_F32 ... SB_I64) gives their element type.
 * `ws`: sb_csr_transpose_workspace_bytes(n, nnz) bytes, 16-byte aligned.  Asynchronous.
 * Replaces: the torch-op fast path of STensor.change_mode_order for 2-D compressed operands,
 *           src/scorch/stensor.py:785-896, which runs before every prebuilt dispatch on an operand
 *           stored in the other mode order (src/scorch/ops.py:299-303,333-346). */
SB_API size_t sb_csr_transpose_workspace_bytes(int64_t n, int64_t nnz);
SB_API int sb_csr_transpose(int dtype, int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                            const int32_t* crd, const void* val, int32_t* tpos, int32_t* tcrd,
                            void* tval, void* ws, size_t ws_bytes, void* stream);

/* Per-row top-k of a dense row-major fp32 matrix, written as CSR with exactly k entries per row:
 * pos[i] = i*k, the columns of the k largest values of row i in ascending order (ties between
 * equal values go to the lower column), val = the kept values, clamped at zero when `relu` is
 * set.  This is how the activations of benchmark configuration 3 are defined (a sparse
 * autoencoder keeps the k largest pre-activations per sample); the reference itself has no such
 * operator, its callers build CSR operands with torch (bench/bench_sparse_autoencoder.py:233,261). */
SB_API int sb_topk_rows_to_csr_f32(int64_t m, int64_t n, int64_t k, const float* X, int64_t ldx,
                                   int relu, int32_t* pos, int32_t* crd, float* val, void* stream);

SB_API int sb_csr_sym_normalize_f32(int64_t m, int64_t nnz, const int32_t* pos, const int32_t* crd,
                                    float* val, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SCORCH_B200_H_ */
