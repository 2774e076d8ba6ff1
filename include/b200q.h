/* b200q — C ABI of the B200 (sm_100a) low-precision linear path.
 *
 * One shared library, plain pointers and sizes.  Every entry point
 *   - returns an int status (0 = ok, < 0 = B200Q_ERR_*), never throws, aborts or traps;
 *   - is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the legacy stream);
 *   - works on buffers the caller owns, on the current device;
 *   - allocates nothing;
 *   - may be called from several host threads at once (no shared host state), with the two
 *     b200q_debug_* hooks at the end of this file as the only exception.
 *
 * The path these replace is the quantized-linear path of gongyisheng/pretrain, which is
 * Python calling torch library kernels; each entry names the reference lines it stands for.
 * All matrices are row-major.  "Contraction dimension" = the dimension the GEMM sums over;
 * quantization scales always run along it (src/quant/fp8.py:52-54).
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200Q_OK = 0,
  B200Q_ERR_INVALID_ARG = -1,   /* null pointer, negative size, unknown enum value */
  B200Q_ERR_SHAPE = -2,         /* size not a multiple the kernel needs (see each entry) */
  B200Q_ERR_ALIGNMENT = -3,     /* pointer or pitch not 16-byte aligned */
  B200Q_ERR_CUDA = -4,          /* a CUDA runtime / driver call failed (b200q_last_cuda_error) */
  B200Q_ERR_NOT_SM100 = -5,     /* current device is not compute capability 10.x */
  B200Q_ERR_DEVICE_TIMEOUT = -6 /* a bounded device-side wait gave up (b200q_device_status) */
};

enum { B200Q_E4M3 = 0, B200Q_E5M2 = 1 };
enum { B200Q_SF_NATURAL = 0, B200Q_SF_SWIZZLE_128x4 = 1 };

const char* b200q_status_string(int status);
/* cudaError_t of the last failing CUDA call made by this library on this thread (0 if none). */
int b200q_last_cuda_error(void);
/* Reads (synchronously) and clears the device-side status word that kernels set when a
 * bounded wait expires: 0 = clean.  Returns B200Q_ERR_DEVICE_TIMEOUT if it was set. */
int b200q_device_status(void);

/* Bytes of a scale-factor buffer for `outer` rows and `nblk` blocks per row. */
int64_t b200q_sf_bytes(int64_t outer, int64_t nblk, int sf_layout);

/* ---- quantizers -------------------------------------------------------------------------
 * x is bf16 [rows, cols] with row pitch `ld` elements (ld % 8 == 0, base 16-byte aligned).
 * axis = 1: scales run along the columns (each row is quantized on its own); codes come out
 *           as [rows, cols].
 * axis = 0: scales run along the rows (per column); codes come out TRANSPOSED as
 *           [cols, rows], so that the contraction dimension is contiguous for the GEMM.
 */

/* max |x| over the whole matrix -> *amax (fp32, device).  The call zeroes *amax first.
 * Stands for `x.abs().max()` of quantize_fp8(dim=None), src/quant/fp8.py:26-27. */
int b200q_amax(const void* x, int64_t rows, int64_t cols, int64_t ld, float* amax, void* stream);

/* quantize_fp8(x, dtype, dim) of src/quant/fp8.py:16-32 with dim=-1 (axis=1) or dim=0
 * (axis=0): scale = max(amax/qmax, 1e-12), codes = cast(clamp(x/scale)).  `scales` is fp32,
 * one per row (axis=1) or per column (axis=0).  cols % 8 == 0; for axis=0 rows % 16 == 0. */
int b200q_quantize_fp8(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis, int fmt,
                       void* codes, float* scales, void* stream);

/* quantize_fp8(x, dtype, dim=None): one scale for the tensor from *tensor_amax (device,
 * e.g. from b200q_amax); writes it to *scale_out (device).  transpose != 0 writes codes
 * as [cols, rows]. */
int b200q_quantize_fp8_tensorwise(const void* x, int64_t rows, int64_t cols, int64_t ld, int transpose,
                                  int fmt, const float* tensor_amax, void* codes, float* scale_out,
                                  void* stream);

/* Both per-row and per-column FP8 copies of one tensor, i.e. quantize_fp8(x, dtype, dim=-1) and
 * quantize_fp8(x, dtype, dim=0) of src/quant/fp8.py:16-32 (a linear layer's step needs both of x, w
 * and the output gradient: src/quant/linear.py:74,98,102), in two reads of x instead of three: the
 * row-wise pass also reduces |x| down the columns, so the column direction needs no amax pass of
 * its own.  Outputs as b200q_quantize_fp8 with axis = 1 (codes_row [rows, cols], scales_row[rows])
 * and axis = 0 (codes_col [cols, rows], scales_col[cols]), bit for bit.  workspace:
 * b200q_quantize_fp8_both_workspace_bytes(cols) bytes.  rows % 16 == 0, cols <= 8192. */
int64_t b200q_quantize_fp8_both_workspace_bytes(int64_t cols);
int b200q_quantize_fp8_both(const void* x, int64_t rows, int64_t cols, int64_t ld, int fmt,
                            void* codes_row, float* scales_row, void* codes_col, float* scales_col,
                            void* workspace, void* stream);

/* quantize_int8(x, qmax, dim) of src/quant/int8.py:9-19, the int8 series (int8 .. int4 in an int8
 * container; qmax = 127, 63, 31, 15, 7 as in src/quant/utils.py:19): scale = max(amax/qmax, 1e-12),
 * codes = clamp(round_half_even(x/scale), +-qmax).  Same axis / shape rules as b200q_quantize_fp8 and
 * b200q_quantize_fp8_tensorwise; codes are int8. */
int b200q_quantize_int8(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis, int qmax,
                        void* codes, float* scales, void* stream);
int b200q_quantize_int8_tensorwise(const void* x, int64_t rows, int64_t cols, int64_t ld, int transpose,
                                   int qmax, const float* tensor_amax, void* codes, float* scale_out,
                                   void* stream);

/* MXFP8: 32-element blocks along the contraction dimension, fp8 codes, one E8M0 byte per
 * block (2^e = smallest power of two >= max(amax/qmax, 1e-12)).  No counterpart in the
 * reference yet (TODO at src/quant/__init__.py:26); extends src/quant/fp8.py:16-32.
 * Contraction length % 32 == 0.  `sf` holds b200q_sf_bytes(outer, C/32, sf_layout) bytes;
 * pad bytes of the swizzled layout are written as zero. */
int b200q_quantize_mxfp8(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis, int fmt,
                         void* codes, void* sf, int sf_layout, void* stream);

/* Both directions of b200q_quantize_mxfp8 from ONE read of x: (codes_row [rows, cols], sf_row) as
 * axis = 1 would give and (codes_col [cols, rows], sf_col) as axis = 0 would give, byte for byte.
 * A linear layer needs both of each tensor: the activation for fprop and wgrad
 * (src/quant/linear.py:74,102), the weight for fprop and dgrad (:74,98), the output gradient for
 * dgrad and wgrad (:98,102); the reference re-reads the bf16 tensor for each.  rows % 32 == 0 and
 * cols % 32 == 0.  4.0625 bytes of traffic per element instead of 2 x 3.03125.
 * num_tiles (device int32, may be NULL): only the first *num_tiles 128-row tiles of x are processed - the rows in use of
 * a padded expert-sorted buffer whose size is an upper bound; outputs belonging to later rows are left untouched. */
int b200q_quantize_mxfp8_dual(const void* x, int64_t rows, int64_t cols, int64_t ld, int fmt,
                              void* codes_row, void* sf_row, void* codes_col, void* sf_col,
                              int sf_layout, const int32_t* num_tiles, void* stream);

/* Row-wise b200q_quantize_mxfp8 (axis = 1) that writes input row r as output row dst_row[r]
 * (codes and scale factors alike); dst_row is a permutation of 0 .. rows-1 in device memory.
 * Used to store gated-MLP weights (src/layers/mlp.py:404-411, expert_gate_up) in the interleaved
 * row order the SwiGLU epilogue reads, without a copy of the bf16 weights. */
int b200q_quantize_mxfp8_rowmap(const void* x, int64_t rows, int64_t cols, int64_t ld, int fmt,
                                const int32_t* dst_row, void* codes, void* sf, int sf_layout,
                                void* stream);

/* Two matrices quantized along their rows by ONE launch (same element format and scale-factor layout): the two weight
 * stacks of an expert FFN, or any two operands of one step; dst_row0 / dst_row1 as in b200q_quantize_mxfp8_rowmap, or
 * NULL for the identity.  Equal to two b200q_quantize_mxfp8(axis = 1) / _rowmap calls bit for bit.  The reference
 * quantizes one tensor per call (src/quant/linear.py:73-80); no counterpart. */
int b200q_quantize_mxfp8_pair(const void* x0, int64_t rows0, int64_t cols0, int64_t ld0, const int32_t* dst_row0,
                              void* codes0, void* sf0, const void* x1, int64_t rows1, int64_t cols1, int64_t ld1,
                              const int32_t* dst_row1, void* codes1, void* sf1, int fmt, int sf_layout, void* stream);

/* NVFP4: 16-element blocks, packed E2M1 codes (element 2i in the low nibble), one E4M3 scale
 * byte per block and one fp32 scale per tensor derived from *tensor_amax (device):
 * s_t = max(amax/2688, 1e-12), written to *tensor_scale_out.  No counterpart in the reference
 * yet (TODOs at src/quant/__init__.py:20,30).  Contraction length % 32 == 0. */
int b200q_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis,
                         const float* tensor_amax, void* codes, void* sf, int sf_layout,
                         float* tensor_scale_out, void* stream);

/* ---- GEMMs: D[M,N] (bf16, pitch ldd) = A[M,K] . B[N,K]^T, fp32 accumulation -------------
 * Both operands have the contraction dimension contiguous ("K-major"), pitch = K codes.
 * Scale-factor buffers are in B200Q_SF_SWIZZLE_128x4 layout.  N % 8 == 0, ldd % 8 == 0.
 */

/* Stands for torch._scaled_mm at src/quant/fp8.py:59-65.  scale_a: per row of A (M values)
 * or one value (a_scale_is_scalar); scale_b: per row of B (N values) or one value.
 * K % 16 == 0. */
int b200q_gemm_fp8(const void* A, int a_fmt, const void* B, int b_fmt, const float* scale_a,
                   int a_scale_is_scalar, const float* scale_b, int b_scale_is_scalar, int64_t M,
                   int64_t N, int64_t K, void* D, int64_t ldd, void* stream);

/* Stands for torch._int_mm and the scaling after it at src/quant/int8.py:49-53:
 * D = bf16((float(A . B^T) * scale_a) * scale_b) with the integer product accumulated exactly in
 * 32 bits (tcgen05.mma kind::i8), so the result equals the reference's bit for bit.  A, B: int8
 * codes; scales as for b200q_gemm_fp8.  K % 16 == 0. */
int b200q_gemm_int8(const void* A, const void* B, const float* scale_a, int a_scale_is_scalar,
                    const float* scale_b, int b_scale_is_scalar, int64_t M, int64_t N, int64_t K,
                    void* D, int64_t ldd, void* stream);

/* Block-scaled MXFP8 GEMM (the `_gemm` seam, src/quant/linear.py:27-56, for MX formats).
 * K % 32 == 0. */
int b200q_gemm_mxfp8(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt,
                     const void* sfB, int64_t M, int64_t N, int64_t K, void* D, int64_t ldd,
                     void* stream);

/* `_gemm(a, b, "mxfp8", "mxfp8", ...)` of src/quant/linear.py:27-56 in ONE call: both bf16 operands quantized to MXFP8
 * along the contraction dimension and multiplied, D (bf16 [M, N], pitch ldd) = A . B^T.  Each operand is given as it
 * lies in memory with the axis its blocks run along, exactly as for b200q_quantize_mxfp8: axis = 1 - a [M, K] (or
 * b [N, K]) with K contiguous; axis = 0 - the operand stored [K, M] (or [K, N]), quantized by the transposing
 * kernel.  When both have K contiguous and the same format, ONE launch quantizes the two; the GEMM is launched
 * behind it with programmatic stream serialization, so its set-up overlaps the quantizer's tail.  Results are
 * bit-identical to b200q_quantize_mxfp8 x 2 + b200q_gemm_mxfp8.  `workspace` (256-byte aligned) holds
 * b200q_linear_mxfp8_workspace_bytes(M, N, K) bytes: the codes and scale factors, which are left there. */
int64_t b200q_linear_mxfp8_workspace_bytes(int64_t M, int64_t N, int64_t K);
int b200q_linear_mxfp8(const void* a, int64_t a_rows, int64_t a_cols, int64_t lda, int a_axis, int a_fmt,
                       const void* b, int64_t b_rows, int64_t b_cols, int64_t ldb, int b_axis, int b_fmt,
                       void* D, int64_t ldd, void* workspace, void* stream);

/* Block-scaled NVFP4 GEMM; D is multiplied by (*tsA) * (*tsB) (device fp32).  K % 32 == 0;
 * A and B hold K/2 bytes per row. */
int b200q_gemm_nvfp4(const void* A, const void* sfA, const void* B, const void* sfB,
                     const float* tsA, const float* tsB, int64_t M, int64_t N, int64_t K, void* D,
                     int64_t ldd, void* stream);

/* Fused GEMM + all-gather of an output sharded by rows across `world` GPUs (new functionality: the
 * reference is single-GPU).  Each call computes this rank's [M, N] block exactly as the plain entry
 * point does and its epilogue stores every block into rows [rank*M, rank*M + M) of EVERY rank's
 * gathered buffer D_all[g] (bf16 [world*M, N], pitch ldd): D_all[rank] is local memory, the others
 * are peer-mapped pointers to the peers' buffers (CUDA IPC or symmetric memory).  Only stores cross
 * NVLink, tile by tile while the main loop runs; nothing is loaded from a peer.  The gathered
 * matrix is complete on a rank once every rank's kernel has finished: synchronize the ranks before
 * reading it.  world <= 8; every rank passes the same M. */
int b200q_gemm_fp8_allgather(const void* A, int a_fmt, const void* B, int b_fmt, const float* scale_a,
                             int a_scale_is_scalar, const float* scale_b, int b_scale_is_scalar,
                             int64_t M, int64_t N, int64_t K, void* const* D_all, int world, int rank,
                             int64_t ldd, void* stream);
int b200q_gemm_mxfp8_allgather(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt,
                               const void* sfB, int64_t M, int64_t N, int64_t K, void* const* D_all,
                               int world, int rank, int64_t ldd, void* stream);
int b200q_gemm_nvfp4_allgather(const void* A, const void* sfA, const void* B, const void* sfB,
                               const float* tsA, const float* tsB, int64_t M, int64_t N, int64_t K,
                               void* const* D_all, int world, int rank, int64_t ldd, void* stream);

/* The same fused GEMM + all-gather with the output leaving as MXFP8 instead of bf16, for the case where the
 * consumer of the gathered matrix is the next block-scaled GEMM (which would quantize the bf16 matrix along its
 * columns first thing, src/quant/linear.py:72-76): every accumulator is rounded to bf16 and then quantized as
 * b200q_quantize_mxfp8(axis = 1, B200Q_E4M3, B200Q_SF_SWIZZLE_128x4) quantizes that bf16 matrix, bit for bit, and
 * what crosses NVLink is 1 code byte per element plus 1 scale byte per 32 - 1.03 bytes instead of 2.
 * C_all[g]: codes [world*M, N] of rank g (pitch ldc bytes, ldc % 16 == 0); SF_all[g]: its scale factors,
 * b200q_sf_bytes(world*M, N/32, B200Q_SF_SWIZZLE_128x4) bytes.  The pair (C_all[g], SF_all[g]) is directly the A
 * operand of b200q_gemm_mxfp8 with K = N.  M % 128 == 0, N % 128 == 0.  world = 1 (C_all = {C}, SF_all = {SF},
 * rank 0) is a plain GEMM with MXFP8 output.  New functionality: the reference is single-GPU. */
int b200q_gemm_mxfp8_allgather_mxfp8(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt,
                                     const void* sfB, int64_t M, int64_t N, int64_t K, void* const* C_all,
                                     void* const* SF_all, int world, int rank, int64_t ldc, void* stream);

/* Fused GEMM + reduce-scatter, first half (new functionality: the data-parallel wgrad the reference, being
 * single-GPU, never needs; src/quant/linear.py:102-109 is the GEMM).  Every rank computes its own [M, N]
 * partial result (e.g. dW from its shard of the tokens); the sum over the ranks is wanted scattered by
 * rows, rank g owning rows [g*M/world, (g+1)*M/world).  The epilogue stores every block (bf16) into THIS
 * rank's slot of the OWNER's staging buffer: stage_all[g] is rank g's buffer, bf16 [world][M/world, N]
 * with pitch ldd (local memory for g == rank, peer-mapped otherwise), slot = sender.  Only stores cross
 * NVLink, tile by tile while the main loop runs.  After the ranks have synchronized, each owner adds
 * its slots with b200q_sum_slots.  world <= 8, M % world == 0, (M / world) % 32 == 0. */
int b200q_gemm_mxfp8_scatter(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt,
                             const void* sfB, int64_t M, int64_t N, int64_t K, void* const* stage_all,
                             int world, int rank, int64_t ldd, void* stream);
/* out[r, c] = bf16(sum_s float(stage[s][r][c])), slots added in order in fp32, one rounding.
 * stage bf16 [slots][rows, cols] pitch ld (slot stride rows * ld); cols % 8 == 0. */
int b200q_sum_slots(const void* stage, int slots, int64_t rows, int64_t cols, int64_t ld, void* out,
                    int64_t ldo, void* stream);

/* ---- MoE: top-k permute, ragged grouped GEMM, SwiGLU, weighted unpermute ------------------
 * Layout used between these calls ("padded expert-sorted"): rows sorted by expert in the
 * reference's order (stable sort of the flattened (token, slot) pairs by expert id,
 * src/layers/mlp.py:447-452), each expert's segment starting on a multiple of 128 rows so
 * that every 128-row GEMM tile belongs to one expert; pad rows are zero.
 */

/* Rows of the padded layout for n_pairs = T*k routed pairs and E experts (upper bound, a
 * multiple of 128), and bytes of the scratch buffer b200q_moe_permute_plan needs. */
int64_t b200q_moe_padded_rows(int64_t n_pairs, int E);
int64_t b200q_moe_plan_workspace_bytes(int64_t n_pairs, int E);

/* Permute plan from the router's choice (src/layers/mlp.py:446-457).  top_idx: int64 [T*k]
 * expert ids, token-major.  Outputs (device): offs int32 [E] cumulative ends of the unpadded
 * segments (the reference's `offs`); padded_offs int32 [E+1] first padded row of each expert;
 * row_of int32 [T*k] padded row of every (token, slot); src_of_row int32 [padded_rows] token
 * of every padded row, -1 for pad rows; tile_expert int32 [padded_rows/128] expert of every
 * 128-row tile, -1 beyond the last; num_tiles int32 [1].  E <= 256.  `workspace` holds
 * b200q_moe_plan_workspace_bytes() bytes of scratch. */
int b200q_moe_permute_plan(const int64_t* top_idx, int64_t n_pairs, int k, int E, int32_t* offs,
                           int32_t* padded_offs, int32_t* row_of, int32_t* src_of_row,
                           int32_t* tile_expert, int32_t* num_tiles, void* workspace, void* stream);

/* b200q_moe_permute_plan without a workspace argument, for callers that cannot allocate
 * device memory when they need the plan: a runtime that carved up all of HBM at start-up and
 * forbids cudaMalloc afterwards (it synchronizes the device and can fail late), or a host in
 * another language that owns only the tensors it passes in.  The scratch is a fixed 1 MiB array
 * inside the library, held by every GPU that loads it until the process exits.  It has no
 * counterpart in the reference.  Limit: ceil(n_pairs / 1024) * E <= 262144, otherwise
 * B200Q_ERR_SHAPE.  The first call on a device looks up the array's device address; make that
 * call before any stream capture.  All calls on a device share the array: calls that overlap
 * on the GPU race on it.  Outputs are identical to b200q_moe_permute_plan's. */
int b200q_moe_permute_plan_static(const int64_t* top_idx, int64_t n_pairs, int k, int E, int32_t* offs,
                                  int32_t* padded_offs, int32_t* row_of, int32_t* src_of_row,
                                  int32_t* tile_expert, int32_t* num_tiles, void* stream);

/* The same plan outputs for rows that are ALREADY expert-sorted (the input convention of
 * grouped_mlp, src/layers/mlp.py:55-72): offs int32 [E] cumulative ends; src_of_row maps a
 * padded row to its row in the sorted input. */
int b200q_moe_pad_plan(const int32_t* offs, int E, int64_t n_rows, int32_t* padded_offs,
                       int32_t* src_of_row, int32_t* tile_expert, int32_t* num_tiles, void* stream);

/* Gather rows into the padded layout: out row r = x[src_of_row[r]] (zero when -1), for the
 * rows of the first *num_tiles tiles.  x bf16 [*, D] pitch ld; D % 32 == 0.
 * quantize = 0: bf16 copy into `out` (the reference's x_flat[token_ids_sorted],
 * src/layers/mlp.py:458).  quantize = 1: MXFP8 codes (fmt) into `out` and E8M0 scale factors,
 * swizzled, into `sf`. */
int b200q_moe_gather(const void* x, int64_t D, int64_t ld, const int32_t* src_of_row,
                     const int32_t* num_tiles, int64_t padded_rows, int quantize, int fmt, void* out,
                     void* sf, void* stream);

/* Ragged grouped GEMM (stands for torch._grouped_mm at src/layers/mlp.py:89,97):
 * D[r, :] = A[r, :] . B[e(r)]^T for the padded layout.  A: MXFP8 codes [padded_rows, K] + sfA;
 * B: codes [E*N, K] + sfB (each expert's [N, K] weight quantized along K, N % 128 == 0);
 * D: bf16 [padded_rows, N].  Only the first *num_tiles row tiles are computed. */
int b200q_grouped_gemm_mxfp8(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt,
                             const void* sfB, const int32_t* tile_expert, const int32_t* num_tiles,
                             int64_t padded_rows, int E, int64_t N, int64_t K, void* D, int64_t ldd,
                             void* stream);

/* The two backward GEMMs of a grouped (per-expert) linear layer y_e = x_e . W_e^T over the padded
 * expert-sorted layout; the reference gets them from autograd through torch._grouped_mm
 * (src/layers/mlp.py:89,97).  MXFP8 operands, bf16 outputs, K % 128 == 0.
 *
 * dgrad: D[r, :] = A[r, :] . Bt[:, e(r)*K : (e(r)+1)*K]^T.  A: codes [padded_rows, K] + sfA (the
 * output gradient, quantized along its columns); Bt: codes [N, E*K] + sfBt = the weight stack
 * [E*K, N] quantized along axis 0 (b200q_quantize_mxfp8 transposes it as a whole, which puts expert
 * e's operand at column offset e*K).  D: bf16 [padded_rows, N].
 *
 * wgrad: D[e*M + m, n] = sum over the rows r of expert e of At[m, r] * Bt[n, r].  At: codes
 * [M, padded_rows] + sfAt and Bt: codes [N, padded_rows] + sfBt (output gradient and layer input,
 * both quantized along the row dimension, i.e. axis 0 of the [padded_rows, .] tensors);
 * padded_offs[E+1] from the permute plan gives every expert's row range.  D: bf16 [E*M, N],
 * zeros for experts without rows.  M % 128 == 0. */
int b200q_grouped_gemm_mxfp8_dgrad(const void* A, int a_fmt, const void* sfA, const void* Bt, int b_fmt,
                                   const void* sfBt, const int32_t* tile_expert,
                                   const int32_t* num_tiles, int64_t padded_rows, int E, int64_t N,
                                   int64_t K, void* D, int64_t ldd, void* stream);
int b200q_grouped_gemm_mxfp8_wgrad(const void* At, int a_fmt, const void* sfAt, const void* Bt, int b_fmt,
                                   const void* sfBt, const int32_t* padded_offs, int E, int64_t M,
                                   int64_t N, int64_t padded_rows, void* D, int64_t ldd, void* stream);

/* h[r, 0:I] = silu(gate) * up with gate = g[r, 0:I], up = g[r, I:2I] (src/layers/activation.py:80-81,
 * the step between the two grouped GEMMs, src/layers/mlp.py:92-94), rounded to bf16 as the
 * reference does, then (quantize = 1) MXFP8-quantized along I into `out` + swizzled `sf`, or
 * (quantize = 0) written as bf16.  I % 32 == 0. */
int b200q_swiglu(const void* g, int64_t rows, int64_t I, int64_t ld, int quantize, int fmt, void* out,
                 void* sf, void* stream);

/* The first GEMM of a gated MLP with the activation and the re-quantization done in its epilogue:
 * the step "h = grouped_mm(x, w_in); h = silu_glu(gate, up)" (src/layers/mlp.py:89-94,
 * src/layers/activation.py:80-81) followed by the MXFP8 quantization of h that the second GEMM
 * needs, without the bf16 [M, 2I] intermediate ever being written.  Same arithmetic as
 * b200q_(grouped_)gemm_mxfp8 -> b200q_swiglu(quantize = 1): accumulators rounded to bf16, SwiGLU in
 * the reference's bf16 steps, one E8M0 scale per 32 outputs; results are bit-identical to that chain.
 *
 * B must hold the N = 2I weight rows (per expert) in GLU-INTERLEAVED order: rows 64j .. 64j+31 are
 * gate rows 32j .. 32j+31 and rows 64j+32 .. 64j+63 are the up rows of the same outputs
 * (b200q_quantize_mxfp8_rowmap writes them so).  N % 64 == 0; grouped form: N % 128 == 0, so that
 * every expert's rows of B start a 128-row scale-factor group.
 * H: E4M3 codes [M, N/2], pitch ldh bytes (ldh % 16 == 0); sfH: 128x4-tiled scale factors over
 * (M, N/64), b200q_sf_bytes(M, N/64, B200Q_SF_SWIZZLE_128x4) bytes. */
int b200q_gemm_mxfp8_swiglu(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt,
                            const void* sfB, int64_t M, int64_t N, int64_t K, void* H, int64_t ldh,
                            void* sfH, void* stream);
/* The same for NVFP4 operands, as far as NVFP4 allows: h cannot be quantized where it is produced
 * (its tensor scale needs max|h| over the whole tensor first), so the epilogue writes h as bf16
 * [M, N/2] (pitch ldh elements) and that maximum to *amax_out - the two things b200q_quantize_nvfp4
 * of h needs - and the bf16 [M, 2I] gate/up tensor, twice the size of h, is never written.  B rows
 * in the interleaved order (b200q_quantize_nvfp4_rowmap).  Bit-identical to b200q_gemm_nvfp4 ->
 * b200q_swiglu(quantize = 0) -> b200q_amax. */
int b200q_gemm_nvfp4_swiglu(const void* A, const void* sfA, const void* B, const void* sfB,
                            const float* tsA, const float* tsB, int64_t M, int64_t N, int64_t K,
                            void* H, int64_t ldh, float* amax_out, void* stream);
int b200q_quantize_nvfp4_rowmap(const void* x, int64_t rows, int64_t cols, int64_t ld,
                                const float* tensor_amax, const int32_t* dst_row, void* codes,
                                void* sf, int sf_layout, float* tensor_scale_out, void* stream);
int b200q_grouped_gemm_mxfp8_swiglu(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt,
                                    const void* sfB, const int32_t* tile_expert,
                                    const int32_t* num_tiles, int64_t padded_rows, int E, int64_t N,
                                    int64_t K, void* H, int64_t ldh, void* sfH, void* stream);

/* Four element-wise steps of the trainable expert path, each fused with b200q_quantize_mxfp8_dual so that
 * the bf16 tensor between the step and its two MXFP8 copies is never written: the outputs are what
 * b200q_quantize_mxfp8_dual gives on the step's result (codes_row [rows, cols] + sf_row, codes_col
 * [cols, rows] + sf_col, 128x4-tiled scale factors), bit for bit.
 *   gather:              rows of x picked by src_of_row (b200q_moe_gather with quantize = 0; -1 = zero row)
 *   unpermute backward:  row r = w[p] * dout[p / k] for p = pair_of_row[r] (-1 = zero row), the dy of
 *                        b200q_moe_unpermute_backward (pair_of_row is the inverse of the plan's row_of).
 *                        With dw != NULL the same pass also gives that function's dw: dw[p] =
 *                        <dout[p / k], y[row_of[p]]> (fp32, 0 for a dropped pair), summed per 128-column
 *                        tile into dot_workspace ((D / 128) * padded_rows floats) and then per pair.
 *   swiglu:              silu(gate) * up of g = [gate | up]  (b200q_swiglu with quantize = 0)
 *   swiglu backward:     [d_gate | d_up] of b200q_swiglu_backward
 * Row counts are multiples of 128; D % 128 == 0; I % 128 == 0 (swiglu) / I % 64 == 0 (swiglu backward).
 * num_tiles (device int32, may be NULL) limits the work to the first *num_tiles 128-row tiles, as for
 * b200q_quantize_mxfp8_dual. */
int b200q_moe_gather_quantize_dual(const void* x, int64_t D, int64_t ld, const int32_t* src_of_row,
                                   int64_t padded_rows, int fmt, void* codes_row, void* sf_row,
                                   void* codes_col, void* sf_col, const int32_t* num_tiles, void* stream);
int b200q_moe_unpermute_backward_quantize_dual(const void* dout, int64_t ld, const void* w,
                                               const int32_t* pair_of_row, int k, int64_t padded_rows,
                                               int64_t D, int fmt, void* codes_row, void* sf_row,
                                               void* codes_col, void* sf_col, const void* y, int64_t ldy,
                                               const int32_t* row_of, int64_t n_pairs,
                                               float* dot_workspace, float* dw, void* stream);
int b200q_swiglu_quantize_dual(const void* g, int64_t rows, int64_t I, int64_t ldg, int fmt,
                               void* codes_row, void* sf_row, void* codes_col, void* sf_col,
                               const int32_t* num_tiles, void* stream);
int b200q_swiglu_backward_quantize_dual(const void* g, int64_t rows, int64_t I, int64_t ldg,
                                        const void* dh, int64_t lddh, int fmt, void* codes_row,
                                        void* sf_row, void* codes_col, void* sf_col,
                                        const int32_t* num_tiles, void* stream);

/* Expert parallelism inside one NVLink domain without a collective on the data path: ranks own
 * contiguous ranges of experts_per_rank experts and expose their buffers to each other (peer-mapped
 * device memory; the reference is single-GPU and has no counterpart).
 *
 * dispatch: the sender walks ITS padded expert-sorted plan over all E experts (src_of_row,
 * tile_expert, padded_offs, num_tiles from b200q_moe_permute_plan) and writes every routed row,
 * MXFP8-quantized along D, into the owner's buffers: row row_base[e] + (rank of the row inside the
 * sender's segment of e) of peer_codes[e / experts_per_rank] ([rows, D] codes) and peer_sf[...]
 * (128x4-tiled scale factors).  row_base[E] comes from the exchanged counts.  Stores only.
 * zero_pad_rows: the owner clears the rows of its own buffers that no sender writes (src_of_row < 0
 * in the owner's b200q_moe_pad_plan).
 * combine: out[t] = sum_j w[t,j] * peer_y[pair_peer[t*k+j]][pair_row[t*k+j]] with the expert
 * outputs (bf16, pitch ldy) loaded in place from their owners; fp32 accumulation, one rounding.
 * The caller orders dispatch -> (all ranks) -> owner's GEMMs -> (all ranks) -> combine.
 * D % 128 == 0, world <= 8. */
int b200q_moe_dispatch_peers(const void* x, int64_t D, int64_t ld, const int32_t* src_of_row,
                             const int32_t* tile_expert, const int32_t* padded_offs,
                             const int32_t* num_tiles, int64_t padded_rows, const int32_t* row_base,
                             int experts_per_rank, int world, void* const* peer_codes,
                             void* const* peer_sf, void* stream);
int b200q_moe_zero_pad_rows(const int32_t* src_of_row, const int32_t* num_tiles, int64_t padded_rows,
                            int64_t D, void* codes, void* sf, void* stream);
int b200q_moe_combine_peers(void* const* peer_y, int world, int64_t ldy, const void* w,
                            const int32_t* pair_peer, const int32_t* pair_row, int64_t T, int k,
                            int64_t D, void* out, void* stream);

/* Expert parallelism, the pieces around the kernels above (all new functionality; the reference is single-GPU).
 *
 * ep_index: from the gathered per-sender cumulative counts all_offs[world][E] (every rank's `offs` of its own permute
 * plan) - row_base[E]: where THIS rank's rows for every global expert start inside the owner's padded expert-sorted
 * buffer (segments of the owner's experts in order, each padded to 128 rows, senders in rank order inside a segment);
 * own_offs[E / world]: cumulative ends of the segments this rank owns (the `offs` input of b200q_moe_pad_plan);
 * pair_peer / pair_row [T*k]: owner and row there of every routed pair.  One launch replaces a dozen index operations.
 *
 * peer_barrier: stream-ordered rendezvous of the ranks through flag words in peer-mapped memory (flag_ptrs[g] = rank g's
 * int32[world] array, zero before the first use; `epoch` must grow by one per call on every rank): every rank stores
 * the epoch into its slot of every array and waits until all slots of its own array have reached it.  The wait is
 * bounded (about a second); a rank that gives up sets the device status word (b200q_device_status) and returns.
 *
 * scatter_rows_peers: out_{pair_peer[p]}[pair_row[p]] = (w[p] *) x[p / k] for every routed pair p, bf16 - the training
 * dispatch (w = NULL) and the backward of the combine (x = dout, w = routing weights).  Stores only.
 * zero_pad_rows_bf16: the owner clears the rows no sender writes (src_of_row < 0 in its pad plan).
 * pair_dots_peers: dw[p] = <dout[p / k], y_{pair_peer[p]}[pair_row[p]]> in fp32, the routing weights' gradient. */
int b200q_moe_ep_index(const int32_t* all_offs, int world, int rank, int E, const int64_t* top_idx,
                       const int32_t* row_of, const int32_t* padded_offs, int64_t n_pairs, int32_t* row_base,
                       int32_t* own_offs, int32_t* pair_peer, int32_t* pair_row, void* stream);
int b200q_peer_barrier(void* const* flag_ptrs, int world, int rank, int epoch, void* stream);
int b200q_moe_scatter_rows_peers(const void* x, int64_t ld, const void* w, const int32_t* pair_peer,
                                 const int32_t* pair_row, int64_t T, int k, int64_t D, void* const* peer_y,
                                 int world, int64_t ldy, void* stream);
int b200q_moe_zero_pad_rows_bf16(const int32_t* src_of_row, const int32_t* num_tiles, int64_t padded_rows,
                                 int64_t D, void* buf, int64_t ld, void* stream);
int b200q_moe_pair_dots_peers(const void* dout, int64_t ld, void* const* peer_y, int world, int64_t ldy,
                              const int32_t* pair_peer, const int32_t* pair_row, int64_t T, int k, int64_t D,
                              float* dw, void* stream);

/* Expert-parallel MoE forward after the index tables (b200q_moe_permute_plan, the all-gather of the counts,
 * b200q_moe_ep_index, b200q_moe_pad_plan) as ONE call: b200q_moe_zero_pad_rows on this rank's receive buffers,
 * b200q_moe_dispatch_peers, rendezvous, b200q_grouped_gemm_mxfp8_swiglu and b200q_grouped_gemm_mxfp8 over the experts
 * this rank owns (the second one writes peer_y[rank]), rendezvous, b200q_moe_combine_peers into out[T, D] bf16,
 * rendezvous.  The rendezvous are b200q_peer_barrier with epochs epoch + 1, epoch + 2, epoch + 3 (the caller advances
 * its epoch by 3).  src_of_row .. padded_rows: this rank's plan over ALL experts; own_*: the plan of the experts it owns
 * (own_padded_rows rows in every receive buffer); w1: (experts_per_rank * 2I, D) gate / up rows interleaved in blocks of
 * 32, w2: (experts_per_rank * D, I), both MXFP8 E4M3 with swizzled scale factors.  D % 128 == 0, I % 64 == 0.
 * workspace: b200q_moe_ep_forward_workspace_bytes(own_padded_rows, I) bytes, 256-byte aligned.  Equal to the separate
 * calls bit for bit. */
int64_t b200q_moe_ep_forward_workspace_bytes(int64_t own_padded_rows, int64_t I);
int b200q_moe_ep_forward(const void* x, int64_t ldx, const void* top_w, int64_t T, int k, int64_t D, int64_t I,
                         int experts_per_rank, int world, int rank, int epoch, const int32_t* src_of_row,
                         const int32_t* tile_expert, const int32_t* padded_offs, const int32_t* num_tiles,
                         int64_t padded_rows, const int32_t* row_base, const int32_t* pair_peer,
                         const int32_t* pair_row, const int32_t* own_src_of_row, const int32_t* own_tile_expert,
                         const int32_t* own_num_tiles, int64_t own_padded_rows, void* const* peer_codes,
                         void* const* peer_sf, void* const* peer_y, void* const* flag_ptrs, const void* w1_codes,
                         const void* w1_sf, const void* w2_codes, const void* w2_sf, void* out, void* workspace,
                         void* stream);

/* Backward of b200q_swiglu(quantize = 0): dg[r] = [dh * up * silu'(gate) | dh * silu(gate)] for
 * g[r] = [gate | up]; bf16 in and out, fp32 arithmetic (the reference gets this from autograd through
 * src/layers/activation.py:80-81).  I % 8 == 0. */
int b200q_swiglu_backward(const void* g, int64_t rows, int64_t I, int64_t ldg, const void* dh,
                          int64_t lddh, void* dg, int64_t lddg, void* stream);

/* Backward of b200q_moe_unpermute (src/layers/mlp.py:472-477 under autograd): from the block's
 * output gradient dout (bf16 [T, D]) it writes dy (bf16 [padded_rows, D]) with
 * dy[row_of[t*k+j]] = w[t,j] * dout[t] and zero rows wherever src_of_row < 0, and, when y (the
 * forward's expert outputs, bf16 [padded_rows, D], pitch ldy) and dw are given, the router-weight
 * gradient dw[t*k+j] = <dout[t], y[row_of[t*k+j]]> in fp32.  dy may be NULL when only dw is wanted. */
int b200q_moe_unpermute_backward(const void* dout, const void* w, const void* y, int64_t ldy,
                                 const int32_t* row_of, const int32_t* src_of_row, int64_t T, int k,
                                 int64_t D, int64_t padded_rows, void* dy, float* dw, void* stream);

/* Everything MoERouter.forward does after the fp32 gate GEMM (src/layers/mlp.py:292-301) and the
 * bincount of the block (:455), in one launch: probs = softmax (score_fn 0) or sigmoid (1) of the
 * fp32 logits [T, E]; the k largest probs per token in descending order -> top_idx (int64 [T, k]);
 * their probs, divided by (their sum + 1e-9) when normalize != 0, -> top_w (bf16 [T, k]); probs as
 * bf16 [T, E] (optional); expert_counts[e] = tokens that chose e (int32 [E], optional).  Equal
 * probs are ordered by logit, then by expert index.  select_bias (fp32 [E], optional): the experts are
 * chosen by prob + select_bias, the load-balancing bias of src/layers/mlp.py:182-216,295-297, while the
 * weights stay the chosen experts' probs.  out_fp32 != 0: top_w and probs are written as fp32 instead
 * of bf16 (the reference returns them in the activations' dtype, :302).  E <= 256, k <= 32. */
int b200q_moe_router_topk(const float* logits, int64_t T, int E, int k, int score_fn, int normalize,
                          int64_t* top_idx, void* top_w, void* probs, int32_t* expert_counts,
                          const float* select_bias, int out_fp32, void* stream);

/* The expert path of the MoE block in one call (src/layers/mlp.py:446-477 with grouped_mlp, :55-100, between
 * permute and unpermute), for bias-free SwiGLU experts, forward only: b200q_moe_permute_plan, b200q_moe_gather with
 * MXFP8 quantization, b200q_grouped_gemm_mxfp8_swiglu, b200q_grouped_gemm_mxfp8 and b200q_moe_unpermute, issued
 * back to back by one host call, every launch after the first allowed to start while its predecessor drains; the
 * result equals the five calls bit for bit.  x bf16 [T, D] (pitch ldx elements); top_idx int64 [T, k]; top_w
 * bf16 [T, k]; w1: the gate/up weight stack [E * 2I, D], rows interleaved gate / up in blocks of 32 per expert as
 * b200q_grouped_gemm_mxfp8_swiglu wants them, MXFP8 along D (E4M3 codes, swizzled scale factors); w2: the down
 * weight stack [E * D, I], MXFP8 along I; out bf16 [T, D] contiguous; offs (optional): int32 [E], the cumulative
 * number of routed pairs per expert as b200q_moe_permute_plan returns it.  workspace: 256-byte aligned,
 * b200q_moe_ffn_workspace_bytes(T, k, D, E, I) bytes, holds the plan's tables and the intermediates (a, h as
 * MXFP8, y as bf16); needs no initialisation and may be reused by the next call on the same stream.
 * D % 128 == 0, I % 64 == 0, E <= 256. */
int64_t b200q_moe_ffn_workspace_bytes(int64_t T, int k, int64_t D, int E, int64_t I);
int b200q_moe_ffn_forward(const void* x, int64_t ldx, const int64_t* top_idx, const void* top_w, int64_t T, int k,
                          int64_t D, int E, int64_t I, const void* w1_codes, const void* w1_sf, const void* w2_codes,
                          const void* w2_sf, void* out, int32_t* offs, void* workspace, void* stream);

/* The TRAINABLE expert path, forward and backward as one call each (bias-free SwiGLU experts; the reference differentiates
 * src/layers/mlp.py:446-477 through torch._grouped_mm with autograd, here the backward is explicit).  Forward =
 * b200q_moe_gather_quantize_dual, b200q_grouped_gemm_mxfp8 (g, kept), b200q_swiglu_quantize_dual, b200q_grouped_gemm_mxfp8
 * (y, kept), b200q_moe_unpermute; backward = b200q_moe_pair_of_row, b200q_moe_unpermute_backward_quantize_dual (with dw),
 * dgrad / wgrad of the second GEMM, b200q_swiglu_backward_quantize_dual, dgrad / wgrad of the first GEMM, unpermute with
 * unit weights.  Results equal the separate calls bit for bit; what the one call adds is that its kernels are issued back to
 * back and may be scheduled while their predecessors drain.  The plan's tables come from b200q_moe_permute_plan.
 * Shapes (R = padded_rows): x bf16 [T, D]; top_w bf16 [T, k]; w1r / w1sr: gate | up stack [E * 2I, D] MXFP8 along D (rows NOT
 * interleaved), w2r / w2sr: down stack [E * D, I] along I; w1c / w1sc and w2c / w2sc: the same stacks quantized along axis 0
 * ([D, E * 2I], [I, E * D]).  Saved by the forward for the backward: ac / asc ([D, R] codes of the gathered rows along R),
 * g bf16 [R, 2I], hc / hsc ([I, R]), y bf16 [R, D].  Gradients: dx bf16 [T, D], dw fp32 [T, k], dw1 bf16 [E, 2I, D],
 * dw2 bf16 [E, D, I].  Activations and weights E4M3, gradients E5M2.  D % 128 == 0, I % 128 == 0; workspaces 256-byte
 * aligned, sized by the *_workspace_bytes functions, no initialisation needed. */
int64_t b200q_moe_ffn_train_forward_workspace_bytes(int64_t padded_rows, int64_t D, int64_t I);
int b200q_moe_ffn_train_forward(const void* x, int64_t ldx, const void* top_w, int64_t T, int k, int64_t D, int E, int64_t I,
                                int64_t padded_rows, const int32_t* row_of, const int32_t* src_of_row,
                                const int32_t* tile_expert, const int32_t* num_tiles, const void* w1r, const void* w1sr,
                                const void* w2r, const void* w2sr, void* ac, void* asc, void* g, void* hc, void* hsc, void* y,
                                void* out, void* workspace, void* stream);
int64_t b200q_moe_ffn_train_backward_workspace_bytes(int64_t padded_rows, int64_t D, int64_t I);
int b200q_moe_ffn_train_backward(const void* dout, int64_t lddout, const void* top_w, int64_t T, int k, int64_t D, int E,
                                 int64_t I, int64_t padded_rows, const int32_t* row_of, const int32_t* padded_offs,
                                 const int32_t* tile_expert, const int32_t* num_tiles, const void* y, const void* g,
                                 const void* ac, const void* asc, const void* hc, const void* hsc, const void* w1c,
                                 const void* w1sc, const void* w2c, const void* w2sc, void* dx, float* dw, void* dw1, void* dw2,
                                 void* workspace, void* stream);

/* Weighted unpermute (src/layers/mlp.py:472-477): out[t, :] = sum_j w[t, j] * y[row_of[t*k+j], :],
 * accumulated in fp32 and rounded once to bf16.  y bf16 [padded_rows, D] pitch ldy; w bf16 [T, k], or
 * NULL for unit weights (the sum over the k slots: the backward of the gather). */
int b200q_moe_unpermute(const void* y, int64_t ldy, const void* w, const int32_t* row_of, int64_t T,
                        int k, int64_t D, void* out, void* stream);

/* Inverse of the plan's row_of (int32 [n_pairs], pair -> padded row, negative = dropped): pair_of_row
 * [padded_rows] = the routed pair t*k+j that owns the row, -1 for pad rows (the reference keeps this as
 * token_ids_sorted / weights_sorted, src/layers/mlp.py:446-458). */
int b200q_moe_pair_of_row(const int32_t* row_of, int64_t n_pairs, int64_t padded_rows,
                          int32_t* pair_of_row, void* stream);

/* ---- test hooks ------------------------------------------------------------------------------
 * Process-wide switches that override the kernel choice every later GEMM call makes, for tests that
 * want to run one shape through every kernel form.  They are plain global variables: not thread-safe,
 * not per device, and not meant for production callers (which never need them: 0 = choose by shape
 * is the default).  No counterpart in the reference.
 *   b200q_debug_set_gemm_bn(bn):    N tile width of the one-CTA kernel, 128 / 192 / 256; 0 = by shape.
 *   b200q_debug_set_gemm_pair(mode): 1 = CTA-pair kernel whenever the shape allows, -1 = never, 0 = by shape.
 *   b200q_debug_set_gemm_bstat(mode): grouped fprop / dgrad GEMMs with K <= 768 on the kernel that keeps the expert's
 *                                    weight tile in shared memory: 1 = whenever the shape allows, -1 = never, 0 = by shape and size.
 *   b200q_debug_set_gemm_rowstat(mode): the same GEMMs on the CTA-pair kernel that keeps the rows of A in shared memory
 *                                    (tried before the one above): 1 = whenever the shape allows, -1 = never, 0 = by shape and size. */
int b200q_debug_set_gemm_bn(int bn);
int b200q_debug_set_gemm_pair(int mode);
int b200q_debug_set_gemm_bstat(int mode);
int b200q_debug_set_gemm_rowstat(int mode);
/* Runs a one-thread kernel whose bounded wait cannot succeed (an mbarrier nobody arrives on), with a limit of
 * `iterations` polls (1 .. 100000, i.e. milliseconds): the kernel gives up, records a non-zero status and returns,
 * exactly as the GEMM kernels' waits do after their ~1 s limit.  The next b200q_device_status() returns
 * B200Q_ERR_DEVICE_TIMEOUT (and clears it).  For testing the failure-reporting path without a fault or a hang. */
int b200q_debug_expire_wait(int iterations, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
