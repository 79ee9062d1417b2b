/*
 * sparse24_b200 — C ABI of the B200 (sm_100a) kernels for the 2:4 sparse-training hot path.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), validates
 * its arguments BEFORE launching anything, and returns SP24_OK (0) or a negative
 * error code.  Nothing here allocates, synchronises, throws or traps: outputs and
 * workspaces are caller-allocated, launches are asynchronous on `stream`.
 * Matrices are described as "logical (rows, cols) + storage order + leading
 * dimension in elements": col_major = 0 means element (r, c) is at r*ld + c,
 * col_major = 1 means it is at c*ld + r.
 *
 * The reference project has one native entry point (a pybind11 function) and
 * launches all its other kernels from Python through Triton; each declaration
 * below names the reference interface it replaces (paths are relative to the
 * reference project root).
 */
#ifndef SPARSE24_B200_H
#define SPARSE24_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
enum {
    SP24_F32 = 0,
    SP24_F16 = 1,
    SP24_BF16 = 2,
    SP24_E4M3 = 3, /* float8_e4m3fn */
    SP24_E5M2 = 4, /* float8_e5m2 */
    SP24_I8 = 5,
    SP24_I32 = 6   /* output of the int8 sparse GEMM only */
};

/* pruning rule of the dense -> 2:4 conversion */
enum {
    SP24_PRUNE_MSE = 0,  /* keep the two largest magnitudes of every four (ties keep the higher index) */
    SP24_PRUNE_MASK = 1, /* keep what a supplied 0/1 byte mask says */
    SP24_PRUNE_MVUE = 2, /* minimum-variance unbiased 2-of-4 sampling, rescaled; IEEE arithmetic, bit-exact
                            against the reference formulas given the uniforms */
    SP24_PRUNE_MVUE_FAST = 3 /* the same estimator for production use: seeded only (no uniforms argument),
                                reciprocal-approximation arithmetic and a 7-round Philox stream; unbiased to
                                float32 rounding, not bit-comparable with SP24_PRUNE_MVUE */
};

/* error codes */
enum {
    SP24_OK = 0,
    SP24_ERR_SHAPE = -1,       /* a dimension is not a positive multiple of what the op needs */
    SP24_ERR_STRIDE = -2,      /* leading dimension too small or not a multiple of the vector width */
    SP24_ERR_DTYPE = -3,       /* element-type combination not supported */
    SP24_ERR_ALIGN = -4,       /* pointer not 16-byte aligned */
    SP24_ERR_ARG = -5,         /* null pointer / contradictory flags / value out of range */
    SP24_ERR_CUDA = -6,        /* the CUDA runtime reported an error at launch */
    SP24_ERR_DEVICE = -7,      /* current device is not compute capability 10.x */
    SP24_ERR_TOO_LARGE = -8    /* size beyond a stated fixed capacity */
};

/* Human-readable text for an error code (static storage). */
const char *sp24_strerror(int code);

/* ABI version of the loaded library (bumped when a signature changes). */
int sp24_abi_version(void);

/*
 * Peer memory for a gradient exchange that runs on the copy engines instead of on SMs (no counterpart in the
 * reference): map a buffer another process of this node exported (a 64-byte cudaIpcMemHandle_t, e.g. from
 * cudaIpcGetMemHandle or the framework's storage-sharing call) into this process; *ptr is then the base address of
 * the exporter's allocation, valid on the current device, and copies from it are ordinary asynchronous
 * device-to-device copies.  One open per handle and process; close before the exporter frees the buffer.
 */
int sp24_ipc_open(const void *handle, int handle_bytes, void **ptr);
int sp24_ipc_close(void *ptr);

/*
 * Dense -> 2:4 compressed (values + reordered metadata), fused prune + compress + metadata.
 * Replaces sparse_semi_structured_from_dense_triton and the Triton kernels
 * _sparse_semi_structured_from_dense_triton_16 / _8
 * (sparse/_semi_structured_conversions.py:431-661, :664-1069, launcher :1072-1132).
 *
 *   dense      logical (m, k), dense_dtype in {F32, F16, BF16}; with packed_dtype I8 also I8
 *   col_major  storage order of dense; packed, mask and uniforms use the same order
 *   packed     logical (m, k/2), packed_dtype in {F16, BF16, E4M3, E5M2, I8}; values are cast on store
 *   meta       m*k/16 int16 (16-bit packed types) or m*k/32 int32 (8-bit), in the reference's
 *              reordered layout (row interleave by 8 within groups of 32 / 16 rows, 2x2 swizzle,
 *              column-major interleaved by 2)
 *   mode       SP24_PRUNE_*; mask (bytes, non-zero = keep, logical (m, k)) only for SP24_PRUNE_MASK
 *   uniforms   optional, SP24_PRUNE_MVUE only: float32 logical (m, k); group g of row r uses [r,4g] and [r,4g+1].
 *              When NULL the kernel draws from Philox4x32-10 keyed by (seed, offset):
 *              group index gi = r*(k/4)+g, counter = (gi>>1, offset), key = seed, even groups take
 *              words 0,1 and odd groups words 2,3, u = (word >> 8) * 2^-24.
 *              SP24_PRUNE_MVUE_FAST takes no uniforms and draws the same way from Philox4x32-7; its arithmetic
 *              replaces the ten IEEE divisions per group by seven reciprocal approximations (the reference's
 *              own GPU kernel also divides approximately), so kept positions and stored values can differ from
 *              SP24_PRUNE_MVUE's in the last float32 bits; it is the mode the training layer uses.
 * Shape rules (sparse/semi_structured.py:24-30,188-200): m % 32 == 0; k % 64 == 0 (16-bit) or
 * k % 128 == 0 (8-bit).  Leading dimensions must keep every row/column start 16-byte aligned.
 */
int sp24_prune_compress(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense, int col_major,
                        void *packed, int packed_dtype, int64_t ld_packed, void *meta, int mode,
                        const void *mask, int64_t ld_mask, const float *uniforms, int64_t ld_uniforms,
                        uint64_t seed, uint64_t offset, void *stream);

/*
 * sp24_prune_compress with three optional extras (each may be NULL); no counterpart in the reference.
 *   offset_dev  the Philox stream is keyed by (seed, offset + *offset_dev), *offset_dev being a 64-bit word in
 *               device memory (8-byte aligned) read when the kernel runs.  A launch that is recorded once and
 *               replayed (a CUDA graph of the training step) draws fresh uniforms on every replay if the caller
 *               bumps that word between replays.  The reference draws a new host seed per call
 *               (sparse/_semi_structured_conversions.py:1076) and has no replayable form.
 *   e_tc        a second copy of the metadata in the order sp24_spmm reads (sp24_meta_tc_bytes(m, k) bytes, 16-byte
 *               aligned), which saves the sp24_meta_to_tc launch.  16-bit packed types and m % 128 == 0 only.
 *   row_sums    m floats: row_sums[r] += sum over k of dense[r, k] (values before pruning; fp32 partial sums added
 *               with atomics, so zero the array first or pass a gradient buffer to add to).  Column-major storage
 *               only.  For dY^T these are the bias gradients of the layer (grad_output.sum(0), README.md:197-198 of
 *               the reference), taken from the pass that reads dY anyway.
 */
int sp24_prune_compress_ex(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense, int col_major,
                           void *packed, int packed_dtype, int64_t ld_packed, void *meta, int mode, const void *mask,
                           int64_t ld_mask, const float *uniforms, int64_t ld_uniforms, uint64_t seed, uint64_t offset,
                           const uint64_t *offset_dev, void *e_tc, float *row_sums, void *stream);

/*
 * Float8 quantising form of sp24_prune_compress: packed_dtype E4M3 or E5M2, stored value = value * out_scale (the
 * caller's per-tensor quantisation scale, > 0; saturating cast), and packed is ALWAYS row-major (m, k/2) with pitch
 * ld_packed, whatever the storage order of dense.  With col_major = 1 (W.T of a row-major weight, dY.T of a row-major
 * gradient) this gives the K-major sparse operand the 8-bit GEMM requires without a transpose pass.  The reference
 * cannot run its backward pass in float8: its 8-bit kernels take row-major A only
 * (sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:735-738, :778-781) while its conversion of a transposed view
 * writes column-major packed values (sparse/semi_structured.py:231-243), and its MVUE branch for 8-bit outputs is
 * incomplete (sparse/_semi_structured_conversions.py:822-839); this entry point defines that path: eight groups per
 * int32 metadata word, one Philox block per two groups as for 16-bit outputs.  mode: MSE, MASK, MVUE (seeded) or
 * MVUE_FAST; mask follows the storage order of dense.
 */
int sp24_prune_compress_q8(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense, int col_major,
                           void *packed, int packed_dtype, int64_t ld_packed, void *meta, int mode, const void *mask,
                           int64_t ld_mask, float out_scale, uint64_t seed, uint64_t offset, void *stream);

/*
 * 2:4 compressed -> dense (zeros at pruned positions).  Replaces
 * _sparse_semi_structured_to_dense_triton / _sparse_semi_structured_to_dense
 * (sparse/_semi_structured_conversions.py:1163-1274, :217-328).
 * packed is row-major (m, k/2) with leading dimension ld_packed; dense is row-major (m, k).
 * dtype: F16, BF16 (int16 metadata) or E4M3, E5M2, I8 (int32 metadata).
 */
int sp24_to_dense(const void *packed, int dtype, int64_t m, int64_t k, int64_t ld_packed, const void *meta,
                  void *dense, int64_t ld_dense, void *stream);

/*
 * Dense-shaped MVUE24: out = x_i / p_i at the two sampled positions of every group of four, +0 elsewhere.
 * Replaces MVUE24_approx_triton (sparse/triton_ops.py:10-81; arithmetic sparse/utils.py:5-59).
 * dtype in {F32, F16, BF16}; uniforms / seed / offset as in sp24_prune_compress.
 */
int sp24_mvue24_dense(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, void *out,
                      int64_t ld_out, const float *uniforms, int64_t ld_uniforms, uint64_t seed, uint64_t offset,
                      void *stream);

/*
 * sp24_mvue24_dense with the arithmetic and the 7-round Philox stream of SP24_PRUNE_MVUE_FAST (seeded only): at the
 * kept positions it writes exactly what sp24_prune_compress stores in that mode for the same (seed, offset).  The
 * reference's own GPU kernel divides with the compiler's approximate division (sparse/utils.py:6-59 as launched
 * from sparse/triton_ops.py:55-81); this is the counterpart of that production path.
 */
int sp24_mvue24_dense_fast(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, void *out,
                           int64_t ld_out, uint64_t seed, uint64_t offset, void *stream);

/*
 * Magnitude 2:4 pruning, dense-shaped: sparse = x where kept else +0, mask = 1 / 0 in x's dtype.
 * Replaces sparse24_triton (sparse/triton_ops.py:84-154).  Every output element is written.
 */
int sp24_sparse24(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, void *sparse,
                  int64_t ld_sparse, void *mask, int64_t ld_mask, void *stream);

/*
 * S-STE soft threshold: kept values move toward zero by the group's second-smallest magnitude
 * (one rounding in x's dtype); mask = 1 / 0 in x's dtype.  Replaces soft_threshold24_triton
 * (sparse/triton_ops.py:157-227; arithmetic sparse/utils.py:72-90).  With use_scale != 0 the kept
 * values are further multiplied by `scale` (one more rounding in x's dtype), which folds the
 * `weight_sparse * scale` pass of the reference's S-STE recipe (README.md:233-260) into the store.
 */
int sp24_soft_threshold24(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, void *sparse,
                          int64_t ld_sparse, void *mask, int64_t ld_mask, int use_scale, float scale, void *stream);

/*
 * The forward pass of the S-STE layer in one pass over W: magnitude 2:4 mask, soft threshold of the two kept values
 * (one rounding in dense's type), optional multiplication by the frozen scale (one more rounding in dense's type), cast
 * to the packed 16-bit type, reordered metadata - bit for bit what sp24_soft_threshold24, a cast and sp24_prune_compress
 * (mask mode) produce in three passes.  Replaces `weight_sparse * scale` of the reference's S-STE recipe
 * (README.md:233-260; soft_threshold24_triton, sparse/triton_ops.py:157-227) followed by to_sparse_semi_structured
 * (sparse/semi_structured.py:575-631) when the forward GEMM runs on the sparse tensor cores.
 * dense: F32 / F16 / BF16, either storage order; packed_dtype F16 / BF16; e_tc optional (as in sp24_prune_compress_ex).
 */
int sp24_soft_threshold24_compress(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense, int col_major,
                                   void *packed, int packed_dtype, int64_t ld_packed, void *meta, int use_scale, float scale,
                                   void *e_tc, void *stream);

/*
 * Transposable 4x4 mask select: for every 4x4 block the first (in descending lexicographic order of
 * the row-major bit string) of the 90 patterns with two ones per row and per column that maximises
 * the float32 score (s0 + s1) + (s2 + s3), s_i = v[i][a_i] + v[i][b_i], v = |x| when use_abs.
 * Replaces _to_transposable_sparse_semi_structured_kernel / TransposableSparse.forward
 * (sparse/transposable_semi_structured.py:8-94, :198-200).
 * x row-major (m, k), m % 32 == 0, k % 64 == 0, dtype in {F32, F16, BF16}.
 * sparse_out (same dtype, may be NULL) = x where mask else +0; mask_out = bytes 0/1 (torch.bool).
 */
int sp24_transposable_select(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int use_abs,
                             void *sparse_out, int64_t ld_sparse, void *mask_out, int64_t ld_mask, void *stream);

/*
 * One mask refresh of the training layer in a single pass over W: transposable select (as above,
 * |w| scores) + 2:4 compression of W (row-major packed (m, k/2) + meta_w of m*k/16 int16) and of
 * W^T under the transposed mask (packed_t is the column-major packed the reference produces for
 * the W.T view: storage (m/2, k) row-major with leading dimension ld_packed_t; meta_t of k*m/16
 * int16 for the logical (k, m) matrix).  Replaces the three-launch sequence of the reference's
 * SparseLinearTranspose.forward (README.md:148-155): TransposableSparse, then
 * to_sparse_semi_structured(W, mask) and to_sparse_semi_structured(W.T, mask.T).
 * If select == 0 the mask is read from mask (bytes) instead of being recomputed.
 * m % 64 == 0 and k % 64 == 0; packed_dtype in {F16, BF16}.
 */
int sp24_select_dual_compress(const void *w, int dtype, int64_t m, int64_t k, int64_t ld_w, int select, void *mask,
                              int64_t ld_mask, void *packed_w, int packed_dtype, int64_t ld_packed_w, void *meta_w,
                              void *packed_t, int64_t ld_packed_t, void *meta_t, void *stream);

/*
 * sp24_select_dual_compress, which also writes the metadata of W (tc_w, sp24_meta_tc_bytes(m, k) bytes) and of
 * W^T (tc_t, sp24_meta_tc_bytes(k, m) bytes) in the order sp24_spmm reads, so that neither operand needs an
 * sp24_meta_to_tc launch.  m % 128 == 0 and k % 128 == 0.  No counterpart in the reference.
 */
int sp24_select_dual_compress_tc(const void *w, int dtype, int64_t m, int64_t k, int64_t ld_w, int select, void *mask,
                                 int64_t ld_mask, void *packed_w, int packed_dtype, int64_t ld_packed_w, void *meta_w,
                                 void *packed_t, int64_t ld_packed_t, void *meta_t, void *tc_w, void *tc_t,
                                 void *stream);

/*
 * sp24_select_dual_compress(_tc) for several matrices of one element type in one launch per 48 matrices: the
 * per-step recompression of every layer of a model (README.md:148-155 of the reference, once per layer), where
 * one matrix alone is too small to fill the GPU.  Fields as the arguments of the same name above; tc_w / tc_t
 * are either both set in every descriptor or NULL in every descriptor.  The descriptors are read on the host
 * during the call.  No counterpart in the reference.
 */
typedef struct sp24_dual_desc {
    const void *w;
    int64_t m, k, ld_w;
    void *mask;
    int64_t ld_mask;
    void *packed_w;
    int64_t ld_packed_w;
    void *meta_w;
    void *packed_t;
    int64_t ld_packed_t;
    void *meta_t;
    void *tc_w, *tc_t;
} sp24_dual_desc;
int sp24_select_dual_compress_batch(const sp24_dual_desc *descs, int count, int dtype, int packed_dtype, int select,
                                    void *stream);

/*
 * Masked decay, in place: grad[i] += p[i] * alpha where mask[i] == 0 (two roundings, no fused
 * multiply-add).  Replaces masked_add_ / masked_add_kernel (sparse/decay.py:7-37).
 * grad, p: float32, n elements, contiguous; mask_itemsize 1 (bool / uint8), 2 (f16 / bf16) or 4 (f32),
 * "zero" meaning numerically zero.
 */
int sp24_masked_add(void *grad, const void *p, const void *mask, int mask_itemsize, int64_t n, float alpha,
                    void *stream);

/*
 * Masked decay and the AdamW update in one pass over a flat float32 range (step 2 of the reference recipe,
 * README.md:205-214 of the reference, followed by torch.optim.AdamW; the reference runs them as separate passes):
 *   g = grad + p * alpha on pruned positions (mask byte 0; same two roundings as sp24_masked_add), grad elsewhere;
 *   p *= 1 - lr * weight_decay;  m += (g - m) * (1 - beta1);  v = v * beta2 + (1 - beta2) * g * g;
 *   p -= lr / (1 - beta1^t) * m / (sqrt(v) / sqrt(1 - beta2^t) + eps).
 * mask: n bytes or NULL (no decay).  t: `step` (>= 1), or the float at `step_dev` (device memory) when that is not
 * NULL, for launches that are recorded once and replayed.  All arrays 16-byte aligned.  grad is not modified.
 */
int sp24_adamw_masked_decay(void *p, const void *grad, const void *mask, void *exp_avg, void *exp_avg_sq, int64_t n,
                            float lr, float beta1, float beta2, float eps, float weight_decay, float alpha, float step,
                            const float *step_dev, void *stream);

/*
 * The same update with the gradient in float32, float16 or bfloat16 (grad_dtype; a 16-bit gradient is what a 16-bit
 * gradient exchange leaves behind: no cast back to float32) and, optionally, a second gradient added to the first
 * grad2_count elements (grad2_count % 4 == 0, <= n): g = grad + grad2 there, grad2 in any of the three types.  For a
 * gradient that arrives in two parts, e.g. a tied embedding whose output-head share is exchanged on its own: no
 * separate pass adds the parts.
 */
int sp24_adamw_masked_decay_ex(void *p, const void *grad, int grad_dtype, const void *mask, void *exp_avg, void *exp_avg_sq,
                               int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay, float alpha,
                               float step, const float *step_dev, const void *grad2, int grad2_dtype, int64_t grad2_count,
                               void *stream);

/*
 * Metadata re-layout for the tensor cores: the reference's reordered metadata (m*k/16 int16 or m*k/32
 * int32) -> the order tcgen05.mma.sp consumes from tensor memory.  The result is a sequence of 2048-byte
 * atoms, one per (128-row block, 128-column block), row blocks outermost; 16-bit types: atom byte
 * 16*L + 4*q + 2*h with L = 16*(r/16) + 8*(c%2) + r%8, q = (c/2)%4, h = (r/8)%2 (r = row in the block,
 * c = 16-column metadata word in the atom); 8-bit types: 128 rows x 16 bytes, row-major.  K is padded
 * up to a multiple of 128 with zero words.  sp24_meta_tc_bytes gives the buffer size.  m % 128 == 0.
 * No counterpart in the reference, whose CUTLASS kernel reads the reordered layout directly
 * (sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:826-851 documents that layout).
 */
int64_t sp24_meta_tc_bytes(int64_t m, int64_t k);
int sp24_meta_to_tc(const void *meta, int meta_itemsize, int64_t m, int64_t k, void *e_tc, void *stream);

/*
 * 2:4 sparse GEMM  D (ms x n) = A_sparse (ms x k) * B (k x n) [+ bias[row]] [activation], fp32 accumulate
 * (int32 for int8 operands).
 * Replaces my_sparse_semi_structured_linear and its CUTLASS SparseGemm instantiations
 * (sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:498-817, :34-233; caller
 * sparse/sparse_semi_structured_linear.py:4-5).
 *
 *   a_packed   compressed values, logical (ms, k/2); a_mn_major = 0: row-major with leading dimension ld_a,
 *              1: column-major (storage (k/2, ms)), the form the reference produces for W.T and dY.T views
 *   e_tc       metadata from sp24_meta_to_tc
 *   b          dense operand, logical (k, n); b_mn_major = 0: stored as (n, k) row-major ("K-major", e.g. the
 *              activations X (tokens, k)), 1: stored as (k, n) row-major
 *   out        trans_out = 0: (ms, n) row-major; 1: (n, ms) row-major, i.e. already transposed back to
 *              (tokens, features); leading dimension ld_out
 *   dtype      F16 / BF16 (out_dtype = dtype), E4M3 / E5M2 (out_dtype = F32) or I8 (out_dtype = I32, no bias, no
 *              activation); the 8-bit types take K-major operands only.  The same table as the reference's
 *              (sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:594-637, 729, 772).
 *              16-bit GEMMs with b_mn_major = 0, trans_out = 1, ms % 256 == 0, n >= 1024 and no activation run on
 *              pairs of CTAs (tcgen05 cta_group::2); the result is bit-equal to the single-CTA kernel's.
 *   bias       ms values in the output type or NULL; activation 0 none, 1 relu, 2 silu, 3 gelu (tanh form; not in the reference)
 *   status     optional device int: set to a non-zero code if a bounded on-device wait gave up
 * Shape rules: ms % 128 == 0, k % 64 == 0 (16-bit) or k % 128 == 0 (8-bit); n % 8 == 0 unless B is stored (n, k)
 * and the output (n, ms) (b_mn_major == 0 and trans_out == 1), where any n > 0 is accepted.
 */
int sp24_spmm(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc, int64_t ms, int64_t k,
              const void *b, int b_mn_major, int64_t ld_b, int64_t n, void *out, int out_dtype, int trans_out,
              int64_t ld_out, const void *bias, int activation, int *status, void *stream);

/*
 * The GEMMs of a transformer MLP block with their element-wise neighbours fused into the epilogue.  16-bit operands,
 * b stored (n, k) (tokens x features), out (n, ms) with pitch ld_out (what sp24_spmm calls trans_out = 1), ms % 256 == 0;
 * runs on the CTA-pair kernel.  bias: ms values, of the output type or (bias_is_f32 != 0) float32, or NULL.
 *   epilogue 0  out = acc + bias                                  (a float32 bias saves the cast launch per call)
 *   epilogue 1  aux = h = acc + bias rounded to the output type;  out = gelu(h), tanh form, evaluated on the rounded h:
 *               the up-projection of the MLP with its activation, keeping the pre-activation for the backward pass
 *   epilogue 2  out = acc * gelu'(aux) (no bias): the input gradient of the down-projection, written as the gradient
 *               of the up-projection's pre-activation aux
 * aux is shaped and aligned like out, pitch ld_aux.  The reference fuses relu / silu into its GEMM epilogue
 * (sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:385-471) and has a fused tanh-GELU forward / backward pair as
 * separate Triton kernels (sparse/GELUglu.py:7-243); its training layer runs bias, activation and their gradients as
 * separate passes (README.md:169-200).
 */
int sp24_spmm_mlp(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc, int64_t ms, int64_t k,
                  const void *b, int64_t ld_b, int64_t n, void *out, int64_t ld_out, const void *bias, int bias_is_f32,
                  int epilogue, void *aux, int64_t ld_aux, int *status, void *stream);

/*
 * sp24_spmm for float8 operands with the dequantisation folded into the epilogue:
 *   D (float32) = alpha * (A_sparse * B) [+ bias[row]] [activation],  alpha = product of the per-tensor scales.
 * Both operands K-major (a_packed row-major (ms, k/2), b stored (n, k)), as for every 8-bit GEMM.  The reference's
 * float8 kernels apply no scale (sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:724-809); its callers multiply the
 * float32 result in a separate pass, which at this output size costs as much as the GEMM.
 */
int sp24_spmm_scaled(const void *a_packed, int dtype, int64_t ld_a, const void *e_tc, int64_t ms, int64_t k, const void *b,
                     int64_t ld_b, int64_t n, float *out, int trans_out, int64_t ld_out, const float *bias, int activation,
                     float alpha, int *status, void *stream);

/*
 * Weight-gradient form of the sparse GEMM with fp32 accumulation into the output:
 *   D (ms x n, fp32, row-major, pitch ld_out) += A_sparse (ms x k) * B (k x n, stored row-major, pitch ld_b).
 * Replaces torch.mm(to_sparse_semi_structured(grad_output.t(), MVUE24=True), input) of the reference's training
 * layer (README.md:190-192 of the reference) followed by the cast of the gradient to fp32 (README.md:211).
 * K is cut into k_splits slices (0 = as many as idle SMs allow); every slice adds its partial product with
 * fp32 reductions in L2, so the caller zeroes D for a plain product, or passes a gradient buffer to accumulate
 * into.  The order of the slice sums is not fixed: results can differ in the last fp32 bits between runs.
 * dtype: SP24_F16 or SP24_BF16 (both operands).  Shape rules: ms % 128 == 0, k % 64 == 0, n % 8 == 0.
 */
int sp24_spmm_accumulate_f32(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *e_tc,
                             int64_t ms, int64_t k, const void *b, int64_t ld_b, int64_t n, float *out,
                             int64_t ld_out, int k_splits, int *status, void *stream);

/*
 * Two streaming kernels of the trainer around the sparse GEMMs.  No counterpart in the reference, whose model and
 * training scripts live in another repository (README.md:18); they replace the framework's generic kernels where those
 * dominate a training step of the GPT-2 configuration (float32 layer norm + cast, its gamma / beta gradient, float32
 * copies of the logits around log-softmax).
 *
 * Layer normalisation over the last dimension, one warp per row: x float32 (rows, d) contiguous, d % 128 == 0,
 * d <= 1024; out in out_dtype (F32 / F16 / BF16: the 16-bit operand of the next GEMM is written directly); mean and
 * rstd (rows floats each) are kept for the backward pass, which takes dy in F32 / F16 / BF16, writes dx (float32) and
 * ADDS the gamma / beta gradients into dgamma / dbeta (d floats each, float32 atomics: zero them or pass gradient
 * buffers to accumulate into).
 */
int sp24_layernorm_fwd(const float *x, const float *gamma, const float *beta, void *out, int out_dtype, float *mean,
                       float *rstd, int64_t rows, int64_t d, float eps, void *stream);
int sp24_layernorm_bwd(const void *dy, int dy_dtype, const float *x, const float *gamma, const float *mean,
                       const float *rstd, float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t d, void *stream);

/*
 * The same two kernels with the residual connection of a pre-norm transformer block folded in.
 *   forward:  res_out = x + delta (float32; delta has the type of `out`: the branch output that joins the residual
 *             stream), out = layer_norm(res_out); mean / rstd as above.  res_out may alias x.
 *   backward: dx = layer-norm input gradient (from dy and x = the saved res_out) + dres, where dres (float32 or NULL)
 *             is the gradient arriving along the residual stream; ddelta (dy's type, or NULL) receives the same
 *             values: the gradient of the branch.  dx may alias dres.
 * One pass over the residual stream per direction instead of three (add, norm, cast / accumulate).
 */
int sp24_add_layernorm_fwd(const float *x, const void *delta, float *res_out, const float *gamma, const float *beta, void *out,
                           int out_dtype, float *mean, float *rstd, int64_t rows, int64_t d, float eps, void *stream);
int sp24_add_layernorm_bwd(const void *dy, int dy_dtype, const float *dres, const float *x, const float *gamma,
                           const float *mean, const float *rstd, float *dx, void *ddelta, float *dgamma, float *dbeta,
                           int64_t rows, int64_t d, void *stream);

/*
 * Cross entropy over 16-bit logits (rows, v) with row pitch ld, v % 8 == 0, int64 class targets in [0, v); float32
 * arithmetic, one block per row, each logit read once per pass.
 *   forward:  lse[row] = log sum_c exp(logits[row, c]);  loss[row] = lse[row] - logits[row, target[row]]
 *   backward: dlogits[row, c] = (exp(logits[row, c] - lse[row]) - [c == target[row]]) * scale * (*upstream),
 *             upstream a device float (the gradient of the summed loss) or NULL for 1; scale e.g. 1 / rows for a mean.
 *             dlogits has the logits' type and may alias logits.
 * A target outside [0, v) reads no logit: its row's loss is 0 and no entry of its gradient row has the 1 subtracted.
 */
int sp24_cross_entropy_fwd(const void *logits, int dtype, const int64_t *targets, float *lse, float *loss, int64_t rows,
                           int64_t v, int64_t ld, void *stream);
int sp24_cross_entropy_bwd(const void *logits, int dtype, const int64_t *targets, const float *lse, const float *upstream,
                           float scale, void *dlogits, int64_t rows, int64_t v, int64_t ld, int64_t ld_out, void *stream);

/*
 * Both passes in one launch, for a loss whose upstream gradient is 1 (a training loss that is differentiated directly):
 * lse and loss as the forward above, and dlogits = (softmax - onehot) * scale written from the same read of the row
 * (kept in shared memory when it fits: v * 2 bytes <= 110 KB; otherwise re-read).  dlogits may alias logits;
 * scale >= 0 and finite.
 * sp24_scale_unless_one multiplies `count` 16-bit values (count % 8 == 0) by the device float *factor, and does
 * nothing (no read, no write) when that is exactly 1: the backward pass of the fused form.
 */
int sp24_cross_entropy_fused(const void *logits, int dtype, const int64_t *targets, float *lse, float *loss, float scale,
                             void *dlogits, int64_t rows, int64_t v, int64_t ld, int64_t ld_out, void *stream);
int sp24_scale_unless_one(void *g, int dtype, const float *factor, int64_t count, void *stream);

/*
 * GELU, tanh form, over `count` contiguous 16-bit values (count % 8 == 0), float32 arithmetic:
 *   dy == NULL: out = gelu(x);   dy != NULL: out = dy * gelu'(x)   (out may alias x or dy).
 * The same formula as the GEMM epilogues of sp24_spmm / sp24_spmm_mlp (tanh.approx).
 */
int sp24_gelu(const void *x, const void *dy, void *out, int dtype, int64_t count, void *stream);

/*
 * Token + learned position embedding of a decoder (float32 tables, d % 4 == 0), one warp per token:
 *   forward:  out[row, :] = wte[ids[row], :] + wpe[row % t, :]          rows = batch * t tokens, ids int64
 *   backward: dwte[ids[row], :] += dx[row, :];  dwpe[row % t, :] += dx[row, :]   (float32 vector reductions: the
 *             gradient tables must hold what the sums are to be added to, e.g. zeros; rows that share a token or a
 *             position are added in no fixed order, so sums can differ in the last bit from run to run)
 * An id outside [0, vocab) reads as a zero row and receives no gradient.  Stands where the framework's sort-based
 * embedding gradient (a dozen launches) sat in the GPT-2 step; no counterpart in the reference.
 */
int sp24_embedding_fwd(const int64_t *ids, const float *wte, const float *wpe, float *out, int64_t rows, int64_t t, int64_t d,
                       int64_t vocab, void *stream);
int sp24_embedding_bwd(const float *dx, const int64_t *ids, float *dwte, float *dwpe, int64_t rows, int64_t t, int64_t d,
                       int64_t vocab, void *stream);

/*
 * Self-test of the failure path of the GEMM kernels: launches one CTA that waits, with a limit of `polls`
 * polls (1 .. 2^20), on a barrier nothing signals.  The wait gives up, *status (a device int the caller
 * zeroed) becomes 9 and the kernel returns normally; the context stays usable.  No counterpart in the
 * reference (its kernels have no bounded waits).
 */
int sp24_selftest_bounded_wait(int *status, int polls, void *stream);

/*
 * The same GEMM for callers that cannot allocate device memory where they call it (a host that replays
 * a fixed memory plan, a loop that must stay clear of the allocator, a plug-in inside an application
 * that owns all GPU memory).  No counterpart in the reference.  It takes the metadata in the
 * reference's reordered layout (what sp24_prune_compress writes) and keeps the tensor-core copy in a
 * 4 MiB array that is part of the library image, so nothing is allocated by this call, by the caller
 * or by any library routine.  Limits and rules:
 *   - ms * k must not exceed 32 Mi elements (sp24_spmm_noalloc_max_bytes() is the array size that
 *     sp24_meta_tc_bytes(ms, k) has to fit in); larger problems return SP24_ERR_TOO_LARGE;
 *   - the first call on each device looks up the array's device address; make that call before any
 *     CUDA stream capture begins on that device;
 *   - all calls share the one array and each call overwrites the part it uses, so two calls that can
 *     overlap on the GPU (different streams, no dependency) race; order them on one stream or with
 *     events;
 *   - every GPU that loads the library holds the 4 MiB until the process exits.
 * All other arguments are those of sp24_spmm.
 */
int64_t sp24_spmm_noalloc_max_bytes(void);
int sp24_spmm_noalloc(const void *a_packed, int dtype, int a_mn_major, int64_t ld_a, const void *meta, int64_t ms,
                      int64_t k, const void *b, int b_mn_major, int64_t ld_b, int64_t n, void *out, int out_dtype,
                      int trans_out, int64_t ld_out, const void *bias, int activation, int *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SPARSE24_B200_H */
