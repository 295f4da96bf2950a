/*
 * cpmk_b200 -- C ABI of the B200 (sm_100a) implementation of cpm_kernels' int8-quantised linear
 * layer and fp16 decode GEMV.
 *
 * Conventions (they mirror cpm_kernels/kernels/*.py, whose functions these replace one for one):
 *   - every tensor argument is a raw device address; the caller owns all tensors;
 *   - sizes are int32; `stream` is a cudaStream_t (CUstream) value, 0 = the legacy default stream;
 *   - all work is enqueued on `stream` and the call returns without synchronising;
 *   - the return value is 0 on success, a CPMK_E* code otherwise; cpmk_last_error() returns a
 *     thread-local description of the last failure.  Nothing throws, traps or calls exit();
 *   - tensors are row-major and contiguous; fp16 = IEEE binary16.
 *
 * File:line citations name the interface of the reference (OpenBMB/cpm_kernels v1.0.11) that each
 * entry point replaces.
 */
#ifndef CPMK_B200_H_
#define CPMK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CPMK_ABI_VERSION 1

enum {
    CPMK_OK = 0,
    CPMK_EINVAL = 1,       /* bad size / null pointer / misaligned pointer                       */
    CPMK_EARCH = 2,        /* the current device is not compute capability 10.x                  */
    CPMK_ECUDA = 3,        /* a CUDA runtime / driver call failed (text in cpmk_last_error)      */
    CPMK_EDEVICE = 4,      /* a kernel reported a bounded-wait timeout through the status word   */
    CPMK_ENOMEM = 5        /* the library's own workspace could not be allocated or is too small */
};

typedef void *cpmk_stream_t;

int32_t cpmk_abi_version(void);
const char *cpmk_last_error(void);

/* Compute capability (major*10+minor) of the current device; CPMK_EARCH unless it is 10.x.
 * Replaces the architecture gate of cpm_kernels/device/__init__.py:143-145. */
int32_t cpmk_check_device(int32_t *arch_out);

/* Reads (and clears) the per-device status word that kernels with bounded waits set when a wait
 * runs out: 0 = no error.  Synchronises the device.  No counterpart in the reference (its cublasLt
 * GEMM has no user-visible waits). */
int32_t cpmk_read_status(uint32_t *status_out);

/* Waits for `stream`, then reports whether a kernel that ran on it gave up a bounded wait: CPMK_EDEVICE (with the
 * kernel's code in cpmk_last_error) if so, CPMK_OK otherwise.  After a failure the status word and the library's
 * ticket counters of that stream are cleared, so later calls on the stream work again; what the failed kernel should
 * have written is undefined.  Unlike cpmk_read_status it synchronises one stream, not the device.  No counterpart
 * in the reference. */
int32_t cpmk_check_stream(cpmk_stream_t stream);

/* Frees the library's workspace of (current device, stream): call it before destroying a stream that ran calls which
 * use the workspace (int8 / fp16 GEMM, column quantisation, transposed GEMV, layer norm), so that a process that
 * creates and destroys streams does not accumulate 16 MiB per stream.  Waits for the device.  At most 256 streams per
 * device hold a workspace at a time (CPMK_ENOMEM beyond).  No counterpart in the reference. */
int32_t cpmk_release_workspace(cpmk_stream_t stream);

/* Self-test of the give-up path of the library's device-side waits: a one-block kernel waits up to `limit_us`
 * microseconds (1..100000) on a barrier on which nothing arrives.  Returns CPMK_OK when the wait ran out, the kernel
 * recorded its code (0x901) in the stream's status word and returned; the next cpmk_check_stream on that stream
 * then returns CPMK_EDEVICE once.  Synchronises the stream.  No counterpart in the reference. */
int32_t cpmk_selftest_bounded_wait(uint32_t limit_us, cpmk_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Quantisation passes (cuda/gemm.cu)
 * ------------------------------------------------------------------------------------------ */

/* kernels/gemm.py:91-107 gemm_calc_scale -> cuda/gemm.cu:60-76.
 * mat (batch, n, m) fp16; out (batch, n) fp16 = half(max_i |mat[b,r,i]| / 127). */
int32_t cpmk_gemm_calc_scale(int32_t batch, int32_t n, int32_t m, const void *mat, void *out, cpmk_stream_t stream);

/* kernels/gemm.py:109-125 gemm_calc_scale_transpose -> cuda/gemm.cu:79-98.
 * inp (batch, n, m) fp16; out (batch, m) fp16 = half(max_r |inp[b,r,c]| / 127). */
int32_t cpmk_gemm_calc_scale_transpose(int32_t batch, int32_t n, int32_t m, const void *inp, void *out, cpmk_stream_t stream);

/* kernels/gemm.py:21-41 gemm_round -> cuda/gemm.cu:6-18.
 * out[b,r,i] = (int8) nearbyintf((float)mat[b,r,i] / (float)scale[b,r]). */
int32_t cpmk_gemm_round(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale, void *out, cpmk_stream_t stream);

/* kernels/gemm.py:43-63 gemm_round_transpose -> cuda/gemm.cu:22-33.  scale is (batch, m). */
int32_t cpmk_gemm_round_transpose(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale, void *out, cpmk_stream_t stream);

/* Fused gemm_calc_scale + gemm_round (cpm_kernels/torch/gemm.py:98-102 calls them back to back on
 * the same tensor): one read of `mat`, writes both scale_out (batch, n) and q_out (batch, n, m). */
int32_t cpmk_quantize_rows(int32_t batch, int32_t n, int32_t m, const void *mat, void *scale_out, void *q_out, cpmk_stream_t stream);

/* cpmk_quantize_rows on two operands whose rows have the same length m, in one launch: (batch0, n0, m) and
 * (batch1, n1, m), e.g. the activations and the weight of a linear layer, which cpm_kernels/torch/gemm.py:98-102
 * quantises back to back.  Same results as two cpmk_quantize_rows calls. */
int32_t cpmk_quantize_rows_pair(int32_t batch0, int32_t n0, const void *mat0, void *scale_out0, void *q_out0,
                                int32_t batch1, int32_t n1, const void *mat1, void *scale_out1, void *q_out1,
                                int32_t m, cpmk_stream_t stream);

/* cpmk_quantize_rows_pair whose FIRST operand (n0, m) is written to `n_dst` (1..8) destinations: scale_dst0[i] and
 * q_dst0[i] are where the scales (n0) and codes (n0, m) of these rows go in destination i -- this GPU's buffers and
 * its peers', mapped into this process.  Rank r of g holds rows [r*M/g, (r+1)*M/g) of the activations, quantises them
 * once, and the stores of the quantising kernel place them at that row offset of every rank's full code buffer: the
 * all-gather of the int8 activations (1 byte per element over NVLink instead of g uploads of 2 bytes per element)
 * happens inside the quantisation pass.  Per-row quantisation makes the gathered codes and scales identical to those
 * of the unsharded tensor.  The second operand (n1, m) -- this rank's weight rows -- is quantised into local buffers
 * by the same launch; n1 may be 0.  m must be a multiple of 8 and at most 16384; otherwise CPMK_EINVAL.
 * The caller synchronises the ranks.  No counterpart in the reference (it has no multi-GPU code). */
int32_t cpmk_quantize_rows_pair_scatter(int32_t n0, const void *mat0, int32_t n_dst, void *const *scale_dst0, void *const *q_dst0,
                                        int32_t n1, const void *mat1, void *scale_out1, void *q_out1, int32_t m, cpmk_stream_t stream);

/* Fused gemm_calc_scale_transpose + gemm_round_transpose (same call sites, transposed operand):
 * writes scale_out (batch, m) and q_out (batch, n, m).  Uses the library workspace. */
int32_t cpmk_quantize_cols(int32_t batch, int32_t n, int32_t m, const void *mat, void *scale_out, void *q_out, cpmk_stream_t stream);

/* kernels/gemm.py:65-89 gemm_scale -> cuda/gemm.cu:37-57.
 * mat int32 (batch, n, m); scale_x (batch or 1, n); scale_y (batch or 1, m); out fp16 (batch, n, m)
 * out = half(((float)mat * sx) * sy). */
int32_t cpmk_gemm_scale(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_x, const void *scale_y,
                        void *out, int32_t broad_cast_x, int32_t broad_cast_y, cpmk_stream_t stream);

/* kernels/gemm.py:309-347 gemm_scale_x / gemm_scale_y -> cuda/gemm.cu:176-205. */
int32_t cpmk_gemm_scale_x(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_x, void *out, cpmk_stream_t stream);
int32_t cpmk_gemm_scale_y(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_y, void *out, cpmk_stream_t stream);

/* kernels/gemm.py:261-283 gemm_backward_round_scale -> cuda/gemm.cu:103-134. */
int32_t cpmk_gemm_backward_round_scale(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_y, void *out,
                                       void *scale_x, int32_t broad_cast_y, cpmk_stream_t stream);
/* kernels/gemm.py:285-307 gemm_backward_scale_round -> cuda/gemm.cu:137-172. */
int32_t cpmk_gemm_backward_scale_round(int32_t batch, int32_t n, int32_t m, const void *mat, const void *scale_x, void *out,
                                       void *scale_y, int32_t broad_cast_x, cpmk_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * int8 GEMM (replaces the cublasLt call)
 * ------------------------------------------------------------------------------------------ */

/* kernels/gemm.py:127-186 gemm_int8 -> library/cublaslt.py:126-150 cublasLtMatmul.
 * A int8 (batchA, k, m), or (batchA, m, k) when aT;  B int8 (batchB, n, k), or (batchB, k, n) when bT;
 * out int32 (max(batchA,batchB), n, m):  out[b,j,i] = sum_l Aop[b,l,i] * Bop[b,j,l].
 * batchA, batchB equal or 1 (broadcast).  m, n, k multiples of 4 (the reference's assert). */
int32_t cpmk_gemm_int8(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT,
                       const void *A, const void *B, void *out, cpmk_stream_t stream);

/* gemm_int8 with gemm_scale fused into its epilogue (cpm_kernels/torch/gemm.py:40-64 runs them back
 * to back through an int32 tensor in HBM).  scale_x is (broad_cast_x ? 1 : batch, n) and multiplies
 * first, scale_y is (broad_cast_y ? 1 : batch, m); out is fp16 (batch, n, m). */
int32_t cpmk_gemm_int8_dequant(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT,
                               const void *A, const void *B, const void *scale_x, const void *scale_y,
                               int32_t broad_cast_x, int32_t broad_cast_y, void *out, cpmk_stream_t stream);

/* cpmk_gemm_int8_dequant whose fp16 result is stored to `n_dst` (1..8) destinations instead of one: dst[i] is the
 * address of element (0, 0, 0) of destination i, every destination has rows `dst_row_pitch` elements apart (>= m,
 * a multiple of 8) and batches n * dst_row_pitch apart.  With one process per GPU and the peers' output buffers mapped
 * into this process (CUDA peer access / symmetric memory), rank r of g computes its N/g columns of y = x W^T and this
 * call writes them straight into columns [r*N/g, (r+1)*N/g) of every rank's full-width y: the all-gather that
 * cpm_kernels' callers would run after a column-parallel linear happens inside the GEMM's epilogue (TMA stores over
 * NVLink), without a second pass over the slice.  No counterpart in the reference (it has no multi-GPU code).
 * Needs the tensor-core kernel (extents and pointers multiples of 16 bytes); otherwise CPMK_EINVAL.
 * dst[0] should be the destination in THIS GPU's memory: when forwarding is switched on (cpmk_set_gemm_forward_sms) the
 * computing CTAs store only there, and a few CTAs of the same grid copy each finished tile from dst[0] to the other
 * destinations (stores over NVLink only).
 * The caller synchronises the ranks (all stores of a call are complete when the call's kernel has finished). */
int32_t cpmk_gemm_int8_dequant_scatter(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT,
                                       const void *A, const void *B, const void *scale_x, const void *scale_y,
                                       int32_t broad_cast_x, int32_t broad_cast_y, int32_t n_dst, void *const *dst,
                                       int64_t dst_row_pitch, cpmk_stream_t stream);

/* One column-parallel int8 linear in one call, all buffers the caller's: cpmk_quantize_rows_pair on the activations
 * x (tokens, k) and this rank's weight rows w (n_local, k), then cpmk_gemm_int8_dequant_scatter of the product into
 * `n_dst` destinations (y[:, r*n_local : (r+1)*n_local] of every rank).  scale_x (tokens), q_x (tokens, k), scale_w
 * (n_local), q_w (n_local, k) receive the quantised operands (what cpm_kernels/torch/gemm.py:107-112 saves for
 * backward).  multicast != 0: n_dst is 2 and dst[1] is the multicast address of the result slice
 * (cpmk_gemm_int8_dequant_multicast).  Replaces the six launches and six allocations of
 * cpm_kernels/torch/gemm.py:86-113 for this layout. */
int32_t cpmk_linear_int8_scatter(int32_t tokens, int32_t k, int32_t n_local, const void *x, const void *w, void *scale_x, void *q_x,
                                 void *scale_w, void *q_w, int32_t n_dst, void *const *dst, int64_t dst_row_pitch, int32_t multicast,
                                 cpmk_stream_t stream);

/* cpmk_gemm_int8_dequant_scatter for buffers that are also mapped through an NVLink multicast object (CUDA multicast
 * objects; torch symmetric memory exposes the address as `multicast_ptr`): dst_local is this GPU's own copy of the
 * result slice, dst_multicast the same slice at the multicast address.  The computing CTAs store to dst_local; the
 * forwarding CTAs of the same grid copy every finished tile to dst_multicast with multimem.st, ONE store that the
 * NVLink switch replicates into every GPU's copy -- each GPU then sends its slice once instead of once per peer.
 * No counterpart in the reference. */
int32_t cpmk_gemm_int8_dequant_multicast(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT,
                                         const void *A, const void *B, const void *scale_x, const void *scale_y,
                                         int32_t broad_cast_x, int32_t broad_cast_y, void *dst_local, void *dst_multicast,
                                         int64_t dst_row_pitch, cpmk_stream_t stream);

/* Layer norm over the MIDDLE axis of mat (batch, n, m) fp16, per-row affine, and quantisation along that same axis,
 * without storing the intermediate tensors: what cpm_kernels runs as four kernels between a layer norm and the int8
 * linear that follows it in the (batch, hidden, seq) layout --
 *   cu_layernorm_forward(eps, rd_mean)                      cuda/layernorm.cu:6-71,  kernels/layernorm.py:18-38
 *   cu_arith_ln_mul (beta == NULL) / cu_arith_ln_mul_add    cuda/arith.cu:97-127,    kernels/arith.py:134-215
 *   cu_gemm_calc_scale_transpose, cu_gemm_round_transpose   cuda/gemm.cu:22-33, 79-98
 * (torch/layernorm.py:8-30 followed by torch/gemm.py:98-102 for an operand B with bT = False).
 * alpha, beta: (n) fp16; scale_out (batch, m) fp16; q_out (batch, n, m) int8.  rd_mean = 0 is the RMS form.
 * Same bits as the chain (the statistics are summed in the reference's order).  m must be a multiple of 8. */
int32_t cpmk_layernorm_quantize_cols(int32_t batch, int32_t n, int32_t m, const void *mat, float eps, int32_t rd_mean,
                                     const void *alpha, const void *beta, void *scale_out, void *q_out, cpmk_stream_t stream);

/* out[b, i] = gelu(mat[b, i]) on fp16, tanh form: replaces cpm_kernels/kernels/gelu.py:14-31 gelu_forward /
 * gelu_inplace_forward (cuda/gelu.cu:6-17); `mat` is (batch, n) contiguous and out may equal mat.  Same bits as the
 * reference's kernel for every fp16 input.  Large inputs use a 65536-entry table that the first call on a device
 * fills on its stream (that call should not be inside a stream capture). */
int32_t cpmk_gelu_forward(int32_t batch, int32_t n, const void *mat, void *out, cpmk_stream_t stream);

/* grad[b, i] = gelu'(mat[b, i]) * grad_out[b, i] on fp16: replaces cpm_kernels/kernels/gelu.py:50-69 gelu_backward
 * (cuda/gelu.cu:20-44), the backward pass of cpm_kernels.torch.gelu (torch/gelu.py:17-32).  The derivative is the
 * reference's expression compiled as the reference compiles it: same bits as its kernel for every (mat, grad_out). */
int32_t cpmk_gelu_backward(int32_t batch, int32_t n, const void *grad_out, const void *mat, void *grad, cpmk_stream_t stream);

/* out[b, c, r] = in[b, r, c] on fp16: replaces cpm_kernels/kernels/transpose.py:11-27 transpose (cuda/transpose.cu:6-22);
 * `in` is (batch, n, m) contiguous, `out` (batch, m, n).  Pure data movement, same bits.  in and out must not overlap. */
int32_t cpmk_transpose(int32_t batch, int32_t n, int32_t m, const void *in, void *out, cpmk_stream_t stream);

/* cpmk_gemm_int8_dequant followed by GELU on the fp16 result, as the feed-forward block applies it after its first
 * linear (cpm_kernels.torch.gelu after bmm): out = gelu(half(((float)acc * sx) * sy)), bit-identical to the two
 * separate calls, enqueued back to back on `stream` so that the activation reads the result out of L2. */
int32_t cpmk_gemm_int8_dequant_gelu(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT,
                                    const void *A, const void *B, const void *scale_x, const void *scale_y,
                                    int32_t broad_cast_x, int32_t broad_cast_y, void *out, cpmk_stream_t stream);

/* fp16 x fp16 -> fp16 GEMM with the argument conventions of cpmk_gemm_int8: out[b, j, i] = sum_l Aop[b, l, i] * Bop[b, j, l].
 * Replaces cpm_kernels/kernels/gemm.py:188-256 gemm_fp16 (cublasLt, CUBLAS_COMPUTE_16F): the int8=False branch of
 * cpm_kernels.torch.bmm (torch/gemm.py:182-239).  Products are accumulated in fp32 (tcgen05 kind::f16 with fp32
 * tensor-memory accumulators) and rounded to fp16 once; the reference accumulates in fp16.  m, n, k even
 * (kernels/gemm.py:200); the tensor-core kernel needs contiguous extents that are multiples of 8 elements and 16-byte
 * aligned pointers, other shapes run on a generic kernel. */
int32_t cpmk_gemm_fp16(int32_t m, int32_t k, int32_t n, int32_t batchA, int32_t batchB, int32_t aT, int32_t bT,
                       const void *A, const void *B, void *out, cpmk_stream_t stream);

/* Keeps the persistent grid of the tensor-core GEMM off `sms` SMs from now on (process-wide), so that kernels of
 * another stream -- a collective, or the quantisation passes of the next layer -- find room to run beside it.
 * 0 = use every SM; a negative value returns the choice to the environment variable CPMK_GEMM_SM_MARGIN.
 * No counterpart in the reference (cublasLt picks its own grid). */
int32_t cpmk_set_gemm_sm_margin(int32_t sms);

/* How many SMs of a scattering GEMM (cpmk_gemm_int8_dequant_scatter with more than one destination) forward finished
 * output tiles from destination 0 to the other destinations instead of computing, from now on (process-wide).
 * 0 = none: every computing CTA stores to all destinations itself; a negative value returns the choice to the
 * environment variable CPMK_GEMM_FORWARD_SMS, and without it to the default (0).
 * No counterpart in the reference. */
int32_t cpmk_set_gemm_forward_sms(int32_t sms);

/* Which GEMM kernel the last cpmk_gemm_int8* / cpmk_gemm_fp16 call on this thread selected:
 * 1 = tcgen05 tensor-core kernel, 2 = generic SIMT kernel.  For tests and the benchmark. */
int32_t cpmk_last_gemm_path(void);

/* Which form of the tensor-core kernel that call used: 1 = one CTA per 128 x 256 tile, 2 = CTA pairs on 256 x 256
 * tiles (tcgen05 cta_group::2), 0 = none (generic kernel).  The environment variable CPMK_GEMM_VARIANT
 * (auto | 1cta | 2cta | generic) overrides the choice.  For tests and the benchmark. */
int32_t cpmk_last_gemm_variant(void);

/* ------------------------------------------------------------------------------------------
 * fp16 decode GEMV (cuda/gemv.cu)
 * ------------------------------------------------------------------------------------------ */

/* kernels/gemv.py:82-148 gemv_fp16 / gemv_fp16_light -> cuda/gemv.cu:79-106.
 * mat (batch, dim_out, dim_in), vec (batch, dim_in), out (batch, dim_out); dim_in even. */
int32_t cpmk_gemv_fp16(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out, cpmk_stream_t stream);

/* kernels/gemv.py:151-216 gemv_fp16_transpose / _light -> cuda/gemv.cu:109-135.
 * mat (batch, dim_in, dim_out).  Uses the library workspace for split partial sums. */
int32_t cpmk_gemv_fp16_transpose(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out, cpmk_stream_t stream);

/* No counterpart in the reference.  Same result as cpmk_gemv_fp16_transpose, for callers that must not trigger a
 * device allocation: serving processes that hand the whole GPU to their own memory pool at start-up (a later
 * cudaMalloc would fail or stall them), code that runs where allocation calls are forbidden by the host
 * application, and latency-critical loops that cannot afford the device-wide synchronisation an allocation implies.  The split partial sums and the
 * tickets that combine them live in a fixed 4 MiB + 16 KiB array inside the library's device image instead of the
 * library workspace; nothing is allocated or freed, by this call or by anything it uses.
 *   Limits: dim_out % 8 == 0, mat 16-byte aligned, batch * dim_out <= 524288 and batch * ceil(dim_out / 256) <= 4096;
 *   beyond them the call returns CPMK_ENOMEM with a message and does nothing.
 *   The first call on each device looks up the array's device address, and -- under CUDA's default lazy module loading --
 *   is also the moment the driver places the part of the library image that holds the array on that device (the one
 *   allocation-like event in this entry point's life, and not one this code makes): make that call early, before any
 *   stream capture and before the process's own pool takes the rest of the memory.
 *   All calls on a device share the one array: two calls that overlap on the GPU (different streams) race. */
int32_t cpmk_gemv_fp16_transpose_noalloc(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out,
                                         cpmk_stream_t stream);

/* Measurement aid, no counterpart in the reference: reads a (rows, row_elems) fp16 matrix once and computes nothing, so
 * that the decode GEMVs can be compared with what merely reading the matrix costs.  mode 0: a plain grid-stride read
 * (16-byte loads, four in flight per thread); mode 1: the launch shape and shared-memory copy pipeline of the streaming
 * row GEMV with the arithmetic left out.  `sink` (at least rows * 2 bytes) is written only if a checksum happens to
 * hit a magic value.  row_elems a multiple of 8, src 16-byte aligned. */
int32_t cpmk_probe_read(int32_t mode, int32_t rows, int32_t row_elems, const void *src, void *sink, cpmk_stream_t stream);

/* kernels/gemv.py:218-283 gemv_broadcast_mat_fp16 / _light -> cuda/gemv.cu:138-164.
 * mat (dim_out, dim_in) shared by all `batch` vectors. */
int32_t cpmk_gemv_broadcast_mat_fp16(int32_t batch, int32_t dim_out, int32_t dim_in, const void *mat, const void *vec, void *out, cpmk_stream_t stream);

/* kernels/gemv.py:18-33 gemv_calc_scale -> cuda/gemv.cu:26-40.  vec (batch, n) -> out (batch,). */
int32_t cpmk_gemv_calc_scale(int32_t batch, int32_t n, const void *vec, void *out, cpmk_stream_t stream);
/* kernels/gemv.py:35-53 gemv_round -> cuda/gemv.cu:43-54. */
int32_t cpmk_gemv_round(int32_t batch, int32_t n, const void *vec, const void *scale, void *out, cpmk_stream_t stream);
/* kernels/gemv.py:56-79 gemv_broadcast_mat_int8 -> cuda/gemv.cu:57-76.  dim_in multiple of 4. */
int32_t cpmk_gemv_broadcast_mat_int8(int32_t batch, int32_t dim_out, int32_t dim_in, const void *scale_mat, const void *mat,
                                     const void *scale_vec, const void *vec, void *out, cpmk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CPMK_B200_H_ */
