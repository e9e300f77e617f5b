/*
 * C ABI of the B200 (sm_100a) Newton-Schulz / Muon-step library.
 *
 * Plain pointers and sizes only.  Every pointer named "device" is a CUDA device
 * pointer owned by the caller; the library never allocates or frees device
 * memory.  Every entry point returns 0 when its work was enqueued on `stream`
 * and a negative I8M_E_* code otherwise (i8m_last_error() gives the message);
 * nothing is thrown and nothing synchronises the stream.  Device-side waits are
 * bounded: a kernel that gives up writes a non-zero code to the caller's
 * `status` word (one 32-bit word, zeroed by the caller) instead of hanging.
 *
 * Each declaration cites the interface of the reference implementation
 * (Triang-jyed-driung/i8muon, paths relative to that project) that it replaces.
 * The stage-level functions replace the reference's three pybind11 modules one
 * operator at a time; the i8m_ns_* functions replace the Python drivers that
 * sequence those operators; i8m_momentum / i8m_apply replace the elementwise
 * torch calls of the optimizer step.
 */
#ifndef I8MUON_B200_H
#define I8MUON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* i8m_stream_t; /* cudaStream_t */

enum i8m_error {
  I8M_OK = 0,
  I8M_E_ARGUMENT = -1,  /* invalid shape, dtype, mode or null pointer */
  I8M_E_WORKSPACE = -2, /* workspace too small */
  I8M_E_CUDA = -3,      /* a CUDA runtime or driver call failed */
  I8M_E_LIMIT = -4      /* size beyond a documented maximum */
};

/* storage dtypes of user tensors and of the floating compute path */
enum i8m_dtype { I8M_F32 = 0, I8M_F16 = 1, I8M_BF16 = 2 };

/* Newton-Schulz routes; mirror RoutingMixin.router, src/i8muon/_optimizer.py:73-93 */
enum i8m_route {
  I8M_ROUTE_FLOAT = 0,   /* _regular_prec  */
  I8M_ROUTE_GRAM = 1,    /* _gram_prec     */
  I8M_ROUTE_INT8 = 2,    /* _regular_i8    */
  I8M_ROUTE_BQ_INT8 = 3, /* _regular_bq, int8 blocks */
  I8M_ROUTE_BQ_FP8 = 4,  /* _regular_bq, E4M3 blocks */
  I8M_ROUTE_INT8_FACTORED = 5, /* _regular_i8_factored: coefficient rows are (c, p, q) of
                                 c * ((G + p I)^2 + q I), src/i8muon/_cutlass.py:93-128 */
  I8M_ROUTE_INT8_CUBIC = 6    /* _regular_i8_grouped_cubic / _regular_i8_cubic_abc (src/i8muon/_cutlass_cubic.py:8-87):
                                 row 0 is (input_gain, 0, 0), rows 1 .. steps-2 are (gain, diagonal shift, 0) of
                                 T <- -gain (T T^T + shift I) T, the last row is the terminal quintic (a, b, c);
                                 always all-INT8, fp16_first is ignored */
};

/* ---- library state ------------------------------------------------------ */
int i8m_version(void);
/* "arch=sm_100a cuda=<ver> tile=128x128 ..." ; static storage */
const char* i8m_build_info(void);
/* message of the last failing call on this thread; static storage */
const char* i8m_last_error(void);
/* number of kernels this library has launched in this process (every stage kernel
 * and GEMM counts once; memsets do not); used to report launches per step */
unsigned long long i8m_launch_count(void);
/* tests only: 1 replaces the TMA/tcgen05 mainloop by plain dot products inside
 * the epilogue threads (same epilogues); 2 keeps the tensor-core kernels of the block-quantised
 * GEMMs but makes their producers issue no copy, so that every bounded device-side wait runs
 * out (about two seconds), the status word receives a code and the kernel returns with nothing
 * in flight; 0 restores the normal path.  Per calling thread. */
int i8m_set_debug_core(int simt);
/* Kernel variants a host-side tuner can choose between, the counterpart of the tile ids
 * that the reference's KernelFactory times (src/i8muon/_cuda_factory.py:62-102).
 * operation "bq_gemm": 0 = tile tail on its own warpgroup (default), 1 / 2 = fused tail with a
 * six- / four-stage operand ring.
 * operation "wholek_gemm" (FP16/BF16/global-INT8 products): 0 = persistent kernel over units of
 * 128 x 256 (default), 1 = persistent kernel with two streams of 128 x 128 tiles, 2 = one CTA per
 * output tile.  All variants of an operation give bit-identical results.
 * The choice belongs to the calling thread (two engines on two threads never see each other's)
 * and applies to the stage-level launches that thread makes afterwards; i8m_ns_run takes its own
 * selection as an argument. */
int i8m_variant_count(const char* operation);
/* The persistent GEMM kernels launch one CTA per SM and each CTA owns its SM's whole register file, so no
 * other kernel can run beside them.  A multi-GPU step that overlaps a collective (an SM kernel) with the
 * GEMMs caps their grid instead: at most max_ctas CTAs per launch (0 = one per SM), which leaves the other
 * SMs to the collective.  Per calling thread, like the variant selection.  No counterpart in the reference
 * (it is single-device). */
int i8m_set_cta_limit(int max_ctas);
int i8m_set_variant(const char* operation, int variant);

/* ---- stage level: statistics ---------------------------------------------
 * norm[b] = ||x_b||_F (FP32 accumulate, deterministic two-pass) and
 * amax[b] = max|x_b| in one read.  Either output may be NULL.
 * Replaces stats (src/i8muon/csrc/int8.cu:492-506) and the torch norm calls
 * (src/i8muon/_cutlass.py:190, _cutlass_prec.py:66-73, _cutlass_bq.py:42).
 * scratch: 2 * batch * ceil(count / 8192) floats of device memory. */
int i8m_stats_scratch_bytes(int batch, long long count, size_t* bytes);
int i8m_stats(const void* x_device, int dtype, int batch, long long count, void* scratch_device,
              size_t scratch_bytes, float* norm_device, float* amax_device, i8m_stream_t stream);

/* One-pass flavour (deterministic=False of the reference: fused sum of squares with atomics,
 * src/i8muon/csrc/int8.cu:41-62): one launch; the floating-point summation order is not reproducible.
 * scratch: 3 * batch 32-bit words of device memory (cleared by the call). */
int i8m_stats_onepass(const void* x_device, int dtype, int batch, long long count, void* scratch_device,
                      size_t scratch_bytes, float* norm_device, float* amax_device, i8m_stream_t stream);

/* Same result as i8m_stats for callers that cannot allocate device memory.
 * No counterpart in the reference.  Some hosts of this library never get to call
 * cudaMalloc: plugins that were handed a fixed memory budget by their framework,
 * code on a latency-critical thread where a call that may synchronise the device
 * is forbidden, or callers whose allocator is not reachable from the thread they
 * are on.  For them the
 * two-pass reduction keeps its partials in a 4 MiB array that is part of the
 * library image on every GPU that loads the library (held until process exit).
 *   limit     batch * ceil(count / 8192) <= 524288, otherwise I8M_E_LIMIT
 *   set-up    the first call on each device looks up the array's device address
 *             (with that device current); that first call should come before any
 *             stream capture begins
 *   sharing   all calls on a device use the same array: calls whose kernels can
 *             overlap on the GPU (different streams) race and must be serialised
 *             by the caller; nothing needs clearing between calls because every
 *             partial read is written earlier in the same call
 * Allocates nothing: no cudaMalloc / cudaFree and no allocating library routine. */
int i8m_stats_static(const void* x_device, int dtype, int batch, long long count,
                     float* norm_device, float* amax_device, i8m_stream_t stream);

/* ---- stage level: floating path -------------------------------------------
 * normalize: src/i8muon/csrc/prec.cu:193-208.  A = E(x / max(norm, eps)) padded to
 * (lp x hp) plus A^T; transpose != 0 means the input has rows > cols and A = x^T.
 * For compute_dtype F32 every matrix is a pair of planes (hi, lo) of TF32-
 * representable floats; *_lo pointers are required then and ignored otherwise. */
int i8m_normalize(const void* x_device, int in_dtype, const float* norm_device, void* a, void* a_t,
                  void* a_lo, void* a_t_lo, int compute_dtype, int batch, int rows, int cols,
                  int lp, int hp, int transpose, float eps, i8m_stream_t stream);
/* gemm: src/i8muon/csrc/prec.cu:248-256.  out = left * right_t^T with the fused
 * epilogue selected by mode (0 plain, 1 polynomial ca*I + cb*left + cc*acc) and
 * `final` (cast to out_dtype, un-pad to lm x ln, optional transposed store). */
int i8m_float_gemm(const void* left, const void* left_lo, const void* right_t,
                   const void* right_t_lo, void* out, void* out_t, void* out_lo, void* out_t_lo,
                   int compute_dtype, int mode, int batch, int m, int n, int k, int lm, int ln,
                   int symmetric, int final, int transpose, int out_dtype, float ca, float cb,
                   float cc, uint32_t* status_device, i8m_stream_t stream);

/* The update product of an FP16 / BF16 iteration whose result leaves as 128 x 128 block-quantised INT8
 * operands: out = left * right_t^T is rounded to `compute`, then to `user_dtype` (what the floating route
 * stores, src/i8muon/csrc/prec.cu:159-164), and each 128 x 128 CTA tile takes its maximum, scale and codes as
 * quant does with inv = 1 (src/i8muon/csrc/bq.cu:41-101): q (batch, lp, hp), q_t (batch, hp, lp), scale
 * (batch, lp/128, hp/128), lp / hp = m / n rounded up to 128.  Replaces, for the fp16-first INT8-BQ call,
 * the final store of gemm (prec.cu) plus quant (bq.cu) of src/i8muon/_cutlass.py:137-142. */
int i8m_float_gemm_to_bq(const void* left, const void* right_t, void* q, void* q_t, float* scale, int compute,
                         int user_dtype, int batch, int m, int n, int k, int lm, int ln, int lp, int hp,
                         uint32_t* status_device, i8m_stream_t stream);

/* ---- stage level: global-scale INT8 path --------------------------------- */
/* input_quant: src/i8muon/csrc/int8.cu:508-527 (norm_device NULL = no normalisation) */
int i8m_input_quant(const void* x_device, int in_dtype, const float* amax_device,
                    const float* norm_device, int8_t* a8, int8_t* a8_t, float* a_scale, int batch,
                    int rows, int cols, int lp, int hp, int transpose, float eps,
                    i8m_stream_t stream);
/* aat / square / update: src/i8muon/csrc/int8.cu:529-537, 539-556, 592-627.
 * mode 0: out int32 (lower tiles), maximum int32[batch];
 * mode 1: out fp32, maximum fp32[batch], alpha = b, beta = c coefficient;
 * mode 2: out fp32 + maximum, or (final) the user's tensor in out_dtype;
 * mode 4: mode 2 with b_scale multiplied by alpha (factored_update, int8.cu:258, 606-627). */
int i8m_i8_gemm(int mode, const int8_t* a, const int8_t* b_t, const int8_t* row_b, void* out,
                void* maximum, const float* a_scale, const float* b_scale, const float* diag,
                int batch, int m, int n, int k, int lm, int ln, float alpha, float beta, int final,
                int transpose, int out_dtype, uint32_t* status_device, i8m_stream_t stream);
/* symmetric_quant: src/i8muon/csrc/int8.cu:558-585 (quad 0: int32 Gram in, c0 is added to the FP32
 * diagonal - the shift of factored_quant, int8.cu:396, 0 otherwise; quad 1: fp32 polynomial in) */
int i8m_symmetric_quant(const void* input, const void* maximum, const float* orig_scale,
                        const float* orig_diag, int8_t* output, float* scale, float* diag,
                        int batch, int m, int quad, float c0, float c1, float c2,
                        i8m_stream_t stream);
/* output_quant: src/i8muon/csrc/int8.cu:629-638 */
int i8m_output_quant(const float* input, const float* maximum, int8_t* out, int8_t* out_t,
                     float* scale, int batch, int m, int n, i8m_stream_t stream);

/* ---- stage level: 128x128 block-quantised path ---------------------------- */
/* quant: src/i8muon/csrc/bq.cu:301-313 */
int i8m_bq_quant(const void* x_device, int in_dtype, const float* norm_device, void* a, void* a_t,
                 float* scale, int fp8, int batch, int rows, int cols, int lp, int hp,
                 int transpose, float eps, i8m_stream_t stream);
/* gemm: src/i8muon/csrc/bq.cu:343-355 (mode 0 Gram, 1 polynomial, 2 update) */
int i8m_bq_gemm(int fp8, int mode, const void* a, const float* sa, const float* da, const void* b_t,
                const float* sb, const void* row_b, void* out, void* out_t, float* so, float* dout,
                int batch, int m, int n, int k, int lm, int ln, float ca, float cb, float cc,
                int final, int transpose, int out_dtype, uint32_t* status_device,
                i8m_stream_t stream);

/* ---- whole Newton-Schulz call ---------------------------------------------
 * Replaces the Python drivers floating (src/i8muon/_cutlass_prec.py:30-131),
 * _regular_i8 / _regular_i8_impl (src/i8muon/_cutlass.py:130-142, 162-251) and
 * regular_bq (src/i8muon/_cutlass_bq.py:15-70).
 *   x, out       (batch, rows, cols) contiguous in `dtype`; out may not alias x
 *   compute      floating routes: I8M_F32 / I8M_F16 / I8M_BF16 (ignored otherwise)
 *   coeffs       steps rows of (a, b, c), host memory
 *   fp16_first   INT8 and BQ-INT8 routes: first row in FP16, rest quantised
 *   deterministic  non-zero: two-pass statistics with a fixed summation order; zero: the one-pass
 *                flavour with atomics (src/i8muon/_cutlass.py:189-194), one launch fewer, sum order free
 *   variants     kernel variants for this call: -1 = the calling thread's i8m_set_variant choices,
 *                otherwise (bq_gemm variant) | (wholek_gemm variant << 8) | (its variant for the
 *                polynomial product of the global-INT8 route << 16) | (for that route's update
 *                product << 24), bits 8-15 then being the Gram product's; the thread's own choices
 *                are untouched
 *   gram_order   GRAM route: restart string such as "00100" (NULL = default)
 *   stats_partials  NULL, or the partials that i8m_momentum left for x (same batch and element count)
 *   workspace    device memory of at least i8m_ns_workspace_bytes(...) bytes,
 *                256-byte aligned; contents are scratch
 */
int i8m_ns_workspace_bytes(int route, int batch, int rows, int cols, int dtype, int compute,
                           int steps, int fp16_first, size_t* bytes);
int i8m_ns_run(int route, const void* x_device, void* out_device, int dtype, int batch, int rows,
               int cols, int compute, const double* coeffs, int steps, float eps, int fp16_first,
               int deterministic, int variants, const char* gram_order, const float* stats_partials_device, void* workspace_device, size_t workspace_bytes,
               uint32_t* status_device, i8m_stream_t stream);

/* ---- optimizer step kernels ------------------------------------------------
 * momentum: buf <- lerp(buf, grad, 1 - mu2); update = nesterov ? lerp(grad, buf, mu) : buf
 * for `count` same-shaped tensors given as host arrays of device pointers; the
 * updates are written stacked into update_device (count x numel).  Replaces
 * src/i8muon/_optimizer.py:472-474.  stats_partials (optional, i8m_stats_scratch_bytes(count, numel) bytes):
 * the kernel also leaves the per-chunk sums of squares and maxima of the update it writes, in the scratch
 * layout of i8m_stats; handed to i8m_ns_run they replace its statistics pass over the update (the torch
 * norm of src/i8muon/_cutlass_prec.py:66-73, _cutlass.py:190, _cutlass_bq.py:42) by the final fold alone,
 * with a bit-identical norm. */
int i8m_momentum(const void* const* grads, void* const* bufs, int count, void* update_device,
                 long long numel, int dtype, float buf_weight, float mu, int nesterov,
                 float* stats_partials_device, i8m_stream_t stream);
/* apply: decay_mode 0 none, 1 param *= decay, 2 update += decay * param; then
 * param += neg_lr * update.  Replaces src/i8muon/_optimizer.py:503-511. */
int i8m_apply(void* const* params, int count, const void* update_device, long long numel,
              int param_dtype, int update_dtype, int decay_mode, float decay, float neg_lr,
              i8m_stream_t stream);

/* AdamW for the parameters Muon does not take (embeddings, heads, vectors).  No counterpart in
 * the reference: its `scalar_optimizer` slot takes any torch optimizer
 * (src/i8muon/_optimizer.py:223,254-255); this is the fused companion for that slot.
 * `count` tensors of possibly different sizes (numel[i]) as host arrays of device pointers;
 * FP32 moments; decoupled decay.  Per element: p *= 1 - lr*weight_decay;
 * m = lerp(m, g, 1-beta1); v = beta2*v + (1-beta2)*g*g;
 * p -= lr/bias_correction1 * m / (sqrt(v)/sqrt(bias_correction2) + eps),
 * with bias_correction_k = 1 - beta_k^step computed by the caller. */
int i8m_adamw(void* const* params, const void* const* grads, float* const* exp_avg,
              float* const* exp_avg_sq, const long long* numel, int count, int param_dtype,
              int grad_dtype, float lr, float beta1, float beta2, float eps, float weight_decay,
              float bias_correction1, float bias_correction2, i8m_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* I8MUON_B200_H */
