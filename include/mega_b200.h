/*
 * mega_b200 — C ABI of the B200 (sm_100a) implementation of Mega's EMA layer
 * and its fused neighbours (TimestepNorm, SequenceNorm, gates, decode step).
 *
 * Conventions shared by every entry point
 *   - Plain pointers and sizes only.  Every pointer is a DEVICE pointer unless
 *     the parameter comment says "host".  The caller allocates every input and
 *     output and keeps it alive until the work queued on `stream` has run.
 *   - The library never allocates, frees or synchronises; every launch goes to
 *     the `stream` argument (a cudaStream_t passed as void*; NULL = default
 *     stream).
 *   - Return value: MEGA_OK or one of the MEGA_ERR_* codes below; nothing is
 *     launched when an argument is rejected.  No exception crosses the ABI and
 *     no kernel traps or asserts.
 *   - Activations may be fp32, bf16 or fp16 (mega_dtype); coefficients,
 *     statistics and recurrent states are always fp32; counts are int64.
 *   - Strides are in ELEMENTS.  An activation tensor is addressed as
 *     base + b*stride_b + d*stride_d + l*stride_l, so both the (B, D, L)
 *     "length last" and the (B, L, D) "channel last" memory orders (and the
 *     time-major (L, B, D) order) are views of the same entry points.
 *   - Padding masks are uint8 (B, L) contiguous, non-zero = padded position.
 *   - Re-entrant: no global state except a launch counter, the test switches of
 *     mega_set_option and, for the fused TimestepNorm -> EMA / EMA / TimestepNorm
 *     calls on large bf16 problems, fixed scratch arrays in device memory (owned by
 *     the library, never allocated or freed by a call): such calls on different
 *     streams are ordered against one another by an event, on the device.
 *
 * "Replaces" comments cite the reference interface each entry point stands in
 * for, as file:line within the fairseq-apollo checkout.
 */
#ifndef MEGA_B200_H_
#define MEGA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MEGA_API __attribute__((visibility("default")))
#else
#define MEGA_API
#endif

#define MEGA_ABI_VERSION 1

enum mega_status {
  MEGA_OK = 0,
  MEGA_ERR_NULL = 1,        /* a required pointer is NULL */
  MEGA_ERR_DTYPE = 2,       /* unknown mega_dtype */
  MEGA_ERR_SHAPE = 3,       /* non-positive or inconsistent extent */
  MEGA_ERR_STRIDE = 4,      /* stride combination the kernels cannot address */
  MEGA_ERR_ALIGN = 5,       /* pointer not aligned for its element type */
  MEGA_ERR_NDIM = 6,        /* ndim outside 1..MEGA_MAX_NDIM */
  MEGA_ERR_UNSUPPORTED = 7, /* valid request this build does not implement */
  MEGA_ERR_CUDA = 8         /* a CUDA launch failed; see mega_last_cuda_error */
};

enum mega_dtype { MEGA_F32 = 0, MEGA_BF16 = 1, MEGA_F16 = 2 };

#define MEGA_MAX_NDIM 32

/* flags of mega_ema_fwd / mega_tsn_ema_fwd */
#define MEGA_EMA_BIDIRECTIONAL 1u /* coefficient arrays hold 2*D rows: causal half then anti-causal half */
#define MEGA_EMA_NO_SHIFT 2u      /* anti-causal half includes lag 0 (reference shift=False) */
#define MEGA_EMA_SILU 4u          /* apply SiLU to (conv + omega*x) before storing */

typedef void* mega_stream_t;

MEGA_API const char* mega_status_string(int status);
MEGA_API const char* mega_last_cuda_error(void);
MEGA_API int mega_abi_version(void);
/* Number of kernels this library has launched in this process (monotonic). */
MEGA_API uint64_t mega_launch_count(void);
/*
 * Process-wide switches meant for tests.  key MEGA_OPT_DISABLE_STREAM (0): non-zero routes every
 * call to the generic kernels instead of the TMA-streamed ones.
 */
#define MEGA_OPT_DISABLE_STREAM 0
#define MEGA_OPT_DISABLE_MMA 1 /* non-zero: skip the tensor-core kernels */
#define MEGA_OPT_MMA_TILE 2    /* 2, 4, 7, 8: force 16-, 32-, 56-, 64-channel tensor-core tiles; 22: 16 channels
                                  with two warps per 16-byte column; 222, 224, 422, 124: forms pipelined along the
                                  sequence (channels / 8, warps per column, depth); 82, 84, 88: the segmented
                                  64-channel form in 2, 4, 8 runs; 71: running state in shared memory;
                                  0: automatic.  A form that does not apply to a call falls back to automatic */
#define MEGA_OPT_WAIT_LIMIT 3    /* > 0: SM cycles after which a bounded device-side wait gives up (default ~2 s) */
#define MEGA_OPT_WITHHOLD_LOAD 4 /* test aid, value k > 0: the tensor-core kernel never issues the TMA load of its
                                    step k (the barrier keeps expecting its bytes), so that every waiter of that
                                    stage runs into the wait limit, the kernel returns early without its final
                                    stores and raises the device error word; nothing faults or traps */
MEGA_API int mega_set_option(int key, int value);
/*
 * Test aid: name of the kernel family of this process's most recent launch ("tsn_ema_mma tile=7 pipe=1",
 * "stream_cl", "rowres", ... or "other").  The string is static; do not free it.
 */
MEGA_API const char* mega_debug_last_kernel(void);
/*
 * Debug aid (synchronises the device): reads the device-side error word that a kernel raises
 * when one of its bounded waits gives up; `reset` != 0 clears it.  host_value is a HOST pointer.
 */
MEGA_API int mega_debug_device_error(int* host_value, int reset);

/*
 * EMA coefficients: p = sigmoid(alpha)*beta, q = 1 - sigmoid(alpha)*sigmoid(delta),
 * gamma_hat = gamma/sqrt(N).  alpha/delta/beta (K,N[,1]) and gamma (K,N) in
 * `param_dtype`; outputs fp32 (K,N).
 * Replaces: MultiHeadEMA._calc_coeffs, fairseq/modules/exponential_moving_average.py:71-80.
 */
MEGA_API int mega_ema_coeffs(const void* alpha, const void* delta, const void* beta, const void* gamma,
                    int param_dtype, int K, int N, float* p, float* q, float* gamma_hat,
                    mega_stream_t stream);

/*
 * EMA convolution kernel k[r,l] = sum_n p*gamma_hat*q^l for l < L; out (K,L) fp32.
 * Replaces: MultiHeadEMA._compute_kernel (exponential_moving_average.py:82-90) and the
 * weight half of ema_parameters_fwd (fairseq/csrc/ops/ema_parameters.cc:37-52).
 */
MEGA_API int mega_ema_kernel(const float* p, const float* q, const float* gamma_hat, int K, int N, int L,
                    float* kernel_out, mega_stream_t stream);

/*
 * Output term of a carried state: bias[b,d,l] = sum_n gamma_hat*q^(l+1)*h[b,d,n]; out (B,D,L) fp32.
 * Replaces: the bias half of ema_parameters_fwd (fairseq/csrc/ops/ema_parameters.cc:54-77).
 */
MEGA_API int mega_ema_bias(const float* q, const float* gamma_hat, const float* h, int B, int D, int N, int L,
                  float* bias_out, mega_stream_t stream);

/*
 * The EMA layer forward: y = conv(k, x*(1-mask)) [+ carried-state term] + omega*x [then SiLU].
 * x, y: activations (B,D,L) by strides.  p, q, gamma_hat: (K,N) with K = D, or 2*D when
 * MEGA_EMA_BIDIRECTIONAL.  omega (D).  pad_mask NULL or (B,L).  h_in NULL or (B,D,N): state
 * carried in; h_out NULL or (B,D,N): state after the last position (ema_hidden).  States are
 * rejected for bidirectional calls.  truncation <= 0 or >= L: full-length kernel; otherwise
 * the kernel support is its first `truncation` taps (bidirectional only, as in the reference).
 * Replaces: BaseMovingLayer.forward (fairseq/modules/base_moving_average.py:120-172) with
 * fftconv / bidirectional_fftconv (fairseq/modules/fused_ops/fftconv.py:13-27,85-100),
 * ema_parameters bias (ema_parameters.cc:54-77) and ema_hidden_fwd (ema_hidden.cc:15-64).
 */
MEGA_API int mega_ema_fwd(const void* x, void* y, int dtype, int B, int D, int L,
                 int64_t x_stride_b, int64_t x_stride_d, int64_t x_stride_l,
                 int64_t y_stride_b, int64_t y_stride_d, int64_t y_stride_l,
                 const float* p, const float* q, const float* gamma_hat, const float* omega, int N,
                 const uint8_t* pad_mask, const float* h_in, float* h_out,
                 unsigned flags, int truncation, mega_stream_t stream);

/*
 * Single-token decode step: h' = p*x + q*h, y = sum_n gamma_hat*h' + omega*x [then SiLU].
 * x, y (B,D) contiguous activations; h_in NULL (zero state) or (B,D,N); h_out (B,D,N), may alias h_in.
 * Replaces: BaseMovingLayer.one_step (base_moving_average.py:105-118) and the L == 1 case of
 * BaseMovingLayer.forward's incremental branch (:144-160).
 */
MEGA_API int mega_ema_step(const void* x, void* y, int dtype, int B, int D,
                  const float* p, const float* q, const float* gamma_hat, const float* omega, int N,
                  const float* h_in, float* h_out, unsigned flags, mega_stream_t stream);

/*
 * TimestepNorm forward.  x, y (B,L,D) by strides.  prev_count (B) int64, prev_mean/prev_var
 * (B,G) fp32 with G = D for num_groups <= 0 or == D, else num_groups.  gamma is the EFFECTIVE
 * scale (module weight + 1), beta the bias, both (D) fp32.  Outputs count_out (B) int64,
 * mean_out/var_out (B,G) fp32 (may alias prev_mean/prev_var; count_out must be a different array
 * than prev_count, MEGA_ERR_UNSUPPORTED otherwise: every thread block of a sequence reads the incoming
 * count).  The same holds for the fused entry points below.  Padded steps output 0 and do not
 * advance the statistics.
 * Replaces: timestep_norm_fwd / group_timestep_norm_fwd (fairseq/csrc/ops/timestep_norm.cc:23-103,
 * 218-316; CUDA fairseq/csrc/ops/timestep_norm_kernel.cu:26-185,269-484) minus the cummean/cumrstd
 * tensors saved for backward.
 */
MEGA_API int mega_timestep_norm_fwd(const void* x, void* y, int dtype, int B, int L, int D,
                           int64_t x_stride_b, int64_t x_stride_l, int64_t x_stride_d,
                           int64_t y_stride_b, int64_t y_stride_l, int64_t y_stride_d,
                           const int64_t* prev_count, const float* prev_mean, const float* prev_var,
                           const float* gamma, const float* beta, const uint8_t* pad_mask,
                           int num_groups, double eps,
                           int64_t* count_out, float* mean_out, float* var_out,
                           mega_stream_t stream);

/*
 * SequenceNorm forward: masked mean/variance over the sequence axis per (batch, channel) or per
 * (batch, group).  x, y (B,D,L) by strides (pass the strides of a (B,L,D) tensor for the
 * reference's length_last=False).  count_out (B) int64; mean_out/rstd_out (B,G) fp32.
 * Replaces: sequence_norm_fwd / group_sequence_norm_fwd (fairseq/csrc/ops/sequence_norm.cc:258-372,
 * 531-655; CUDA fairseq/csrc/ops/sequence_norm_kernel.cu:27-213,425-599).
 */
MEGA_API int mega_sequence_norm_fwd(const void* x, void* y, int dtype, int B, int D, int L,
                           int64_t x_stride_b, int64_t x_stride_d, int64_t x_stride_l,
                           int64_t y_stride_b, int64_t y_stride_d, int64_t y_stride_l,
                           const float* gamma, const float* beta, const uint8_t* pad_mask,
                           int num_groups, double eps,
                           int64_t* count_out, float* mean_out, float* rstd_out,
                           mega_stream_t stream);

/*
 * Fused per-feature TimestepNorm -> EMA (causal): y = EMA(TimestepNorm(x)) in one pass over x.
 * x (B,L,D) by strides; y by strides; xn_out NULL or a tensor (same strides as y) receiving the
 * normalised activations (the Mega block feeds them to v_proj).  TimestepNorm state as in
 * mega_timestep_norm_fwd with G = D; EMA arguments as in mega_ema_fwd (causal only; flags may
 * carry MEGA_EMA_SILU).
 * Replaces: the sequence self.norm(...) -> transpose -> self.move(...) [-> move_act] of
 * MovingAverageGatedAttention.forward (fairseq/modules/moving_average_gated_attention.py:306-316).
 */
MEGA_API int mega_tsn_ema_fwd(const void* x, void* y, void* xn_out, int dtype, int B, int L, int D,
                     int64_t x_stride_b, int64_t x_stride_l, int64_t x_stride_d,
                     int64_t y_stride_b, int64_t y_stride_l, int64_t y_stride_d,
                     const int64_t* prev_count, const float* prev_mean, const float* prev_var,
                     const float* gamma, const float* beta, double eps,
                     int64_t* count_out, float* mean_out, float* var_out,
                     const float* p, const float* q, const float* gamma_hat, const float* omega, int N,
                     const uint8_t* pad_mask, const float* h_in, float* h_out,
                     unsigned flags, mega_stream_t stream);

/*
 * mega_tsn_ema_fwd in its segmented form, on request: the sequence is cut into `runs` (2, 4 or 8) runs,
 * one thread block per run and tile of 64 channels x 8 sequences; a run starts from the running sums
 * and pole states that the run before left in device memory.  Same arguments, meaning and results
 * (bit for bit) as mega_tsn_ema_fwd without xn_out and pad_mask; bf16, channel strides 1, L a
 * multiple of 32 x runs, B >= 4, N <= 16.
 * No counterpart in the reference (a scheduling variant of this library's own kernel).
 * Allocates nothing: its scratch (hand-off of the states, work counter and flags) are fixed arrays
 * in device memory owned by the library: 16 MiB of pole states (B x D x N <= 4 Mi values, unused
 * when h_out is given), 2 MiB of running sums (B x D <= 256 Ki) and 16384 work items; a call
 * beyond these, or outside the envelope above, returns MEGA_ERR_UNSUPPORTED and launches nothing.
 * The arrays are shared by every call on the device (mega_tsn_ema_fwd may use them too for large
 * problems): calls that use them must not overlap in time, whatever their streams; this entry
 * point does not order them.  The counter and flags are cleared on the stream before each launch.
 */
MEGA_API int mega_tsn_ema_fwd_runs(const void* x, void* y, int dtype, int B, int L, int D,
                     int64_t x_stride_b, int64_t x_stride_l, int64_t x_stride_d,
                     int64_t y_stride_b, int64_t y_stride_l, int64_t y_stride_d,
                     const int64_t* prev_count, const float* prev_mean, const float* prev_var,
                     const float* gamma, const float* beta, double eps,
                     int64_t* count_out, float* mean_out, float* var_out,
                     const float* p, const float* q, const float* gamma_hat, const float* omega, int N,
                     const float* h_in, float* h_out, unsigned flags, int runs, mega_stream_t stream);

/*
 * Fused per-channel SequenceNorm -> EMA (causal or bidirectional) on length-contiguous rows:
 * x, y (B,D,L) with stride_l == 1.  norm_gamma is the EFFECTIVE scale (module weight + 1).
 * count_out (B), mean_out / rstd_out (B,D) may be NULL.  flags as in mega_ema_fwd.  Returns
 * MEGA_ERR_UNSUPPORTED when the row does not fit the shared-memory resident kernel (L < 512, L
 * beyond ~27k positions bidirectional / ~54k causal, ndim > 16, stride_l != 1): callers then run
 * mega_sequence_norm_fwd followed by mega_ema_fwd.
 * Replaces: x = self.norm(x, padding_mask); mx = self.move(x, padding_mask) of the bidirectional
 * branch of MovingAverageGatedAttention.forward (moving_average_gated_attention.py:298-303,313).
 */
MEGA_API int mega_sqn_ema_fwd(const void* x, void* y, int dtype, int B, int D, int L,
                              int64_t x_stride_b, int64_t x_stride_d, int64_t x_stride_l,
                              int64_t y_stride_b, int64_t y_stride_d, int64_t y_stride_l,
                              const float* norm_gamma, const float* norm_beta, double eps,
                              int64_t* count_out, float* mean_out, float* rstd_out,
                              const float* p, const float* q, const float* gamma_hat, const float* omega, int N,
                              const uint8_t* pad_mask, unsigned flags, mega_stream_t stream);

/*
 * Single-token decode step of the fused pair, all running state updated IN PLACE:
 * count (B) int64, mean/var (B,D) fp32 (pass count = NULL to skip the TimestepNorm),
 * h (B,D,N) fp32 pole states (16-byte aligned when N is a multiple of 4).  x, y, xn_out (B,D)
 * contiguous activations; xn_out may be NULL.  count_next: NULL or == count: the counts are
 * bumped in place, by a second launch after the element kernel (every CTA reads them); a
 * DISTINCT array (B): it receives count + 1 from the element kernel itself and count is left as it
 * was - one launch per step; the caller alternates two arrays.
 * Replaces: the L == 1 case of TimestepNorm.forward + BaseMovingLayer.forward with an
 * incremental state (norm_layer/timestep_norm.py:100-139, base_moving_average.py:144-160).
 */
MEGA_API int mega_tsn_ema_step(const void* x, void* y, void* xn_out, int dtype, int B, int D,
                               int64_t* count, int64_t* count_next, float* mean, float* var,
                               const float* gamma, const float* beta, double eps,
                               const float* p, const float* q, const float* gamma_hat, const float* omega, int N,
                               float* h, unsigned flags, mega_stream_t stream);

/*
 * Mega gate elementwise ops on (rows, D) contiguous activations.
 *   mega_gate_silu:    y = silu(a [+ b])            (b may be NULL)
 *   mega_gate_mul_silu y = a * silu(r)              (attn * silu(r) with r pre-activation)
 *   mega_gate_output:  out = residual + sigmoid(u) * (silu(hx + h_lin) - residual)
 *   mega_gate_qk:      zn = z / max(||z||_2, eps) per row; q = zn * (gamma[0] + 1) + beta[0],
 *                      k = zn * (gamma[1] + 1) + beta[1]; gamma, beta are (2, cols) fp32
 * u, hx, z may be column slices of a wider matrix: `ld_*` are their row pitches in elements.
 * Replaces: moving_average_gated_attention.py:308,316,322,324-328,330,407-412
 * (sigmoid / silu / addcmul chain; F.normalize + the (2, S) affine that makes query and key).
 */
MEGA_API int mega_gate_silu(const void* a, int64_t ld_a, const void* b, int64_t ld_b, void* y, int64_t ld_y,
                   int dtype, int64_t rows, int cols, mega_stream_t stream);
MEGA_API int mega_gate_mul_silu(const void* a, int64_t ld_a, const void* r, int64_t ld_r, void* y, int64_t ld_y,
                       int dtype, int64_t rows, int cols, mega_stream_t stream);
MEGA_API int mega_gate_output(const void* residual, int64_t ld_res, const void* u, int64_t ld_u,
                     const void* hx, int64_t ld_hx, const void* h_lin, int64_t ld_h,
                     void* out, int64_t ld_out, int dtype, int64_t rows, int cols,
                     mega_stream_t stream);
MEGA_API int mega_gate_qk(const void* z, int64_t ld_z, const float* gamma, const float* beta, void* q,
                 int64_t ld_q, void* k, int64_t ld_k, int dtype, int64_t rows, int cols, double eps,
                 mega_stream_t stream);
/*
 * mega_gate_qk followed by the block's rotary position embedding on both results
 * (fairseq/modules/relative_positional_bias.py:47-97 as MovingAverageGatedAttention applies it,
 * moving_average_gated_attention.py:217-221): the pair of features (2j, 2j + 1) of row r is rotated by
 * the angle of position (r % period) [+ q_offset for the query] and frequency j.  rot: fp32
 * (positions, cols / 2, 2) = (cos, sin) of those angles, 8-byte aligned; period + q_offset <= positions;
 * cols even.  The rotation runs in fp32 on the unrounded affine results; q, k come back in `dtype`.
 */
MEGA_API int mega_gate_qk_rotary(const void* z, int64_t ld_z, const float* gamma, const float* beta,
                        const float* rot, int positions, int period, int q_offset,
                        void* q, int64_t ld_q, void* k, int64_t ld_k,
                        int dtype, int64_t rows, int cols, double eps, mega_stream_t stream);

/*
 * ---- Training: forward with saved statistics, and backward ---------------------------------
 *
 * mega_timestep_norm_fwd_train: mega_timestep_norm_fwd that also writes the per-step statistics
 * the backward needs: cummean, cumrstd (B, L, G) fp32 contiguous, and group_mean (B, L, G) for
 * the grouped form (NULL otherwise); G = D for the per-feature form.  At a padded step cummean
 * holds the unchanged running mean.
 * Replaces: timestep_norm_fwd / group_timestep_norm_fwd as called by TimestepNormFunc.forward
 * (norm_layer/timestep_norm.py:29-41), which return (Y, count, mean, var, [group_mean,] cummean,
 * cumrstd).
 */
MEGA_API int mega_timestep_norm_fwd_train(const void* x, void* y, int dtype, int B, int L, int D, int64_t xsb,
                                 int64_t xsl, int64_t xsd, int64_t ysb, int64_t ysl, int64_t ysd,
                                 const int64_t* prev_count, const float* prev_mean, const float* prev_var,
                                 const float* gamma, const float* beta, const uint8_t* pad_mask,
                                 int num_groups, double eps, int64_t* count_out, float* mean_out,
                                 float* var_out, float* cummean, float* cumrstd, float* group_mean,
                                 mega_stream_t stream);

/*
 * mega_timestep_norm_bwd: gradients of TimestepNorm.  dy, x, dx are (B, L, D) with strides in
 * elements; dmean, dvar (B, G) are the gradients flowing into the returned statistics (NULL = 0);
 * count is the FINAL count returned by the forward; cummean / cumrstd / group_mean are the
 * forward's saves.  Outputs: dx, dprev_mean, dprev_var (B, G), dgamma, dbeta (D); the last two
 * are zeroed on the stream and accumulated with atomic adds over the batch.
 * Grouped form: at most 256 features per group (MEGA_ERR_UNSUPPORTED beyond).
 * Replaces: timestep_norm_bwd / group_timestep_norm_bwd (fairseq/csrc/ops/timestep_norm.cc:105-216,
 * 318-446).
 */
MEGA_API int mega_timestep_norm_bwd(const void* dy, const void* x, void* dx, int dtype, int B, int L, int D,
                           int64_t gsb, int64_t gsl, int64_t gsd, int64_t xsb, int64_t xsl, int64_t xsd,
                           int64_t dsb, int64_t dsl, int64_t dsd, const float* dmean, const float* dvar,
                           const float* prev_mean, const int64_t* count, const float* cummean,
                           const float* cumrstd, const float* group_mean, const float* gamma,
                           const uint8_t* pad_mask, int num_groups, float* dprev_mean, float* dprev_var,
                           float* dgamma, float* dbeta, mega_stream_t stream);

/*
 * mega_sequence_norm_bwd: gradients of SequenceNorm (per-channel and grouped forms; mean, rstd are (B, G)).  dy, x, dx are (B, D, L)
 * with strides in elements (the length-major order of a (B, L, D) tensor is a stride pattern);
 * count (B), mean, rstd (B, D) are the forward's outputs.  dgamma, dbeta (D) are zeroed on the
 * stream and accumulated over the batch.
 * Replaces: sequence_norm_bwd, group_sequence_norm_bwd (fairseq/csrc/ops/sequence_norm.cc:374-529, 657-860).
 */
MEGA_API int mega_sequence_norm_bwd(const void* dy, const void* x, void* dx, int dtype, int B, int D, int L,
                           int64_t gsb, int64_t gsd, int64_t gsl, int64_t xsb, int64_t xsd, int64_t xsl,
                           int64_t dsb, int64_t dsd, int64_t dsl, const int64_t* count, const float* mean,
                           const float* rstd, const float* gamma, const uint8_t* pad_mask, int num_groups,
                           float* dgamma, float* dbeta, mega_stream_t stream);

/*
 * mega_ema_bwd: gradients of mega_ema_fwd (without the SiLU flag; truncation as in the forward:
 * bidirectional form only).
 * dy, x, dx are (B, D, L) with strides in elements; p, q, gamma_hat are (K, N) with K = D or 2D
 * (bidirectional).  h_in (B, D, N) is the state the forward started from, dh_out the gradient
 * flowing into the state it returned (either may be NULL; causal form only).  Outputs: dx;
 * dp, dq, dgamma_hat (K, N) and domega (D), zeroed on the stream and accumulated over the batch
 * with atomic adds; dh_in (B, D, N) or NULL.
 * Replaces: the backward chain FFTConvFunc.backward -> ema_parameters_bwd -> ema_hidden_bwd
 * (fused_ops/fftconv.py:29-38,65-82; fairseq/csrc/ops/ema_parameters.cc, ema_hidden.cc) and the
 * autograd of the mask / omega elementwise ops in base_moving_average.py:137-172.
 */
MEGA_API int mega_ema_bwd(const void* dy, const void* x, void* dx, int dtype, int B, int D, int L, int64_t gsb,
                 int64_t gsd, int64_t gsl, int64_t xsb, int64_t xsd, int64_t xsl, int64_t dsb, int64_t dsd,
                 int64_t dsl, const float* p, const float* q, const float* gamma_hat, const float* omega,
                 int N, const uint8_t* pad_mask, const float* h_in, const float* dh_out, unsigned flags,
                 int truncation, float* dp, float* dq, float* dgamma_hat, float* domega, float* dh_in,
                 mega_stream_t stream);

/*
 * mega_ema_coeffs_bwd: chain rule from (dp, dq, dgamma_hat), each (K, N), to the raw parameters
 * alpha, delta, beta (K, N[, 1]) and gamma (K, N).
 * Replaces: autograd through _calc_coeffs (exponential_moving_average.py:71-80).
 */
MEGA_API int mega_ema_coeffs_bwd(const float* alpha, const float* delta, const float* beta, const float* dp,
                        const float* dq, const float* dgamma_hat, int K, int N, float* dalpha, float* ddelta,
                        float* dbeta, float* dgamma, mega_stream_t stream);

/*
 * ---- Complex EMA (MultiHeadComplexEMA) ----------------------------------------------------
 * Poles q_n = (1 - sigmoid(alpha) sigmoid(delta)) e^{i theta_n}, theta_n = (n + 1) sigmoid(theta)
 * 2 pi / N; input gain p = sigmoid(alpha); gamma_hat = (gamma_re + i gamma_im) / sqrt(N).
 * Complex arrays are interleaved (re, im) fp32: q, gamma_hat are (K, N, 2); states are (B, D, N, 2)
 * — the memory of a complex64 tensor.
 *
 * mega_cema_coeffs: alpha, delta (K, N[, 1]), theta (K[, 1, 1]), gamma (K, N, 2) in param_dtype
 *   -> p (K, N), q (K, N, 2), gamma_hat (K, N, 2).
 *   Replaces: MultiHeadComplexEMA._calc_coeffs (complex_exponential_moving_average.py:79-96).
 * mega_cema_kernel: k[row, l] = Re(sum_n p gamma_hat q^l), (K, L) fp32.
 *   Replaces: _compute_kernel (:98-109) / the weight half of ema_parameters_fwd.
 * mega_cema_fwd: same contract as mega_ema_fwd (strides, mask, flags, truncation for the
 *   bidirectional form, carried state in / out for the causal form) with complex poles.
 *   Replaces: BaseMovingLayer.forward (base_moving_average.py:120-172) for the complex layer:
 *   ema_parameters_fwd + fftconv / bidirectional_fftconv + bias + ema_hidden_fwd + residual.
 * mega_cema_step: single-token update, x, y (B, D) contiguous; h_in may be NULL or equal h_out.
 *   Replaces: BaseMovingLayer.one_step (:105-118) + the omega residual.
 */
MEGA_API int mega_cema_coeffs(const void* alpha, const void* delta, const void* theta, const void* gamma,
                     int param_dtype, int K, int N, float* p, float* q, float* gamma_hat,
                     mega_stream_t stream);
MEGA_API int mega_cema_kernel(const float* p, const float* q, const float* gamma_hat, int K, int N, int L,
                     float* kernel_out, mega_stream_t stream);
MEGA_API int mega_cema_fwd(const void* x, void* y, int dtype, int B, int D, int L, int64_t xsb, int64_t xsd,
                  int64_t xsl, int64_t ysb, int64_t ysd, int64_t ysl, const float* p, const float* q,
                  const float* gamma_hat, const float* omega, int N, const uint8_t* pad_mask,
                  const float* h_in, float* h_out, unsigned flags, int truncation, mega_stream_t stream);
MEGA_API int mega_cema_step(const void* x, void* y, int dtype, int B, int D, const float* p, const float* q,
                   const float* gamma_hat, const float* omega, int N, const float* h_in, float* h_out,
                   unsigned flags, mega_stream_t stream);

/*
 * mega_tsn_cema_fwd: mega_tsn_ema_fwd with the complex layer's coefficients (q, gamma_hat
 * interleaved (K, N, 2); h_in / h_out (B, D, N, 2)): per-feature TimestepNorm fused with the causal
 * complex EMA on x (B, L, D), one pass over x when the channels are contiguous.  x and y must not
 * alias.
 * Replaces: self.norm -> transpose -> self.move [-> move_act] of MovingAverageGatedAttention.forward
 * (moving_average_gated_attention.py:306-316) with moving_layer='cema'.
 */
MEGA_API int mega_tsn_cema_fwd(const void* x, void* y, void* xn_out, int dtype, int B, int L, int D, int64_t xsb,
                      int64_t xsl, int64_t xsd, int64_t ysb, int64_t ysl, int64_t ysd,
                      const int64_t* prev_count, const float* prev_mean, const float* prev_var,
                      const float* gamma, const float* beta, double eps, int64_t* count_out, float* mean_out,
                      float* var_out, const float* p, const float* q, const float* gamma_hat,
                      const float* omega, int N, const uint8_t* pad_mask, const float* h_in, float* h_out,
                      unsigned flags, mega_stream_t stream);

/*
 * mega_tsn_cema_step: single-token decode step of TimestepNorm -> MultiHeadComplexEMA, all running
 * state updated IN PLACE like mega_tsn_ema_step: count (B) int64, mean/var (B,D) fp32, h (B,D,N,2)
 * fp32 complex pole states (16-byte aligned).  N must be 2, 4, 8, 16 or 32 (MEGA_ERR_UNSUPPORTED
 * otherwise: run the two operators in turn).  count_next as in mega_tsn_ema_step (a distinct array:
 * one launch; NULL or == count: two launches).
 * Replaces: the L == 1 case of TimestepNorm.forward + BaseMovingLayer.forward with an incremental
 * state and the complex layer (norm_layer/timestep_norm.py:100-139, base_moving_average.py:144-160,
 * complex_exponential_moving_average.py:79-109).
 */
MEGA_API int mega_tsn_cema_step(const void* x, void* y, void* xn_out, int dtype, int B, int D, int64_t* count,
                       int64_t* count_next, float* mean, float* var, const float* gamma, const float* beta, double eps,
                       const float* p, const float* q, const float* gamma_hat, const float* omega, int N,
                       float* h, unsigned flags, mega_stream_t stream);

/*
 * mega_cema_bwd / mega_cema_coeffs_bwd: gradients of mega_cema_fwd (no SiLU flag, no carried state;
 * truncation as in the forward), same argument conventions as mega_ema_bwd; dq and dgamma_hat are (K, N, 2) with
 * the gradients of the real and imaginary parts, dtheta is (K).
 * Replaces: autograd through MultiHeadComplexEMA (ema_parameters_bwd + the FFT convolution backward +
 * _calc_coeffs, complex_exponential_moving_average.py:79-109).
 */
MEGA_API int mega_cema_bwd(const void* dy, const void* x, void* dx, int dtype, int B, int D, int L, int64_t gsb,
                  int64_t gsd, int64_t gsl, int64_t xsb, int64_t xsd, int64_t xsl, int64_t dsb, int64_t dsd,
                  int64_t dsl, const float* p, const float* q, const float* gamma_hat, const float* omega,
                  int N, const uint8_t* pad_mask, unsigned flags, int truncation, float* dp, float* dq,
                  float* dgamma_hat, float* domega, mega_stream_t stream);
MEGA_API int mega_cema_coeffs_bwd(const float* alpha, const float* delta, const float* theta, const float* q,
                         const float* dp, const float* dq, const float* dgamma_hat, int K, int N,
                         float* dalpha, float* ddelta, float* dtheta, float* dgamma, mega_stream_t stream);

/*
 * Attention-weight softmax of the Mega block.  x, y (and dy, dx) are contiguous (batch, outer, inner)
 * score tensors; softmax over `inner`; with `causal` row r keeps its first inner - outer + r + 1
 * columns and the rest of the row is 0; a row whose kept scores are all -inf is all zeros.
 * inner <= 8192.
 * Replaces: attention_softmax_fwd / attention_softmax_bwd with dropout = 0
 * (fairseq/csrc/ops/attention_softmax.cc:6-18, fairseq/csrc/softmax.cuh:90-153; called from
 * fairseq/modules/attention_softmax.py:11-40).
 *
 * mega_attention_dropkey_softmax_fwd: the same with DropKey, the reference's training option
 * (fairseq/csrc/softmax.cuh:155-232): each kept score is set to -inf with probability `dropout`
 * (0 <= dropout < 1) before the softmax, without rescaling; a row that loses every score is all
 * zeros.  The backward is mega_attention_softmax_bwd (dropped columns have y = 0).  Column c of
 * row i (i over batch x outer) is dropped when word c % 4 of Philox4x32-10 with counter
 * (c / 4, i, offset low, offset high) and key (seed low, seed high) is below dropout * 2^32: the mask
 * is a function of (seed, offset, i, c) only.  The reference draws from curand's Philox stream
 * indexed by its own thread layout, so the masks are equal in distribution, not bit for bit.
 */
MEGA_API int mega_attention_softmax_fwd(const void* x, void* y, int dtype, int64_t batch, int64_t outer, int inner,
                               int causal, mega_stream_t stream);
MEGA_API int mega_attention_softmax_bwd(const void* dy, const void* y, void* dx, int dtype, int64_t batch,
                               int64_t outer, int inner, int causal, mega_stream_t stream);
MEGA_API int mega_attention_dropkey_softmax_fwd(const void* x, void* y, int dtype, int64_t batch, int64_t outer,
                                       int inner, int causal, double dropout, uint64_t seed, uint64_t offset,
                                       mega_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MEGA_B200_H_ */
