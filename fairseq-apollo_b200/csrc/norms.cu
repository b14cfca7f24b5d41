// TimestepNorm (plain + grouped) and SequenceNorm (plain + grouped, any memory order).
//
// TimestepNorm is a causal cumulative normalisation: the statistics at step t are the Welford
// moments of the unmasked prefix (plus a prior that acts as prev_count pseudo-samples).
// SequenceNorm normalises with the masked moments of the whole sequence.
#include <mutex>

#include "common.cuh"
#include "stream_bwd.cuh"
#include "stream_cl.cuh"

namespace mega {

struct TsnArgs {
  const void* x;
  void* y;
  int B, L, D, G;
  long long xsb, xsl, xsd, ysb, ysl, ysd;
  const long long* prev_count;
  const float *prev_mean, *prev_var, *gamma, *beta;
  const unsigned char* mask;
  float eps;
  long long* count_out;
  float *mean_out, *var_out;
  // training-mode saves (all NULL in inference): per-step statistics, fp32, contiguous (B, L, G);
  // group_mean only for the grouped form
  float *cummean, *cumrstd, *group_mean;
};

// Welford step with the update rule of the reference (fairseq/csrc/utils.h:56-65).
__device__ __forceinline__ void welford_step(float coef, float x, float mean, float var, float& m1,
                                             float& m2) {
  const float d1 = x - mean;
  m1 = fmaf(coef, d1, mean);
  const float d2 = fmaf(d1, x - m1, -var);
  m2 = fmaf(coef, d2, var);
}

// One thread per (batch, feature), feature fastest; sequential over time.  The presence of a
// mask and of the training saves are template parameters: a run-time test of those pointers
// inside the unrolled load batch turns it into branchy code whose loads no longer overlap
// (measured: 4x slower with the mask test, 2x with the save test, even when both are null).
template <typename T, bool kMask, bool kSave>
__global__ void __launch_bounds__(128) tsn_plain_kernel(TsnArgs a) {
  long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)a.B * a.D) return;
  const int d = (int)(gid % a.D);
  const int b = (int)(gid / a.D);
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ysb + d * a.ysd;
  const unsigned char* mp = kMask ? a.mask + (size_t)b * a.L : nullptr;
  float* cmp = kSave ? a.cummean + (size_t)b * a.L * a.D + d : nullptr;
  float* crp = kSave ? a.cumrstd + (size_t)b * a.L * a.D + d : nullptr;
  // the count as a 32-bit step counter on top of the incoming count (64-bit integer to float
  // conversions inside the serial loop are slow)
  const long long cnt0 = a.prev_count[b];
  const float cnt0f = (float)cnt0;
  int seen = 0;
  float mean = a.prev_mean[gid], var = a.prev_var[gid];
  const float w = __ldg(a.gamma + d), bb = __ldg(a.beta + d);
  constexpr int U = 32;  // loads in flight per thread: B x D threads are few, latency is hidden per thread
  for (int t0 = 0; t0 < a.L; t0 += U) {
    float xv[U];
    bool mk[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u;
      xv[u] = 0.f; mk[u] = true;
      if (t < a.L) {
        xv[u] = Elem<T>::ld(xp + t * a.xsl);
        mk[u] = kMask ? __ldg(mp + t) != 0 : false;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u;
      if (t < a.L) {
        float m1, m2;
        const float coef = rcp_approx(cnt0f + (float)(seen + 1));
        welford_step(coef, xv[u], mean, var, m1, m2);
        const float rstd = rsqrt_approx(m2 + a.eps);
        const float out = mk[u] ? 0.f : fmaf((xv[u] - m1) * rstd, w, bb);
        Elem<T>::st(yp + t * a.ysl, out);
        if (!mk[u]) { mean = m1; var = m2; ++seen; }
        if (kSave) {  // the running mean AFTER step t (unchanged by a padded step)
          cmp[(size_t)t * a.D] = mean;
          crp[(size_t)t * a.D] = rstd;
        }
      }
    }
  }
  a.mean_out[gid] = mean;
  a.var_out[gid] = var;
  if (d == 0) a.count_out[b] = cnt0 + seen;
}

// Grouped: one warp per (batch, group); per step the group's D/G features are reduced to
// (mean, var), combined into the running state with weight 1, then normalised.
template <typename T>
__global__ void __launch_bounds__(128) tsn_group_kernel(TsnArgs a) {
  const int lane = threadIdx.x & 31;
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (wid >= (long long)a.B * a.G) return;
  const int g = (int)(wid % a.G);
  const int b = (int)(wid / a.G);
  const int gs = a.D / a.G;
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + (long long)g * gs * a.xsd;
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ysb + (long long)g * gs * a.ysd;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  long long cnt = a.prev_count[b];
  float mean = a.prev_mean[wid], var = a.prev_var[wid];
  const float inv_gs = 1.0f / (float)gs;
  for (int t = 0; t < a.L; ++t) {
    const T* xr = xp + t * a.xsl;
    float s = 0.f;
    for (int k = lane; k < gs; k += 32) s += Elem<T>::ld(xr + k * a.xsd);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float gm = s * inv_gs;
    float v = 0.f;
    for (int k = lane; k < gs; k += 32) {
      const float dlt = Elem<T>::ld(xr + k * a.xsd) - gm;
      v = fmaf(dlt, dlt, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const float gv = v * inv_gs;
    // WelfordCombine(cnt, mean, var, 1, gm, gv)  (fairseq/csrc/utils.h:67-76)
    const float m0 = (float)(cnt + 1);
    const float c1 = (float)cnt / m0, c2 = 1.0f / m0;
    const float dl = gm - mean;
    const float m1 = c1 * mean + c2 * gm;
    const float m2 = c1 * var + c2 * gv + (c1 * dl) * (c2 * dl);
    const float rstd = rsqrtf(m2 + a.eps);
    const bool mk = mp != nullptr && mp[t] != 0;
    T* yr = yp + t * a.ysl;
    for (int k = lane; k < gs; k += 32) {
      const int f = g * gs + k;
      const float xv = Elem<T>::ld(xr + k * a.xsd);
      const float out = mk ? 0.f : fmaf((xv - m1) * rstd, __ldg(a.gamma + f), __ldg(a.beta + f));
      Elem<T>::st(yr + k * a.ysd, out);
    }
    if (!mk) { mean = m1; var = m2; ++cnt; }
    if (a.cummean && lane == 0) {
      const size_t o = ((size_t)b * a.L + t) * a.G + g;
      a.cummean[o] = mean;
      a.cumrstd[o] = rstd;
      a.group_mean[o] = gm;
    }
  }
  if (lane == 0) {
    a.mean_out[wid] = mean;
    a.var_out[wid] = var;
    if (g == 0) a.count_out[b] = cnt;
  }
}

// ---------------------------------------------------------------------------
// SequenceNorm
// ---------------------------------------------------------------------------
struct SqnArgs {
  const void* x;
  void* y;
  int B, D, L, G;
  long long xsb, xsd, xsl, ysb, ysd, ysl;
  const float *gamma, *beta;
  const unsigned char* mask;
  float eps;
  long long* count_out;
  float *mean_out, *rstd_out;
};

__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = 0.f;
  const int nw = (blockDim.x + 31) >> 5;
  for (int i = 0; i < nw; ++i) r += red[i];
  return r;
}

// One CTA per (batch, group): the group's gs channels x L positions.  Two reduction passes
// (mean, then centred second moment) and a normalisation pass; when the segment fits the
// dynamic shared memory it is cached there after the first read.
template <typename T>
__global__ void __launch_bounds__(256) sqn_segment_kernel(SqnArgs a, int cache_elems) {
  extern __shared__ float cache[];
  __shared__ float red[8];
  const int g = blockIdx.x % a.G;
  const int b = blockIdx.x / a.G;
  const int gs = a.D / a.G;
  const long long n = (long long)gs * a.L;
  const bool len_fast = a.xsl <= a.xsd;  // iterate the contiguous axis fastest
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + (long long)g * gs * a.xsd;
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ysb + (long long)g * gs * a.ysd;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  const bool cached = n <= cache_elems;

  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const int j = len_fast ? (int)(i / a.L) : (int)(i % gs);
    const int t = len_fast ? (int)(i % a.L) : (int)(i / gs);
    const float xv = Elem<T>::ld(xp + j * a.xsd + t * a.xsl);
    if (cached) cache[i] = xv;
    const bool mk = mp != nullptr && mp[t] != 0;
    if (!mk) s += xv;
  }
  __shared__ int valid_steps;
  if (threadIdx.x == 0) valid_steps = 0;
  __syncthreads();
  int c = 0;
  for (int t = threadIdx.x; t < a.L; t += blockDim.x) c += (mp == nullptr || mp[t] == 0) ? 1 : 0;
  if (c) atomicAdd(&valid_steps, c);
  __syncthreads();
  const float tot = (float)valid_steps * (float)gs;
  const float sum = block_sum(s, red);
  const float mean = tot > 0.f ? sum / tot : 0.f;
  float v = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const int j = len_fast ? (int)(i / a.L) : (int)(i % gs);
    const int t = len_fast ? (int)(i % a.L) : (int)(i / gs);
    const float xv = cached ? cache[i] : Elem<T>::ld(xp + j * a.xsd + t * a.xsl);
    const bool mk = mp != nullptr && mp[t] != 0;
    if (!mk) { const float dl = xv - mean; v = fmaf(dl, dl, v); }
  }
  const float var = tot > 0.f ? block_sum(v, red) / tot : 0.f;
  const float rstd = rsqrtf(var + a.eps);
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const int j = len_fast ? (int)(i / a.L) : (int)(i % gs);
    const int t = len_fast ? (int)(i % a.L) : (int)(i / gs);
    const float xv = cached ? cache[i] : Elem<T>::ld(xp + j * a.xsd + t * a.xsl);
    const bool mk = mp != nullptr && mp[t] != 0;
    const int f = g * gs + j;
    const float out = mk ? 0.f : fmaf((xv - mean) * rstd, __ldg(a.gamma + f), __ldg(a.beta + f));
    Elem<T>::st(yp + j * a.ysd + t * a.ysl, out);
  }
  if (threadIdx.x == 0) {
    a.mean_out[blockIdx.x] = mean;
    a.rstd_out[blockIdx.x] = rstd;
    if (g == 0) a.count_out[b] = (long long)valid_steps;
  }
}

// Plain SequenceNorm on channel-contiguous memory: one thread per (batch, channel) column,
// masked Welford over time, then a second sweep that normalises.
template <typename T>
__global__ void __launch_bounds__(128) sqn_column_kernel(SqnArgs a) {
  long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)a.B * a.D) return;
  const int d = (int)(gid % a.D);
  const int b = (int)(gid / a.D);
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ysb + d * a.ysd;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  long long cnt = 0;
  float mean = 0.f, var = 0.f;
  for (int t = 0; t < a.L; ++t) {
    const bool mk = mp != nullptr && mp[t] != 0;
    if (!mk) {
      const float xv = Elem<T>::ld(xp + t * a.xsl);
      float m1, m2;
      welford_step(__frcp_rn((float)(cnt + 1)), xv, mean, var, m1, m2);
      mean = m1; var = m2; ++cnt;
    }
  }
  const float rstd = rsqrtf(var + a.eps);
  const float w = __ldg(a.gamma + d), bb = __ldg(a.beta + d);
  for (int t = 0; t < a.L; ++t) {
    const bool mk = mp != nullptr && mp[t] != 0;
    const float xv = Elem<T>::ld(xp + t * a.xsl);
    Elem<T>::st(yp + t * a.ysl, mk ? 0.f : fmaf((xv - mean) * rstd, w, bb));
  }
  a.mean_out[gid] = mean;
  a.rstd_out[gid] = rstd;
  if (d == 0) a.count_out[b] = cnt;
}

// ---------------------------------------------------------------------------
// gates
// ---------------------------------------------------------------------------
template <typename T, int OP>
__global__ void gate_kernel(const T* a, long long lda, const T* b, long long ldb, const T* c, long long ldc,
                            const T* d, long long ldd, T* y, long long ldy, long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int col = (int)(i % cols);
    float out;
    if (OP == 0) {  // silu(a [+ b])
      float v = Elem<T>::ld(a + r * lda + col);
      if (b) v += Elem<T>::ld(b + r * ldb + col);
      out = siluf_(v);
    } else if (OP == 1) {  // a * silu(b)
      out = Elem<T>::ld(a + r * lda + col) * siluf_(Elem<T>::ld(b + r * ldb + col));
    } else {  // a = residual, b = u, c = hx, d = h_lin
      const float res = Elem<T>::ld(a + r * lda + col);
      const float u = sigmoidf_(Elem<T>::ld(b + r * ldb + col));
      const float h = siluf_(Elem<T>::ld(c + r * ldc + col) + Elem<T>::ld(d + r * ldd + col));
      out = fmaf(u, h - res, res);
    }
    Elem<T>::st(y + r * ldy + col, out);
  }
}

// The same gates, 16 bytes per access (8 bf16 / fp16 or 4 fp32 values), for column counts, row
// pitches and base addresses that are multiples of 16 bytes; a thread takes kU vectors a grid
// stride apart, all loads first.  vpr = vectors per row.
template <typename T>
struct GateVec {
  static constexpr int kN = 16 / (int)sizeof(T);
  static __device__ __forceinline__ void load(const T* p, float (&f)[kN]) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));   // read once: streaming
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int k = 0; k < kN; ++k) f[k] = Elem<T>::ld_shared(e + k);
  }
  static __device__ __forceinline__ void store(T* p, const float (&f)[kN]) {
    uint4 v;
    T* e = reinterpret_cast<T*>(&v);
#pragma unroll
    for (int k = 0; k < kN; ++k) Elem<T>::st(e + k, f[k]);
    __stcs(reinterpret_cast<uint4*>(p), v);
  }
};

template <typename T, int OP, int kU>
__global__ void __launch_bounds__(256) gate_vec_kernel(const T* a, long long lda, const T* b, long long ldb, const T* c,
                                                       long long ldc, const T* d, long long ldd, T* y, long long ldy,
                                                       unsigned nvec, unsigned vpr) {
  constexpr int kN = GateVec<T>::kN;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned v0 = blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += kU * stride) {
    float fa[kU][kN], fb[kU][kN], fc[kU][kN], fd[kU][kN];
    long long off[kU][5];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const unsigned v = v0 + u * stride;
      if (v < nvec) {
        const unsigned r = v / vpr;
        const long long col = (long long)(v - r * vpr) * kN;
        off[u][0] = r * lda + col; off[u][1] = r * ldb + col; off[u][2] = r * ldc + col; off[u][3] = r * ldd + col;
        off[u][4] = r * ldy + col;
        GateVec<T>::load(a + off[u][0], fa[u]);
        if (OP != 0 || b != nullptr) GateVec<T>::load(b + off[u][1], fb[u]);
        if (OP == 2) {
          GateVec<T>::load(c + off[u][2], fc[u]);
          GateVec<T>::load(d + off[u][3], fd[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const unsigned v = v0 + u * stride;
      if (v < nvec) {
        float out[kN];
        // 16-bit outputs: SiLU and the sigmoid from one tanh.approx each (relative error ~2^-11, below
        // the rounding of the output); fp32 keeps the exponential forms
        constexpr bool kFast = sizeof(T) == 2;
#pragma unroll
        for (int k = 0; k < kN; ++k) {
          if (OP == 0) {  // silu(a [+ b])
            const float v = b != nullptr ? fa[u][k] + fb[u][k] : fa[u][k];
            out[k] = kFast ? silu_tanh(v) : siluf_(v);
          } else if (OP == 1) {  // a * silu(b)
            out[k] = fa[u][k] * (kFast ? silu_tanh(fb[u][k]) : siluf_(fb[u][k]));
          } else {  // a = residual, b = u, c = hx, d = h_lin
            float g;
            if (kFast) {
              float t;
              asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * fb[u][k]));
              g = fmaf(0.5f, t, 0.5f);
            } else {
              g = sigmoidf_(fb[u][k]);
            }
            const float hs = fc[u][k] + fd[u][k];
            const float h = kFast ? silu_tanh(hs) : siluf_(hs);
            out[k] = fmaf(g, h - fa[u][k], fa[u][k]);
          }
        }
        GateVec<T>::store(y + off[u][4], out);
      }
    }
  }
}

// One warp per row: z / max(||z||_2, eps), then the two affine rows (query, key).
template <typename T>
__global__ void gate_qk_kernel(const T* z, long long ldz, const float* gamma, const float* beta, T* qo,
                               long long ldq, T* ko, long long ldk, long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += warps) {
    const T* zr = z + r * ldz;
    float ss = 0.f;
    for (int c = lane; c < cols; c += 32) {
      const float v = Elem<T>::ld(zr + c);
      ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.f / fmaxf(sqrtf(ss), eps);
    for (int c = lane; c < cols; c += 32) {
      const float v = Elem<T>::ld(zr + c) * inv;
      Elem<T>::st(qo + r * ldq + c, fmaf(v, gamma[c] + 1.f, beta[c]));
      Elem<T>::st(ko + r * ldk + c, fmaf(v, gamma[cols + c] + 1.f, beta[cols + c]));
    }
  }
}

// The same with the rotary position embedding of the block applied to both results (pairs of
// features (2j, 2j + 1) of row r rotated by the angle of position r % period and frequency j;
// rot (positions, cols / 2, 2) holds (cos, sin)): a lane owns whole pairs, the rotation runs in fp32
// on the unrounded affine results.
template <typename T>
__global__ void gate_qk_rotary_kernel(const T* z, long long ldz, const float* gamma, const float* beta,
                                      const float* rot, int period, int q_offset, T* qo, long long ldq, T* ko,
                                      long long ldk, long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int half = cols >> 1;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += warps) {
    const T* zr = z + r * ldz;
    float ss = 0.f;
    for (int j = lane; j < half; j += 32) {
      const float a = Elem<T>::ld(zr + 2 * j), b = Elem<T>::ld(zr + 2 * j + 1);
      ss = fmaf(a, a, fmaf(b, b, ss));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.f / fmaxf(sqrtf(ss), eps);
    const int pos = (int)(r % period);
    const float2* rk = reinterpret_cast<const float2*>(rot) + (size_t)pos * half;
    const float2* rq = reinterpret_cast<const float2*>(rot) + (size_t)(pos + q_offset) * half;
    for (int j = lane; j < half; j += 32) {
      const int c = 2 * j;
      const float a = Elem<T>::ld(zr + c) * inv, b = Elem<T>::ld(zr + c + 1) * inv;
      const float qa = fmaf(a, gamma[c] + 1.f, beta[c]), qb = fmaf(b, gamma[c + 1] + 1.f, beta[c + 1]);
      const float ka = fmaf(a, gamma[cols + c] + 1.f, beta[cols + c]);
      const float kb = fmaf(b, gamma[cols + c + 1] + 1.f, beta[cols + c + 1]);
      const float2 wq = __ldg(rq + j), wk = __ldg(rk + j);
      Elem<T>::st(qo + r * ldq + c, qa * wq.x - qb * wq.y);
      Elem<T>::st(qo + r * ldq + c + 1, qa * wq.y + qb * wq.x);
      Elem<T>::st(ko + r * ldk + c, ka * wk.x - kb * wk.y);
      Elem<T>::st(ko + r * ldk + c + 1, ka * wk.y + kb * wk.x);
    }
  }
}

}  // namespace mega

using namespace mega;

static int tsn_fwd_common(const void* x, void* y, int dtype, int B, int L, int D, int64_t xsb, int64_t xsl,
                          int64_t xsd, int64_t ysb, int64_t ysl, int64_t ysd, const int64_t* prev_count,
                          const float* prev_mean, const float* prev_var, const float* gamma, const float* beta,
                          const uint8_t* pad_mask, int num_groups, double eps, int64_t* count_out,
                          float* mean_out, float* var_out, float* cummean, float* cumrstd, float* group_mean,
                          mega_stream_t stream) {
  if (!x || !y || !prev_count || !prev_mean || !prev_var || !gamma || !beta || !count_out || !mean_out ||
      !var_out)
    return MEGA_ERR_NULL;
  // every thread block of a sequence reads its incoming count; one of them writes the new one
  if ((const void*)count_out == (const void*)prev_count) return MEGA_ERR_UNSUPPORTED;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || L <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  const int G = (num_groups <= 0 || num_groups == D) ? D : num_groups;
  if (D % G != 0) return MEGA_ERR_SHAPE;
  if (!aligned_to(x, elem_size(dtype)) || !aligned_to(y, elem_size(dtype))) return MEGA_ERR_ALIGN;
  TsnArgs a{};
  a.x = x; a.y = y; a.B = B; a.L = L; a.D = D; a.G = G;
  a.xsb = xsb; a.xsl = xsl; a.xsd = xsd; a.ysb = ysb; a.ysl = ysl; a.ysd = ysd;
  a.prev_count = (const long long*)prev_count; a.prev_mean = prev_mean; a.prev_var = prev_var;
  a.gamma = gamma; a.beta = beta; a.mask = pad_mask; a.eps = (float)eps;
  a.count_out = (long long*)count_out; a.mean_out = mean_out; a.var_out = var_out;
  a.cummean = cummean; a.cumrstd = cumrstd; a.group_mean = group_mean;
  if (G == D) {
    if (x != y) {
      StreamArgs sa{};
      sa.B = B; sa.L = L; sa.D = D; sa.N = 0;
      sa.prev_count = a.prev_count; sa.prev_mean = prev_mean; sa.prev_var = prev_var; sa.gamma = gamma;
      sa.beta = beta; sa.eps = (float)eps; sa.count_out = a.count_out; sa.mean_out = mean_out; sa.var_out = var_out;
      sa.mask = pad_mask;
      sa.cummean = cummean; sa.cumrstd = cumrstd;
      // bf16 without a mask and without the saves for backward: the tensor-core kernel's prefix sums
      if (!cummean && mma_cl_try(dtype, x, y, nullptr, xsb, xsl, xsd, ysb, ysl, ysd, true, sa, (cudaStream_t)stream))
        return check_launch("timestep_norm_fwd(mma)");
      if (stream_cl_try(dtype, x, y, nullptr, xsb, xsl, xsd, ysb, ysl, ysd, true, false, sa, (cudaStream_t)stream))
        return check_launch("timestep_norm_fwd(stream)");
    }
    const unsigned grid = (unsigned)(((long long)B * D + 127) / 128);
    MEGA_DISPATCH_DTYPE(dtype, {
      if (pad_mask && cummean) launch(tsn_plain_kernel<T, true, true>, grid, 128, 0, stream, a);
      else if (pad_mask) launch(tsn_plain_kernel<T, true, false>, grid, 128, 0, stream, a);
      else if (cummean) launch(tsn_plain_kernel<T, false, true>, grid, 128, 0, stream, a);
      else launch(tsn_plain_kernel<T, false, false>, grid, 128, 0, stream, a);
    });
  } else {
    GroupStreamArgs ga{};
    ga.B = B; ga.L = L; ga.D = D; ga.G = G;
    ga.prev_count = a.prev_count; ga.prev_mean = prev_mean; ga.prev_var = prev_var; ga.gamma = gamma; ga.beta = beta;
    ga.mask = pad_mask; ga.eps = (float)eps; ga.count_out = a.count_out; ga.mean_out = mean_out; ga.var_out = var_out;
    ga.cummean = cummean; ga.cumrstd = cumrstd; ga.group_mean = group_mean;
    if (tsn_group_stream_try(dtype, x, y, xsb, xsl, xsd, ysb, ysl, ysd, ga, (cudaStream_t)stream))
      return check_launch("timestep_norm_fwd(group stream)");
    const unsigned grid = (unsigned)(((long long)B * G * 32 + 127) / 128);
    MEGA_DISPATCH_DTYPE(dtype, launch(tsn_group_kernel<T>, grid, 128, 0, stream, a));
  }
  return check_launch("timestep_norm_fwd");
}

extern "C" int mega_timestep_norm_fwd(const void* x, void* y, int dtype, int B, int L, int D, int64_t xsb,
                                      int64_t xsl, int64_t xsd, int64_t ysb, int64_t ysl, int64_t ysd,
                                      const int64_t* prev_count, const float* prev_mean,
                                      const float* prev_var, const float* gamma, const float* beta,
                                      const uint8_t* pad_mask, int num_groups, double eps,
                                      int64_t* count_out, float* mean_out, float* var_out,
                                      mega_stream_t stream) {
  return tsn_fwd_common(x, y, dtype, B, L, D, xsb, xsl, xsd, ysb, ysl, ysd, prev_count, prev_mean, prev_var,
                        gamma, beta, pad_mask, num_groups, eps, count_out, mean_out, var_out, nullptr, nullptr,
                        nullptr, stream);
}

extern "C" int mega_timestep_norm_fwd_train(const void* x, void* y, int dtype, int B, int L, int D, int64_t xsb,
                                            int64_t xsl, int64_t xsd, int64_t ysb, int64_t ysl, int64_t ysd,
                                            const int64_t* prev_count, const float* prev_mean,
                                            const float* prev_var, const float* gamma, const float* beta,
                                            const uint8_t* pad_mask, int num_groups, double eps,
                                            int64_t* count_out, float* mean_out, float* var_out, float* cummean,
                                            float* cumrstd, float* group_mean, mega_stream_t stream) {
  if (!cummean || !cumrstd) return MEGA_ERR_NULL;
  const bool grouped = num_groups > 0 && num_groups != D;
  if (grouped && !group_mean) return MEGA_ERR_NULL;
  return tsn_fwd_common(x, y, dtype, B, L, D, xsb, xsl, xsd, ysb, ysl, ysd, prev_count, prev_mean, prev_var,
                        gamma, beta, pad_mask, num_groups, eps, count_out, mean_out, var_out, cummean, cumrstd,
                        grouped ? group_mean : nullptr, stream);
}

extern "C" int mega_sequence_norm_fwd(const void* x, void* y, int dtype, int B, int D, int L, int64_t xsb,
                                      int64_t xsd, int64_t xsl, int64_t ysb, int64_t ysd, int64_t ysl,
                                      const float* gamma, const float* beta, const uint8_t* pad_mask,
                                      int num_groups, double eps, int64_t* count_out, float* mean_out,
                                      float* rstd_out, mega_stream_t stream) {
  if (!x || !y || !gamma || !beta || !count_out || !mean_out || !rstd_out) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || L <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  const int G = (num_groups <= 0 || num_groups == D) ? D : num_groups;
  if (D % G != 0) return MEGA_ERR_SHAPE;
  if (!aligned_to(x, elem_size(dtype)) || !aligned_to(y, elem_size(dtype))) return MEGA_ERR_ALIGN;
  SqnArgs a{};
  a.x = x; a.y = y; a.B = B; a.D = D; a.L = L; a.G = G;
  a.xsb = xsb; a.xsd = xsd; a.xsl = xsl; a.ysb = ysb; a.ysd = ysd; a.ysl = ysl;
  a.gamma = gamma; a.beta = beta; a.mask = pad_mask; a.eps = (float)eps;
  a.count_out = (long long*)count_out; a.mean_out = mean_out; a.rstd_out = rstd_out;
  if (G == D && xsd == 1 && xsl != 1) {
    const unsigned grid = (unsigned)(((long long)B * D + 127) / 128);
    MEGA_DISPATCH_DTYPE(dtype, launch(sqn_column_kernel<T>, grid, 128, 0, stream, a));
  } else {
    if ((long long)B * G > 0x7fffffffLL) return MEGA_ERR_SHAPE;
    const long long n = (long long)(D / G) * L;
    // cache the segment in shared memory when it fits (opt-in limit, leaves room for 1 KB of statics)
    static bool attr_ok = false;
    static std::once_flag once;
    std::call_once(once, [] {
      attr_ok = cudaFuncSetAttribute(sqn_segment_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess &&
                cudaFuncSetAttribute(sqn_segment_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess &&
                cudaFuncSetAttribute(sqn_segment_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess;
      cudaGetLastError();
    });
    const int cap = (attr_ok ? 200 : 40) * 1024 / 4;
    const int cache_elems = n <= cap ? (int)n : 0;
    MEGA_DISPATCH_DTYPE(dtype, launch(sqn_segment_kernel<T>, (unsigned)(B * G), 256,
                                      (size_t)cache_elems * sizeof(float), stream, a, cache_elems));
  }
  return check_launch("sequence_norm_fwd");
}

static int gate_common(int op, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
                       int64_t ldc, const void* d, int64_t ldd, void* y, int64_t ldy, int dtype,
                       int64_t rows, int cols, mega_stream_t stream) {
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (rows <= 0 || cols <= 0) return MEGA_ERR_SHAPE;
  const long long n = rows * cols;
  {
    // 16-byte path: every operand present has a 16-byte aligned base and pitch, cols a multiple of the vector
    const int vn = 16 / elem_size(dtype);
    const long long es = elem_size(dtype);
    auto ok16 = [&](const void* p, long long ld) { return p == nullptr || (aligned_to(p, 16) && (ld * es) % 16 == 0); };
    const long long nvec = n / vn;
    if (cols % vn == 0 && ok16(a, lda) && ok16(b, ldb) && ok16(c, ldc) && ok16(d, ldd) && ok16(y, ldy) &&
        nvec < 0xffffffffLL) {
      constexpr int kU = 2;
      const long long want = (nvec + 256 * kU - 1) / (256 * kU);
      const unsigned gridv = (unsigned)(want > 148 * 32 ? 148 * 32 : want);
      const unsigned vpr = (unsigned)(cols / vn);
      MEGA_DISPATCH_DTYPE(dtype, {
        if (op == 0)
          launch(gate_vec_kernel<T, 0, kU>, gridv, 256, 0, stream, (const T*)a, lda, (const T*)b, ldb, (const T*)c, ldc,
                 (const T*)d, ldd, (T*)y, ldy, (unsigned)nvec, vpr);
        else if (op == 1)
          launch(gate_vec_kernel<T, 1, kU>, gridv, 256, 0, stream, (const T*)a, lda, (const T*)b, ldb, (const T*)c, ldc,
                 (const T*)d, ldd, (T*)y, ldy, (unsigned)nvec, vpr);
        else
          launch(gate_vec_kernel<T, 2, kU>, gridv, 256, 0, stream, (const T*)a, lda, (const T*)b, ldb, (const T*)c, ldc,
                 (const T*)d, ldd, (T*)y, ldy, (unsigned)nvec, vpr);
      });
      return check_launch("gate");
    }
  }
  const unsigned grid = (unsigned)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  MEGA_DISPATCH_DTYPE(dtype, {
    if (op == 0)
      launch(gate_kernel<T, 0>, grid, 256, 0, stream, (const T*)a, lda, (const T*)b, ldb, (const T*)c, ldc,
             (const T*)d, ldd, (T*)y, ldy, rows, cols);
    else if (op == 1)
      launch(gate_kernel<T, 1>, grid, 256, 0, stream, (const T*)a, lda, (const T*)b, ldb, (const T*)c, ldc,
             (const T*)d, ldd, (T*)y, ldy, rows, cols);
    else
      launch(gate_kernel<T, 2>, grid, 256, 0, stream, (const T*)a, lda, (const T*)b, ldb, (const T*)c, ldc,
             (const T*)d, ldd, (T*)y, ldy, rows, cols);
  });
  return check_launch("gate");
}

extern "C" int mega_gate_silu(const void* a, int64_t ld_a, const void* b, int64_t ld_b, void* y,
                              int64_t ld_y, int dtype, int64_t rows, int cols, mega_stream_t stream) {
  if (!a || !y) return MEGA_ERR_NULL;
  return gate_common(0, a, ld_a, b, ld_b, nullptr, 0, nullptr, 0, y, ld_y, dtype, rows, cols, stream);
}

extern "C" int mega_gate_mul_silu(const void* a, int64_t ld_a, const void* r, int64_t ld_r, void* y,
                                  int64_t ld_y, int dtype, int64_t rows, int cols, mega_stream_t stream) {
  if (!a || !r || !y) return MEGA_ERR_NULL;
  return gate_common(1, a, ld_a, r, ld_r, nullptr, 0, nullptr, 0, y, ld_y, dtype, rows, cols, stream);
}

extern "C" int mega_gate_output(const void* residual, int64_t ld_res, const void* u, int64_t ld_u,
                                const void* hx, int64_t ld_hx, const void* h_lin, int64_t ld_h, void* out,
                                int64_t ld_out, int dtype, int64_t rows, int cols, mega_stream_t stream) {
  if (!residual || !u || !hx || !h_lin || !out) return MEGA_ERR_NULL;
  return gate_common(2, residual, ld_res, u, ld_u, hx, ld_hx, h_lin, ld_h, out, ld_out, dtype, rows, cols,
                     stream);
}

extern "C" int mega_gate_qk(const void* z, int64_t ld_z, const float* gamma, const float* beta, void* q,
                            int64_t ld_q, void* k, int64_t ld_k, int dtype, int64_t rows, int cols, double eps,
                            mega_stream_t stream) {
  if (!z || !gamma || !beta || !q || !k) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (rows <= 0 || cols <= 0) return MEGA_ERR_SHAPE;
  if (ld_z < cols || ld_q < cols || ld_k < cols) return MEGA_ERR_STRIDE;
  const long long blocks = (rows + 7) / 8;  // 8 warps per block, one row per warp and pass
  const unsigned grid = (unsigned)(blocks > 148 * 8 ? 148 * 8 : blocks);
  MEGA_DISPATCH_DTYPE(dtype, launch(gate_qk_kernel<T>, grid, 256, 0, stream, (const T*)z, (long long)ld_z, gamma,
                                    beta, (T*)q, (long long)ld_q, (T*)k, (long long)ld_k, (long long)rows, cols,
                                    (float)eps));
  return check_launch("gate_qk");
}

extern "C" int mega_gate_qk_rotary(const void* z, int64_t ld_z, const float* gamma, const float* beta, const float* rot,
                                   int positions, int period, int q_offset, void* q, int64_t ld_q, void* k,
                                   int64_t ld_k, int dtype, int64_t rows, int cols, double eps, mega_stream_t stream) {
  if (!z || !gamma || !beta || !rot || !q || !k) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (rows <= 0 || cols <= 0 || (cols & 1) || period <= 0 || q_offset < 0 || period + q_offset > positions)
    return MEGA_ERR_SHAPE;
  if (ld_z < cols || ld_q < cols || ld_k < cols) return MEGA_ERR_STRIDE;
  if (!aligned_to(rot, 8)) return MEGA_ERR_ALIGN;
  const long long blocks = (rows + 7) / 8;  // 8 warps per block, one row per warp and pass
  const unsigned grid = (unsigned)(blocks > 148 * 8 ? 148 * 8 : blocks);
  MEGA_DISPATCH_DTYPE(dtype, launch(gate_qk_rotary_kernel<T>, grid, 256, 0, stream, (const T*)z, (long long)ld_z, gamma,
                                    beta, rot, period, q_offset, (T*)q, (long long)ld_q, (T*)k, (long long)ld_k,
                                    (long long)rows, cols, (float)eps));
  return check_launch("gate_qk_rotary");
}
