// Fused per-feature TimestepNorm -> causal EMA: one pass over x, one write of y.
//
// Generic variant: one thread per (batch, channel), sequential over time, so every
// per-channel quantity (Welford state, pole states) lives in registers.  Works for any
// strides; coalesced when the channel stride is 1.
#include <type_traits>

#include "common.cuh"
#include "stream_cl.cuh"

namespace mega {

struct FusedArgs {
  const void* x;
  void* y;
  void* xn;
  int B, L, D, N;
  long long xsb, xsl, xsd, ysb, ysl, ysd;
  const long long* prev_count;
  long long count_offset;  // added to prev_count (a call that continues another call's positions)
  const float *prev_mean, *prev_var, *gamma, *beta;
  float eps;
  long long* count_out;
  float *mean_out, *var_out;
  const float *p, *q, *g, *omega;
  const unsigned char* mask;
  const float* h_in;
  float* h_out;
  int silu;
};

template <typename T, int NP, bool kState>
__global__ void __launch_bounds__(128) tsn_ema_rows_kernel(FusedArgs a) {
  long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)a.B * a.D) return;
  const int d = (int)(gid % a.D);
  const int b = (int)(gid / a.D);
  float q[NP], c[NP], s[NP], pp[kState ? NP : 1];
#pragma unroll
  for (int n = 0; n < NP; ++n) {
    float pn = 0.f, qn = 0.f, gn = 0.f;
    if (n < a.N) {
      pn = __ldg(a.p + (size_t)d * a.N + n);
      qn = __ldg(a.q + (size_t)d * a.N + n);
      gn = __ldg(a.g + (size_t)d * a.N + n);
    }
    q[n] = qn;
    if (kState) {
      c[n] = gn; pp[n] = pn;
      s[n] = (a.h_in != nullptr && n < a.N) ? __ldg(a.h_in + (size_t)gid * a.N + n) : 0.f;
    } else {
      c[n] = pn * gn; s[n] = 0.f;
    }
  }
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ysb + d * a.ysd;
  T* np_ = a.xn ? reinterpret_cast<T*>(a.xn) + b * a.ysb + d * a.ysd : nullptr;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  const long long cnt0 = a.prev_count[b] + a.count_offset;
  const float cnt0f = (float)cnt0;  // 32-bit step counter on top: no 64-bit conversions in the loop
  int seen = 0;
  float mean = a.prev_mean[gid], var = a.prev_var[gid];
  const float w = __ldg(a.gamma + d), bb = __ldg(a.beta + d), om = __ldg(a.omega + d);
  constexpr int U = 8;
  // mask presence is compile-time inside the loop (a run-time pointer test between the loads of
  // a batch serialises them)
  auto scan = [&](auto mask_tag) {
  constexpr bool kMask = decltype(mask_tag)::value;
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
        const float d1 = xv[u] - mean;
        m1 = fmaf(coef, d1, mean);
        const float d2 = fmaf(d1, xv[u] - m1, -var);
        m2 = fmaf(coef, d2, var);
        const float rstd = rsqrt_approx(m2 + a.eps);
        const float xn = mk[u] ? 0.f : fmaf((xv[u] - m1) * rstd, w, bb);
        if (!mk[u]) { mean = m1; var = m2; ++seen; }
        if (np_) Elem<T>::st(np_ + t * a.ysl, xn);
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int n = 0; n < NP; n += 2) {
          if (kState) {
            s[n] = fmaf(q[n], s[n], pp[n] * xn);
            s[n + 1] = fmaf(q[n + 1], s[n + 1], pp[n + 1] * xn);
          } else {
            s[n] = fmaf(q[n], s[n], xn);
            s[n + 1] = fmaf(q[n + 1], s[n + 1], xn);
          }
          a0 = fmaf(c[n], s[n], a0);
          a1 = fmaf(c[n + 1], s[n + 1], a1);
        }
        float v = fmaf(om, xn, a0 + a1);
        if (a.silu) v = siluf_(v);
        Elem<T>::st(yp + t * a.ysl, v);
      }
    }
  }
  };
  if (mp) scan(std::true_type{}); else scan(std::false_type{});
  a.mean_out[gid] = mean;
  a.var_out[gid] = var;
  if (d == 0) a.count_out[b] = cnt0 + seen;
  if (kState && a.h_out) {
#pragma unroll
    for (int n = 0; n < NP; ++n)
      if (n < a.N) a.h_out[(size_t)gid * a.N + n] = s[n];
  }
}

// Single-token decode step of the fused pair: one thread per (sequence, channel) updates the
// TimestepNorm statistics and the pole states in place and emits one output element.
template <typename T, int NP>
__global__ void __launch_bounds__(128) tsn_ema_step_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                           T* __restrict__ xn_out, int B, int D, int N,
                                                           long long* count, float* mean, float* var,
                                                           const float* __restrict__ gamma,
                                                           const float* __restrict__ beta, float eps,
                                                           const float* __restrict__ p, const float* __restrict__ q,
                                                           const float* __restrict__ g,
                                                           const float* __restrict__ omega, float* h, int silu,
                                                           int use_norm) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)B * D) return;
  const int d = (int)(gid % D);
  const int b = (int)(gid / D);
  float xv = Elem<T>::ld(x + gid);
  if (use_norm) {
    const long long c = count[b];
    float m1, m2;
    const float coef = __frcp_rn((float)(c + 1));
    const float d1 = xv - mean[gid];
    m1 = fmaf(coef, d1, mean[gid]);
    const float d2 = fmaf(d1, xv - m1, -var[gid]);
    m2 = fmaf(coef, d2, var[gid]);
    xv = fmaf((xv - m1) * rsqrtf(m2 + eps), __ldg(gamma + d), __ldg(beta + d));
    mean[gid] = m1;
    var[gid] = m2;
    if (xn_out) Elem<T>::st(xn_out + gid, xv);
  }
  float acc = 0.f;
  float4* hp = reinterpret_cast<float4*>(h + gid * N);
  if (NP >= 4 && (N & 3) == 0) {
#pragma unroll
    for (int n4 = 0; n4 < NP / 4; ++n4) {
      if (n4 * 4 < N) {
        float4 hv = hp[n4];
        const float4 qv = __ldg(reinterpret_cast<const float4*>(q + (size_t)d * N) + n4);
        const float4 pv = __ldg(reinterpret_cast<const float4*>(p + (size_t)d * N) + n4);
        const float4 gv = __ldg(reinterpret_cast<const float4*>(g + (size_t)d * N) + n4);
        hv.x = fmaf(qv.x, hv.x, pv.x * xv); hv.y = fmaf(qv.y, hv.y, pv.y * xv);
        hv.z = fmaf(qv.z, hv.z, pv.z * xv); hv.w = fmaf(qv.w, hv.w, pv.w * xv);
        acc = fmaf(gv.x, hv.x, acc); acc = fmaf(gv.y, hv.y, acc);
        acc = fmaf(gv.z, hv.z, acc); acc = fmaf(gv.w, hv.w, acc);
        hp[n4] = hv;
      }
    }
  } else {
#pragma unroll
    for (int n = 0; n < NP; ++n) {
      if (n < N) {
        const float hn = fmaf(__ldg(q + (size_t)d * N + n), h[gid * N + n], __ldg(p + (size_t)d * N + n) * xv);
        h[gid * N + n] = hn;
        acc = fmaf(__ldg(g + (size_t)d * N + n), hn, acc);
      }
    }
  }
  float v = fmaf(__ldg(omega + d), xv, acc);
  if (silu) v = siluf_(v);
  Elem<T>::st(y + gid, v);
}

// The same step with LN = N / 4 lanes per (sequence, channel): a lane owns four poles, so a warp
// reads and writes the states as whole contiguous rows (32 / LN channels x N floats per access),
// and a thread walks BB sequences with the coefficients of its poles in registers (all loads of
// the BB steps are issued before the arithmetic).  With use_norm the TimestepNorm update runs
// redundantly in the LN lanes; lane 0 stores the statistics and the output.  h_in may be NULL
// (zero state) and may alias h_out.
template <typename T, int LN, int BB>
__global__ void __launch_bounds__(128) tsn_ema_step_lanes_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                 T* __restrict__ xn_out, int B, int D,
                                                                 const long long* count, float* mean, float* var,
                                                                 const float* __restrict__ gamma,
                                                                 const float* __restrict__ beta, float eps,
                                                                 const float* __restrict__ p,
                                                                 const float* __restrict__ q,
                                                                 const float* __restrict__ g,
                                                                 const float* __restrict__ omega, const float* h_in,
                                                                 float* h_out, int silu, int use_norm,
                                                                 long long* count_next) {
  constexpr int N = LN * 4;
  const int sub = threadIdx.x % LN;
  const int d = blockIdx.x * (128 / LN) + threadIdx.x / LN;
  const bool live = d < D;  // dead lanes stay for the shuffles
  const int b0 = blockIdx.y * BB;
  float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), pv = qv, gv = qv;
  float om = 0.f, gam = 1.f, bet = 0.f;
  if (live) {
    qv = __ldg(reinterpret_cast<const float4*>(q + (size_t)d * N) + sub);
    pv = __ldg(reinterpret_cast<const float4*>(p + (size_t)d * N) + sub);
    gv = __ldg(reinterpret_cast<const float4*>(g + (size_t)d * N) + sub);
    om = __ldg(omega + d);
    if (use_norm) {
      gam = __ldg(gamma + d);
      bet = __ldg(beta + d);
    }
  }
  float4 hv[BB];
  float xv[BB], mu[BB], vr[BB], coef[BB];
#pragma unroll
  for (int j = 0; j < BB; ++j) {
    const int b = b0 + j;
    const bool ok = live && b < B;
    const size_t gid = (size_t)b * D + d;
    hv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    xv[j] = mu[j] = 0.f;
    vr[j] = coef[j] = 1.f;
    if (ok) {
      if (h_in) hv[j] = *(reinterpret_cast<const float4*>(h_in + gid * N) + sub);
      xv[j] = Elem<T>::ld(x + gid);
      if (use_norm) {
        mu[j] = mean[gid];
        vr[j] = var[gid];
        coef[j] = __frcp_rn((float)(count[b] + 1));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < BB; ++j) {
    const int b = b0 + j;
    const bool ok = live && b < B;
    const size_t gid = (size_t)b * D + d;
    float xin = xv[j];
    float m1 = 0.f, m2 = 0.f;
    if (use_norm) {
      const float d1 = xin - mu[j];
      m1 = fmaf(coef[j], d1, mu[j]);
      const float d2 = fmaf(d1, xin - m1, -vr[j]);
      m2 = fmaf(coef[j], d2, vr[j]);
      xin = fmaf((xin - m1) * rsqrtf(m2 + eps), gam, bet);
    }
    float4 hn = hv[j];
    hn.x = fmaf(qv.x, hn.x, pv.x * xin); hn.y = fmaf(qv.y, hn.y, pv.y * xin);
    hn.z = fmaf(qv.z, hn.z, pv.z * xin); hn.w = fmaf(qv.w, hn.w, pv.w * xin);
    float acc = fmaf(gv.x, hn.x, fmaf(gv.y, hn.y, fmaf(gv.z, hn.z, gv.w * hn.w)));
#pragma unroll
    for (int o = 1; o < LN; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (ok) {
      *(reinterpret_cast<float4*>(h_out + gid * N) + sub) = hn;
      if (sub == 0) {
        float v = fmaf(om, xin, acc);
        if (silu) v = siluf_(v);
        Elem<T>::st(y + gid, v);
        if (use_norm) {
          mean[gid] = m1;
          var[gid] = m2;
          if (xn_out) Elem<T>::st(xn_out + gid, xin);
        }
      }
    }
  }
  // the counts after this step go to a second array (never the one every CTA is reading)
  if (count_next && d == 0 && sub == 0) {
#pragma unroll
    for (int j = 0; j < BB; ++j)
      if (b0 + j < B) count_next[b0 + j] = count[b0 + j] + 1;
  }
}

// Launches the lane-split step when the pole count allows it (N = 4, 8, 16 or 32, states 16-byte
// aligned); returns false otherwise.
template <typename T>
static bool launch_step_lanes(const T* x, T* y, T* xn_out, int B, int D, int N, const long long* count, float* mean,
                              float* var, const float* gamma, const float* beta, float eps, const float* p,
                              const float* q, const float* g, const float* omega, const float* h_in, float* h_out,
                              int silu, int use_norm, mega_stream_t stream, long long* count_next) {
  if (N != 4 && N != 8 && N != 16 && N != 32) return false;
  if (!aligned_to(h_out, 16) || (h_in && !aligned_to(h_in, 16)) || !aligned_to(p, 16) || !aligned_to(q, 16) ||
      !aligned_to(g, 16))
    return false;
  constexpr int BB = 4;
  const int ln = N / 4;
  dim3 grid((unsigned)((D + 128 / ln - 1) / (128 / ln)), (unsigned)((B + BB - 1) / BB));
  if (grid.y > 65535) return false;
#define MEGA_STEP_LANES(LNV)                                                                              \
  launch(tsn_ema_step_lanes_kernel<T, LNV, BB>, grid, 128, 0, stream, x, y, xn_out, B, D, count, mean, var, \
         gamma, beta, eps, p, q, g, omega, h_in, h_out, silu, use_norm, count_next)
  if (ln == 1) MEGA_STEP_LANES(1);
  else if (ln == 2) MEGA_STEP_LANES(2);
  else if (ln == 4) MEGA_STEP_LANES(4);
  else MEGA_STEP_LANES(8);
#undef MEGA_STEP_LANES
  return true;
}

bool step_lanes_try(int dtype, const void* x, void* y, void* xn_out, int B, int D, int N, const long long* count,
                    float* mean, float* var, const float* gamma, const float* beta, float eps, const float* p,
                    const float* q, const float* g, const float* omega, const float* h_in, float* h_out, int silu,
                    void* stream, long long* count_next) {
  const int use_norm = count != nullptr;
  switch (dtype) {
    case MEGA_F32:
      return launch_step_lanes<float>((const float*)x, (float*)y, (float*)xn_out, B, D, N, count, mean, var, gamma,
                                      beta, eps, p, q, g, omega, h_in, h_out, silu, use_norm, stream, count_next);
    case MEGA_BF16:
      return launch_step_lanes<__nv_bfloat16>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (__nv_bfloat16*)xn_out, B,
                                              D, N, count, mean, var, gamma, beta, eps, p, q, g, omega, h_in, h_out,
                                              silu, use_norm, stream, count_next);
    case MEGA_F16:
      return launch_step_lanes<__half>((const __half*)x, (__half*)y, (__half*)xn_out, B, D, N, count, mean, var,
                                       gamma, beta, eps, p, q, g, omega, h_in, h_out, silu, use_norm, stream,
                                       count_next);
    default:
      return false;
  }
}

// One thread per sequence bumps the counts after the element kernel has read them.
__global__ void tsn_count_step_kernel(long long* count, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) count[b] += 1;
}

__global__ void tsn_count_next_kernel(const long long* count, long long* next, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) next[b] = count[b] + 1;
}

}  // namespace mega

using namespace mega;

extern "C" MEGA_API int mega_tsn_ema_step(const void* x, void* y, void* xn_out, int dtype, int B, int D,
                                          int64_t* count, int64_t* count_next, float* mean, float* var,
                                          const float* gamma, const float* beta, double eps, const float* p,
                                          const float* q,
                                          const float* gamma_hat, const float* omega, int N, float* h,
                                          unsigned flags, mega_stream_t stream) {
  if (!x || !y || !p || !q || !gamma_hat || !omega || !h) return MEGA_ERR_NULL;
  const int use_norm = count != nullptr;
  if (use_norm && (!mean || !var || !gamma || !beta)) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  if (!aligned_to(h, 16) && (N & 3) == 0) return MEGA_ERR_ALIGN;
  const int np = next_pow2_ndim(N);
  const unsigned grid = (unsigned)(((long long)B * D + 127) / 128);
  const int silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
  // a distinct count_next array takes the bumped counts from the element kernel itself
  long long* next = (use_norm && count_next && count_next != count) ? (long long*)count_next : nullptr;
  if (step_lanes_try(dtype, x, y, xn_out, B, D, N, (const long long*)count, mean, var, gamma, beta, (float)eps, p, q,
                     gamma_hat, omega, h, h, silu, stream, next)) {
    if (next) return check_launch("tsn_ema_step");
  } else {
    MEGA_DISPATCH_DTYPE(dtype, MEGA_DISPATCH_NP(np, launch(tsn_ema_step_kernel<T, NP>, grid, 128, 0, stream,
                                                           (const T*)x, (T*)y, (T*)xn_out, B, D, N,
                                                           (long long*)count, mean, var, gamma, beta, (float)eps,
                                                           p, q, gamma_hat, omega, h, silu, use_norm)));
  }
  if (use_norm) {
    if (next)  // generic kernel: the second array is filled by a copy-and-increment launch
      launch(tsn_count_next_kernel, (unsigned)((B + 127) / 128), 128, 0, stream, (const long long*)count, next, B);
    else
      launch(tsn_count_step_kernel, (unsigned)((B + 127) / 128), 128, 0, stream, (long long*)count, B);
  }
  return check_launch("tsn_ema_step");
}

extern "C" int mega_tsn_ema_fwd_runs(const void* x, void* y, int dtype, int B, int L, int D, int64_t xsb, int64_t xsl,
                                     int64_t xsd, int64_t ysb, int64_t ysl, int64_t ysd, const int64_t* prev_count,
                                     const float* prev_mean, const float* prev_var, const float* gamma,
                                     const float* beta, double eps, int64_t* count_out, float* mean_out,
                                     float* var_out, const float* p, const float* q, const float* gamma_hat,
                                     const float* omega, int N, const float* h_in, float* h_out, unsigned flags,
                                     int runs, mega_stream_t stream) {
  if (!x || !y || !prev_count || !prev_mean || !prev_var || !gamma || !beta || !count_out || !mean_out ||
      !var_out || !p || !q || !gamma_hat || !omega)
    return MEGA_ERR_NULL;
  // every thread block of a sequence reads its incoming count; one of them writes the new one
  if ((const void*)count_out == (const void*)prev_count) return MEGA_ERR_UNSUPPORTED;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || L <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  if (flags & MEGA_EMA_BIDIRECTIONAL) return MEGA_ERR_UNSUPPORTED;
  if (runs != 2 && runs != 4 && runs != 8) return MEGA_ERR_SHAPE;
  if (!aligned_to(x, elem_size(dtype)) || !aligned_to(y, elem_size(dtype))) return MEGA_ERR_ALIGN;
  StreamArgs sa{};
  sa.B = B; sa.L = L; sa.D = D; sa.N = N;
  sa.prev_count = (const long long*)prev_count; sa.prev_mean = prev_mean; sa.prev_var = prev_var; sa.gamma = gamma;
  sa.beta = beta; sa.eps = (float)eps; sa.count_out = (long long*)count_out; sa.mean_out = mean_out;
  sa.var_out = var_out; sa.p = p; sa.q = q; sa.g = gamma_hat; sa.omega = omega; sa.h_in = h_in; sa.h_out = h_out;
  sa.silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
  if (!mma_cl_runs(dtype, x, y, xsb, xsl, xsd, ysb, ysl, ysd, sa, runs, (cudaStream_t)stream))
    return MEGA_ERR_UNSUPPORTED;
  return check_launch("tsn_ema_fwd_runs");
}

extern "C" int mega_tsn_ema_fwd(const void* x, void* y, void* xn_out, int dtype, int B, int L, int D,
                                int64_t xsb, int64_t xsl, int64_t xsd, int64_t ysb, int64_t ysl, int64_t ysd,
                                const int64_t* prev_count, const float* prev_mean, const float* prev_var,
                                const float* gamma, const float* beta, double eps, int64_t* count_out,
                                float* mean_out, float* var_out, const float* p, const float* q,
                                const float* gamma_hat, const float* omega, int N, const uint8_t* pad_mask,
                                const float* h_in, float* h_out, unsigned flags, mega_stream_t stream) {
  if (!x || !y || !prev_count || !prev_mean || !prev_var || !gamma || !beta || !count_out || !mean_out ||
      !var_out || !p || !q || !gamma_hat || !omega)
    return MEGA_ERR_NULL;
  // every thread block of a sequence reads its incoming count; one of them writes the new one
  if ((const void*)count_out == (const void*)prev_count) return MEGA_ERR_UNSUPPORTED;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || L <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  if (flags & MEGA_EMA_BIDIRECTIONAL) return MEGA_ERR_UNSUPPORTED;
  if (!aligned_to(x, elem_size(dtype)) || !aligned_to(y, elem_size(dtype)) ||
      (xn_out && !aligned_to(xn_out, elem_size(dtype))))
    return MEGA_ERR_ALIGN;
  FusedArgs a{};
  a.x = x; a.y = y; a.xn = xn_out; a.B = B; a.L = L; a.D = D; a.N = N;
  a.xsb = xsb; a.xsl = xsl; a.xsd = xsd; a.ysb = ysb; a.ysl = ysl; a.ysd = ysd;
  a.prev_count = (const long long*)prev_count; a.prev_mean = prev_mean; a.prev_var = prev_var;
  a.gamma = gamma; a.beta = beta; a.eps = (float)eps;
  a.count_out = (long long*)count_out; a.mean_out = mean_out; a.var_out = var_out;
  a.p = p; a.q = q; a.g = gamma_hat; a.omega = omega; a.mask = pad_mask; a.h_in = h_in; a.h_out = h_out;
  a.silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
  {
    StreamArgs sa{};
    sa.B = B; sa.L = L; sa.D = D; sa.N = N;
    sa.prev_count = a.prev_count; sa.prev_mean = prev_mean; sa.prev_var = prev_var; sa.gamma = gamma;
    sa.beta = beta; sa.eps = (float)eps; sa.count_out = a.count_out; sa.mean_out = mean_out; sa.var_out = var_out;
    sa.p = p; sa.q = q; sa.g = gamma_hat; sa.omega = omega; sa.h_in = h_in; sa.h_out = h_out; sa.mask = pad_mask;
    sa.silu = a.silu;
    // A state is exported and L is not a multiple of the tensor-core kernel's step of 32 positions (it
    // cannot stop a pole state in mid-step): the head, a multiple of 32, goes to the tensor-core
    // kernel and the ragged tail of fewer than 32 positions to the streamed (or generic) kernel, which
    // continues in place from the statistics and states the head has written.
    const int Lh = L - L % 32;
    if (h_out && Lh > 0 && Lh < L && !pad_mask && (const void*)count_out != (const void*)prev_count) {
      StreamArgs head = sa;
      head.L = Lh;
      if (mma_cl_try(dtype, x, y, xn_out, xsb, xsl, xsd, ysb, ysl, ysd, true, head, (cudaStream_t)stream)) {
        const size_t es = (size_t)elem_size(dtype);
        const void* xt = (const char*)x + (size_t)Lh * xsl * es;
        void* yt = (char*)y + (size_t)Lh * ysl * es;
        void* nt = xn_out ? (char*)xn_out + (size_t)Lh * ysl * es : nullptr;
        StreamArgs tail = sa;
        tail.L = L - Lh;
        tail.count_offset = Lh;
        tail.prev_mean = mean_out; tail.prev_var = var_out; tail.h_in = h_out;
        if (stream_cl_try(dtype, xt, yt, nt, xsb, xsl, xsd, ysb, ysl, ysd, true, true, tail, (cudaStream_t)stream))
          return check_launch("tsn_ema_fwd(mma head + stream tail)");
        a.x = xt; a.y = yt; a.xn = nt; a.L = L - Lh; a.count_offset = Lh;
        a.prev_mean = mean_out; a.prev_var = var_out; a.h_in = h_out;
        const int npt = next_pow2_ndim(N);
        const unsigned gridt = (unsigned)(((long long)B * D + 127) / 128);
        MEGA_DISPATCH_DTYPE(dtype, MEGA_DISPATCH_NP(npt, launch(tsn_ema_rows_kernel<T, NP, true>, gridt, 128, 0,
                                                                stream, a)));
        return check_launch("tsn_ema_fwd(mma head + generic tail)");
      }
    }
    // (the tensor-core kernel writes the normalised activations too when xn_out is given)
    if (mma_cl_try(dtype, x, y, xn_out, xsb, xsl, xsd, ysb, ysl, ysd, true, sa, (cudaStream_t)stream))
      return check_launch("tsn_ema_fwd(mma)");
    if (stream_cl_try(dtype, x, y, xn_out, xsb, xsl, xsd, ysb, ysl, ysd, true, true, sa, (cudaStream_t)stream))
      return check_launch("tsn_ema_fwd(stream)");
  }
  const int np = next_pow2_ndim(N);
  const unsigned grid = (unsigned)(((long long)B * D + 127) / 128);
  const bool state = h_in || h_out;
  MEGA_DISPATCH_DTYPE(dtype, MEGA_DISPATCH_NP(np, {
    if (state) launch(tsn_ema_rows_kernel<T, NP, true>, grid, 128, 0, stream, a);
    else launch(tsn_ema_rows_kernel<T, NP, false>, grid, 128, 0, stream, a);
  }));
  return check_launch("tsn_ema_fwd");
}
