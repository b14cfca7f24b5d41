// Backward kernels of the EMA layer, TimestepNorm and SequenceNorm.
//
// EMA.  Forward: h_t = q h_{t-1} + p x~_t, y_t = sum_n g_n h_{n,t} + omega x_t (x~ = x zeroed at
// pads).  The input gradient is the time-reversed scan lambda_t = g dy_t + q lambda_{t+1},
// dx~_t = sum_n p_n lambda_{n,t}.  The parameter gradients are accumulated forward in time from the
// state sensitivities s = dh/dq (s_t = q s_{t-1} + h_{t-1}) and r = dh/dp (r_t = q r_{t-1} + x~_t):
//   dg_n = sum_t dy_t h_{n,t},  dp_n = g_n sum_t dy_t r_{n,t},  dq_n = g_n sum_t dy_t s_{n,t},
// so no state history is stored.  The anti-causal half of a bidirectional layer is the same
// computation on the reversed sequence, delayed by one step when the kernel is shifted.
// Four lanes share a (batch, channel) row and split its poles; sums over the batch are atomic adds.
#include "common.cuh"
#include "stream_bwd.cuh"

namespace mega {

struct EmaBwdArgs {
  const void* dy;
  const void* x;
  void* dx;
  int B, D, L, N;
  long long gsb, gsd, gsl, xsb, xsd, xsl, dsb, dsd, dsl;
  const float *p, *q, *g, *omega;
  const unsigned char* mask;
  const float *h_in, *dh_out;
  float *dp, *dq, *dg, *domega, *dh_in;
  int bidir, shift;
  int ksize;  // kTrunc: support of the truncated kernel (taps 0 .. ksize - 1)
};

// kMask: whether a padding mask is given (a run-time pointer test inside the unrolled load
// batches would serialise their loads).
// kTrunc: the kernel is cut after ksize taps.  The states then are sliding-window sums: with
// Q = q^ksize the sample leaving the window is taken out again,
//   h_t = q h_{t-1} + p (x~_t - Q x~_{t-ksize}),   r_t = q r_{t-1} + x~_t - Q x~_{t-ksize},
//   s_t = q s_{t-1} + h_{t-1} - p ksize q^(ksize-1) x~_{t-ksize},
//   lambda_t = q lambda_{t+1} + g (dy_t - Q dy_{t+ksize}).
template <typename T, int NP, bool kMask, bool kTrunc>
__global__ void __launch_bounds__(128) ema_bwd_kernel(EmaBwdArgs a) {
  constexpr int U = 8;
  const int sub = threadIdx.x & 3;
  const long long row = (long long)blockIdx.x * 32 + (threadIdx.x >> 2);
  const bool live = row < (long long)a.B * a.D;  // dead rows keep running for the shuffles
  const int d = live ? (int)(row % a.D) : 0;
  const int b = live ? (int)(row / a.D) : 0;
  const int L = a.L;
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  const T* gp = reinterpret_cast<const T*>(a.dy) + b * a.gsb + d * a.gsd;
  T* dxp = reinterpret_cast<T*>(a.dx) + b * a.dsb + d * a.dsd;
  const unsigned char* mp = kMask ? a.mask + (size_t)b * L : nullptr;
  const float om = __ldg(a.omega + d);
  float aw = 0.f;

  for (int half = 0; half < (a.bidir ? 2 : 1); ++half) {
    const bool rev = half == 1;
    const bool shift = rev && a.shift;
    const size_t prow = (size_t)(d + half * a.D) * a.N;
    const size_t srow = ((size_t)b * a.D + d) * a.N;
    float pp[NP], qq[NP], gg[NP], h[NP], s[NP], r[NP], ag[NP], aq[NP], ap[NP];
    float qw[kTrunc ? NP : 1], tq[kTrunc ? NP : 1];  // q^ksize, p ksize q^(ksize-1)
#pragma unroll
    for (int k = 0; k < NP; ++k) {
      const int n = k * 4 + sub;
      const bool ok = n < a.N;
      pp[k] = ok ? __ldg(a.p + prow + n) : 0.f;
      qq[k] = ok ? __ldg(a.q + prow + n) : 0.f;
      gg[k] = ok ? __ldg(a.g + prow + n) : 0.f;
      if (kTrunc) {
        const float qm1 = qq[k] > 0.f ? expf((float)(a.ksize - 1) * logf(qq[k])) : 0.f;
        qw[k] = qm1 * qq[k];
        tq[k] = pp[k] * (float)a.ksize * qm1;
      }
      h[k] = (ok && live && half == 0 && a.h_in) ? __ldg(a.h_in + srow + n) : 0.f;
      s[k] = r[k] = ag[k] = aq[k] = ap[k] = 0.f;
    }
    // ---- forward in (possibly reversed) time: states, sensitivities, parameter sums -------
    for (int u0 = 0; u0 < L; u0 += U) {
      float xv[U], gv[U], xd[kTrunc ? U : 1];
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int u = u0 + j;
        xv[j] = gv[j] = 0.f;
        if (kTrunc) xd[j] = 0.f;
        if (u < L && live) {
          const int t = rev ? L - 1 - u : u;
          const float xt = Elem<T>::ld(xp + t * a.xsl);
          gv[j] = Elem<T>::ld(gp + t * a.gsl);
          if (half == 0) aw = fmaf(gv[j], xt, aw);
          xv[j] = (kMask && __ldg(mp + t) != 0) ? 0.f : xt;
          if (kTrunc && u >= a.ksize) {  // the sample leaving the window
            const int td = rev ? t + a.ksize : t - a.ksize;
            if (!(kMask && __ldg(mp + td) != 0)) xd[j] = Elem<T>::ld(xp + td * a.xsl);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < U; ++j) {
        if (u0 + j < L) {
#pragma unroll
          for (int k = 0; k < NP; ++k) {
            if (shift) {
              ag[k] = fmaf(gv[j], h[k], ag[k]);
              aq[k] = fmaf(gv[j], s[k], aq[k]);
              ap[k] = fmaf(gv[j], r[k], ap[k]);
            }
            if (kTrunc) {
              const float xin = fmaf(-qw[k], xd[j], xv[j]);
              s[k] = fmaf(qq[k], s[k], fmaf(-tq[k], xd[j], h[k]));
              h[k] = fmaf(qq[k], h[k], pp[k] * xin);
              r[k] = fmaf(qq[k], r[k], xin);
            } else {
              s[k] = fmaf(qq[k], s[k], h[k]);
              h[k] = fmaf(qq[k], h[k], pp[k] * xv[j]);
              r[k] = fmaf(qq[k], r[k], xv[j]);
            }
            if (!shift) {
              ag[k] = fmaf(gv[j], h[k], ag[k]);
              aq[k] = fmaf(gv[j], s[k], aq[k]);
              ap[k] = fmaf(gv[j], r[k], ap[k]);
            }
          }
        }
      }
    }
    float lam[NP];
#pragma unroll
    for (int k = 0; k < NP; ++k) {
      const int n = k * 4 + sub;
      const bool ok = n < a.N && live;
      const float dh = (ok && half == 0 && a.dh_out) ? __ldg(a.dh_out + srow + n) : 0.f;
      lam[k] = dh;
      if (ok) {
        atomicAdd(a.dg + prow + n, ag[k]);
        atomicAdd(a.dp + prow + n, fmaf(gg[k], ap[k], dh * r[k]));
        atomicAdd(a.dq + prow + n, fmaf(gg[k], aq[k], dh * s[k]));
      }
    }
    // ---- backward in time: input gradient ---------------------------------------------------
    for (int u0 = L - 1; u0 >= 0; u0 -= U) {
      float gv[U], old[U], gd[kTrunc ? U : 1];
      bool mk[U];
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int u = u0 - j;
        gv[j] = old[j] = 0.f;
        if (kTrunc) gd[j] = 0.f;
        mk[j] = false;
        if (u >= 0 && live) {
          const int t = rev ? L - 1 - u : u;
          gv[j] = Elem<T>::ld(gp + t * a.gsl);
          if (kTrunc && u + a.ksize < L) gd[j] = Elem<T>::ld(gp + (rev ? t - a.ksize : t + a.ksize) * a.gsl);
          mk[j] = kMask && __ldg(mp + t) != 0;
          if (half == 1 && sub == 0) old[j] = Elem<T>::ld_shared(dxp + t * a.dsl);  // plain load: written above
        }
      }
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int u = u0 - j;
        if (u >= 0) {
          float part = 0.f;
#pragma unroll
          for (int k = 0; k < NP; ++k) {
            const float gin = kTrunc ? fmaf(-qw[k], gd[j], gv[j]) : gv[j];
            if (shift) {
              part = fmaf(pp[k], lam[k], part);
              lam[k] = fmaf(qq[k], lam[k], gg[k] * gin);
            } else {
              const float l = fmaf(gg[k], gin, lam[k]);
              part = fmaf(pp[k], l, part);
              lam[k] = qq[k] * l;
            }
          }
          part += __shfl_xor_sync(0xffffffffu, part, 1);
          part += __shfl_xor_sync(0xffffffffu, part, 2);
          if (live && sub == 0) {
            const int t = rev ? L - 1 - u : u;
            const float v = mk[j] ? 0.f : part;
            Elem<T>::st(dxp + t * a.dsl, half == 0 ? fmaf(om, gv[j], v) : old[j] + v);
          }
        }
      }
    }
    if (half == 0 && a.dh_in && live) {
#pragma unroll
      for (int k = 0; k < NP; ++k) {
        const int n = k * 4 + sub;
        if (n < a.N) a.dh_in[srow + n] = lam[k];
      }
    }
  }
  if (live && sub == 0) atomicAdd(a.domega + d, aw);  // every lane of a row holds the same sum
}

// Chain rule from (p, q, gamma_hat) to the raw parameters:
// p = sigmoid(alpha) beta, q = 1 - sigmoid(alpha) sigmoid(delta), gamma_hat = gamma / sqrt(N).
__global__ void ema_coeffs_bwd_kernel(const float* alpha, const float* delta, const float* beta,
                                      const float* dp, const float* dq, const float* dgh, float* dalpha,
                                      float* ddelta, float* dbeta, float* dgamma, int total, float scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float sa = 1.f / (1.f + __expf(-alpha[i])), sd = 1.f / (1.f + __expf(-delta[i]));
  const float dsa = sa * (1.f - sa), dsd = sd * (1.f - sd);
  dalpha[i] = dp[i] * beta[i] * dsa - dq[i] * sd * dsa;
  ddelta[i] = -dq[i] * sa * dsd;
  dbeta[i] = dp[i] * sa;
  dgamma[i] = dgh[i] * scale;
}

// ---------------------------------------------------------------------------------------------
// TimestepNorm backward (fairseq/csrc/ops/timestep_norm.cc:105-216 plain, :318-446 grouped): a scan
// backward in time carrying the gradients of the running mean and variance.
// ---------------------------------------------------------------------------------------------
struct TsnBwdArgs {
  const void *dy, *x;
  void* dx;
  int B, L, D, G;
  long long gsb, gsl, gsd, xsb, xsl, xsd, dsb, dsl, dsd;
  const float *dmean, *dvar;  // (B, G) or NULL
  const float* prev_mean;     // (B, G)
  const long long* count;     // (B) final counts
  const float *cummean, *cumrstd, *group_mean;  // (B, L, G)
  const float* gamma;
  const unsigned char* mask;
  float *dprev_mean, *dprev_var;  // (B, G)
  float *dgamma, *dbeta;          // (D) accumulators
};

template <typename T, bool kMask>
__global__ void __launch_bounds__(128) tsn_bwd_plain_kernel(TsnBwdArgs a) {
  constexpr int U = 16;  // loads in flight per thread
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)a.B * a.D) return;
  const int d = (int)(gid % a.D);
  const int b = (int)(gid / a.D);
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  const T* gp = reinterpret_cast<const T*>(a.dy) + b * a.gsb + d * a.gsd;
  T* dxp = reinterpret_cast<T*>(a.dx) + b * a.dsb + d * a.dsd;
  const float* cm = a.cummean + (size_t)b * a.L * a.D + d;
  const float* cr = a.cumrstd + (size_t)b * a.L * a.D + d;
  const unsigned char* mp = kMask ? a.mask + (size_t)b * a.L : nullptr;
  const float w = __ldg(a.gamma + d);
  const float pm = a.prev_mean[gid];
  long long cnt = a.count[b];
  float ug = a.dmean ? a.dmean[gid] : 0.f, vg = a.dvar ? a.dvar[gid] : 0.f;
  float wg = 0.f, bg = 0.f;
  for (int t0 = a.L - 1; t0 >= 0; t0 -= U) {
    float xv[U], gv[U], uv[U], pv[U], rv[U];
    bool mk[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int t = t0 - j;
      xv[j] = gv[j] = uv[j] = pv[j] = rv[j] = 0.f;
      mk[j] = true;
      if (t >= 0) {
        mk[j] = kMask && __ldg(mp + t) != 0;
        xv[j] = Elem<T>::ld(xp + t * a.xsl);
        gv[j] = Elem<T>::ld(gp + t * a.gsl);
        uv[j] = __ldg(cm + (size_t)t * a.D);
        rv[j] = __ldg(cr + (size_t)t * a.D);
        pv[j] = t > 0 ? __ldg(cm + (size_t)(t - 1) * a.D) : pm;
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int t = t0 - j;
      if (t < 0) break;
      if (mk[j]) {
        Elem<T>::st(dxp + t * a.dsl, 0.f);
        continue;
      }
      const float coef = 1.f / (float)cnt;
      --cnt;
      const float dy = gv[j], x = xv[j], u = uv[j], r = rv[j];
      const float dyr = dy * r, delta = x - u, xp_ = x - pv[j];
      const float dv = vg - 0.5f * dy * w * delta * (r * r * r);
      const float du = ug - (w * dyr + coef * dv * xp_);
      Elem<T>::st(dxp + t * a.dsl, w * dyr + dv * coef * (delta + xp_) + coef * du);
      ug = (1.f - coef) * du - coef * delta * dv;
      vg = (1.f - coef) * dv;
      wg = fmaf(dyr, delta, wg);
      bg += dy;
    }
  }
  a.dprev_mean[gid] = ug;
  a.dprev_var[gid] = vg;
  atomicAdd(a.dgamma + d, wg);
  atomicAdd(a.dbeta + d, bg);
}

// Grouped: one warp per (batch, group); a lane owns features lane, lane + 32, ... of the group
// (at most kGF of them).
constexpr int kGF = 8;
template <typename T>
__global__ void __launch_bounds__(128) tsn_bwd_group_kernel(TsnBwdArgs a) {
  const int lane = threadIdx.x & 31;
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (wid >= (long long)a.B * a.G) return;
  const int g = (int)(wid % a.G);
  const int b = (int)(wid / a.G);
  const int gs = a.D / a.G;
  const float cg = 1.f / (float)gs;
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + (long long)g * gs * a.xsd;
  const T* gp = reinterpret_cast<const T*>(a.dy) + b * a.gsb + (long long)g * gs * a.gsd;
  T* dxp = reinterpret_cast<T*>(a.dx) + b * a.dsb + (long long)g * gs * a.dsd;
  const size_t sbase = (size_t)b * a.L * a.G + g;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  float w[kGF], wg[kGF], bg[kGF];
#pragma unroll
  for (int k = 0; k < kGF; ++k) {
    const int f = lane + 32 * k;
    w[k] = f < gs ? __ldg(a.gamma + g * gs + f) : 0.f;
    wg[k] = bg[k] = 0.f;
  }
  long long cnt = a.count[b];
  float ug = a.dmean ? a.dmean[wid] : 0.f, vg = a.dvar ? a.dvar[wid] : 0.f;
  for (int t = a.L - 1; t >= 0; --t) {
    const bool mk = mp && mp[t];
    if (mk) {
#pragma unroll
      for (int k = 0; k < kGF; ++k) {
        const int f = lane + 32 * k;
        if (f < gs) Elem<T>::st(dxp + t * a.dsl + f * a.dsd, 0.f);
      }
      continue;
    }
    const float c1 = (float)(cnt - 1) / (float)cnt, c2 = 1.f / (float)cnt;
    --cnt;
    const float pu = t > 0 ? __ldg(a.cummean + sbase + (size_t)(t - 1) * a.G) : a.prev_mean[wid];
    const float ux = __ldg(a.group_mean + sbase + (size_t)t * a.G);
    const float u = __ldg(a.cummean + sbase + (size_t)t * a.G);
    const float r = __ldg(a.cumrstd + sbase + (size_t)t * a.G);
    float xv[kGF], gv[kGF];
    float ds = 0.f, db = 0.f;
#pragma unroll
    for (int k = 0; k < kGF; ++k) {
      const int f = lane + 32 * k;
      xv[k] = gv[k] = 0.f;
      if (f < gs) {
        xv[k] = Elem<T>::ld(xp + t * a.xsl + f * a.xsd);
        gv[k] = Elem<T>::ld(gp + t * a.gsl + f * a.gsd);
      }
      ds = fmaf(gv[k] * (xv[k] - u), w[k], ds);
      db = fmaf(gv[k], w[k], db);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ds += __shfl_xor_sync(0xffffffffu, ds, o);
      db += __shfl_xor_sync(0xffffffffu, db, o);
    }
    const float du = ug - r * db;
    const float dv = vg - 0.5f * (r * r * r) * ds;
    const float dux = c2 * du + 2.f * c1 * c2 * dv * (ux - pu);
    const float dvx = c2 * dv;
#pragma unroll
    for (int k = 0; k < kGF; ++k) {
      const int f = lane + 32 * k;
      if (f < gs) {
        Elem<T>::st(dxp + t * a.dsl + f * a.dsd,
                    gv[k] * r * w[k] + dux * cg + 2.f * dvx * cg * (xv[k] - ux));
        wg[k] = fmaf(gv[k] * (xv[k] - u), r, wg[k]);
        bg[k] += gv[k];
      }
    }
    ug = c1 * du - 2.f * c1 * c2 * dv * (ux - pu);
    vg = c1 * dv;
  }
  if (lane == 0) {
    a.dprev_mean[wid] = ug;
    a.dprev_var[wid] = vg;
  }
#pragma unroll
  for (int k = 0; k < kGF; ++k) {
    const int f = lane + 32 * k;
    if (f < gs) {
      atomicAdd(a.dgamma + g * gs + f, wg[k]);
      atomicAdd(a.dbeta + g * gs + f, bg[k]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// SequenceNorm backward, one statistic per (batch, channel)
// (fairseq/csrc/ops/sequence_norm.cc:374-529).  One CTA per (b, channel) row: masked sums of
// dy and dy * x over the length, then the input gradient.
// ---------------------------------------------------------------------------------------------
struct SqnBwdArgs {
  const void *dy, *x;
  void* dx;
  int B, D, L;
  long long gsb, gsd, gsl, xsb, xsd, xsl, dsb, dsd, dsl;
  const long long* count;  // (B)
  const float *mean, *rstd;  // (B, D)
  const float* gamma;
  const unsigned char* mask;
  float *dgamma, *dbeta;  // (D) accumulators
};

template <typename T>
__global__ void __launch_bounds__(256) sqn_bwd_kernel(SqnBwdArgs a) {
  __shared__ float red[2][8];
  const int row = blockIdx.x;
  const int d = row % a.D, b = row / a.D;
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  const T* gp = reinterpret_cast<const T*>(a.dy) + b * a.gsb + d * a.gsd;
  T* dxp = reinterpret_cast<T*>(a.dx) + b * a.dsb + d * a.dsd;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  float ds = 0.f, db = 0.f;
  for (int t = threadIdx.x; t < a.L; t += blockDim.x) {
    if (mp && mp[t]) continue;
    const float dy = Elem<T>::ld(gp + t * a.gsl);
    ds = fmaf(dy, Elem<T>::ld(xp + t * a.xsl), ds);
    db += dy;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ds += __shfl_xor_sync(0xffffffffu, ds, o);
    db += __shfl_xor_sync(0xffffffffu, db, o);
  }
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = ds;
    red[1][threadIdx.x >> 5] = db;
  }
  __syncthreads();
  ds = db = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    ds += red[0][k];
    db += red[1][k];
  }
  const float u = a.mean[row], r = a.rstd[row], w = __ldg(a.gamma + d);
  const long long cnt = a.count[b];
  const float coef = cnt > 0 ? 1.f / (float)cnt : 0.f;
  const float dv = 0.5f * (r * r * r) * w * (u * db - ds);
  const float du = -r * w * db;
  for (int t = threadIdx.x; t < a.L; t += blockDim.x) {
    float out = 0.f;
    if (!(mp && mp[t])) {
      const float dy = Elem<T>::ld(gp + t * a.gsl), x = Elem<T>::ld(xp + t * a.xsl);
      out = r * w * dy + 2.f * coef * (x - u) * dv + coef * du;
    }
    Elem<T>::st(dxp + t * a.dsl, out);
  }
  if (threadIdx.x == 0) {
    atomicAdd(a.dgamma + d, r * (ds - u * db));
    atomicAdd(a.dbeta + d, db);
  }
}

// Grouped SequenceNorm backward (fairseq/csrc/ops/sequence_norm.cc:657-860): statistics are shared by
// the D / G channels of a group.  One CTA per (batch, group): per-channel masked sums of dy and
// dy * x (kept for dgamma / dbeta), combined with the scale into the group's sums, then dx.
struct SqnGroupBwdArgs {
  SqnBwdArgs base;
  int G;
};

template <typename T>
__global__ void __launch_bounds__(256) sqn_bwd_group_kernel(SqnGroupBwdArgs ga) {
  extern __shared__ float chan[];  // [2][gs]: ds, db per channel of the group
  __shared__ float red[2][8];
  const SqnBwdArgs& a = ga.base;
  const int gs = a.D / ga.G;
  const int g = blockIdx.x % ga.G, b = blockIdx.x / ga.G;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  float dsw = 0.f, dbw = 0.f;  // meaningful in thread 0
  for (int k = 0; k < gs; ++k) {
    const int d = g * gs + k;
    const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
    const T* gp = reinterpret_cast<const T*>(a.dy) + b * a.gsb + d * a.gsd;
    float ds = 0.f, db = 0.f;
    for (int t = threadIdx.x; t < a.L; t += blockDim.x) {
      if (mp && mp[t]) continue;
      const float dy = Elem<T>::ld(gp + t * a.gsl);
      ds = fmaf(dy, Elem<T>::ld(xp + t * a.xsl), ds);
      db += dy;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ds += __shfl_xor_sync(0xffffffffu, ds, o);
      db += __shfl_xor_sync(0xffffffffu, db, o);
    }
    if ((threadIdx.x & 31) == 0) {
      red[0][threadIdx.x >> 5] = ds;
      red[1][threadIdx.x >> 5] = db;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      ds = db = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        ds += red[0][w];
        db += red[1][w];
      }
      chan[k] = ds;
      chan[gs + k] = db;
      const float w = __ldg(a.gamma + d);
      dsw = fmaf(ds, w, dsw);
      dbw = fmaf(db, w, dbw);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    red[0][0] = dsw;
    red[1][0] = dbw;
  }
  __syncthreads();
  dsw = red[0][0];
  dbw = red[1][0];
  const float u = a.mean[blockIdx.x], r = a.rstd[blockIdx.x];
  const long long cnt = a.count[b];
  const float coef = cnt > 0 ? 1.f / ((float)cnt * (float)gs) : 0.f;
  const float dv = 0.5f * (r * r * r) * (u * dbw - dsw);
  const float du = -r * dbw;
  for (int k = 0; k < gs; ++k) {
    const int d = g * gs + k;
    const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
    const T* gp = reinterpret_cast<const T*>(a.dy) + b * a.gsb + d * a.gsd;
    T* dxp = reinterpret_cast<T*>(a.dx) + b * a.dsb + d * a.dsd;
    const float w = __ldg(a.gamma + d);
    for (int t = threadIdx.x; t < a.L; t += blockDim.x) {
      float out = 0.f;
      if (!(mp && mp[t])) {
        const float dy = Elem<T>::ld(gp + t * a.gsl), x = Elem<T>::ld(xp + t * a.xsl);
        out = r * w * dy + 2.f * coef * (x - u) * dv + coef * du;
      }
      Elem<T>::st(dxp + t * a.dsl, out);
    }
  }
  for (int k = threadIdx.x; k < gs; k += blockDim.x) {
    atomicAdd(a.dgamma + g * gs + k, r * (chan[k] - u * chan[gs + k]));
    atomicAdd(a.dbeta + g * gs + k, chan[gs + k]);
  }
}

}  // namespace mega

using namespace mega;

extern "C" int mega_ema_bwd(const void* dy, const void* x, void* dx, int dtype, int B, int D, int L, int64_t gsb,
                            int64_t gsd, int64_t gsl, int64_t xsb, int64_t xsd, int64_t xsl, int64_t dsb,
                            int64_t dsd, int64_t dsl, const float* p, const float* q, const float* gamma_hat,
                            const float* omega, int N, const uint8_t* pad_mask, const float* h_in,
                            const float* dh_out, unsigned flags, int truncation, float* dp, float* dq,
                            float* dgamma_hat, float* domega, float* dh_in, mega_stream_t stream) {
  if (!dy || !x || !dx || !p || !q || !gamma_hat || !omega || !dp || !dq || !dgamma_hat || !domega)
    return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || D <= 0 || L <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  const bool bidir = (flags & MEGA_EMA_BIDIRECTIONAL) != 0;
  if (flags & MEGA_EMA_SILU) return MEGA_ERR_UNSUPPORTED;  // differentiate the activation outside
  const bool trunc = truncation > 0 && truncation < L;
  if (trunc && !bidir) return MEGA_ERR_UNSUPPORTED;  // as the forward: one direction is never truncated
  if (bidir && (h_in || dh_out || dh_in)) return MEGA_ERR_UNSUPPORTED;
  const size_t es = elem_size(dtype);
  if (!aligned_to(dy, es) || !aligned_to(x, es) || !aligned_to(dx, es)) return MEGA_ERR_ALIGN;
  const size_t K = (size_t)(bidir ? 2 : 1) * D;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(dp, 0, K * N * sizeof(float), s) != cudaSuccess ||
      cudaMemsetAsync(dq, 0, K * N * sizeof(float), s) != cudaSuccess ||
      cudaMemsetAsync(dgamma_hat, 0, K * N * sizeof(float), s) != cudaSuccess ||
      cudaMemsetAsync(domega, 0, (size_t)D * sizeof(float), s) != cudaSuccess)
    return check_launch("ema_bwd(memset)");
  if (!bidir) {  // channel-contiguous activations: the streamed TMA kernel
    EmaBwdStreamArgs sa{};
    sa.B = B; sa.L = L; sa.D = D; sa.N = N;
    sa.p = p; sa.q = q; sa.g = gamma_hat; sa.omega = omega; sa.mask = pad_mask; sa.h_in = h_in; sa.dh_out = dh_out;
    sa.dp = dp; sa.dq = dq; sa.dg = dgamma_hat; sa.domega = domega; sa.dh_in = dh_in;
    if (ema_bwd_stream_try(dtype, dy, x, dx, gsb, gsl, gsd, xsb, xsl, xsd, dsb, dsl, dsd, sa, s))
      return check_launch("ema_bwd(stream)");
  }
  EmaBwdArgs a{};
  a.dy = dy; a.x = x; a.dx = dx; a.B = B; a.D = D; a.L = L; a.N = N;
  a.gsb = gsb; a.gsd = gsd; a.gsl = gsl; a.xsb = xsb; a.xsd = xsd; a.xsl = xsl;
  a.dsb = dsb; a.dsd = dsd; a.dsl = dsl;
  a.p = p; a.q = q; a.g = gamma_hat; a.omega = omega; a.mask = pad_mask; a.h_in = h_in; a.dh_out = dh_out;
  a.dp = dp; a.dq = dq; a.dg = dgamma_hat; a.domega = domega; a.dh_in = dh_in;
  a.bidir = bidir ? 1 : 0;
  a.shift = (flags & MEGA_EMA_NO_SHIFT) ? 0 : 1;
  a.ksize = trunc ? truncation : L;
  const unsigned grid = (unsigned)(((long long)B * D + 31) / 32);
  const int np = N <= 4 ? 1 : N <= 8 ? 2 : N <= 16 ? 4 : 8;
#define MEGA_EMA_BWD(NPV)                                                                 \
  if (trunc) {                                                                            \
    if (pad_mask) launch(ema_bwd_kernel<T, NPV, true, true>, grid, 128, 0, stream, a);     \
    else launch(ema_bwd_kernel<T, NPV, false, true>, grid, 128, 0, stream, a);             \
  } else if (pad_mask) launch(ema_bwd_kernel<T, NPV, true, false>, grid, 128, 0, stream, a); \
  else launch(ema_bwd_kernel<T, NPV, false, false>, grid, 128, 0, stream, a)
  MEGA_DISPATCH_DTYPE(dtype, {
    if (np == 1) { MEGA_EMA_BWD(1); }
    else if (np == 2) { MEGA_EMA_BWD(2); }
    else if (np == 4) { MEGA_EMA_BWD(4); }
    else { MEGA_EMA_BWD(8); }
  });
#undef MEGA_EMA_BWD
  return check_launch("ema_bwd");
}

extern "C" int mega_ema_coeffs_bwd(const float* alpha, const float* delta, const float* beta, const float* dp,
                                   const float* dq, const float* dgamma_hat, int K, int N, float* dalpha,
                                   float* ddelta, float* dbeta, float* dgamma, mega_stream_t stream) {
  if (!alpha || !delta || !beta || !dp || !dq || !dgamma_hat || !dalpha || !ddelta || !dbeta || !dgamma)
    return MEGA_ERR_NULL;
  if (K <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  const int total = K * N;
  launch(ema_coeffs_bwd_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, alpha, delta, beta, dp, dq,
         dgamma_hat, dalpha, ddelta, dbeta, dgamma, total, rsqrtf((float)N));
  return check_launch("ema_coeffs_bwd");
}

extern "C" int mega_timestep_norm_bwd(const void* dy, const void* x, void* dx, int dtype, int B, int L, int D,
                                      int64_t gsb, int64_t gsl, int64_t gsd, int64_t xsb, int64_t xsl,
                                      int64_t xsd, int64_t dsb, int64_t dsl, int64_t dsd, const float* dmean,
                                      const float* dvar, const float* prev_mean, const int64_t* count,
                                      const float* cummean, const float* cumrstd, const float* group_mean,
                                      const float* gamma, const uint8_t* pad_mask, int num_groups,
                                      float* dprev_mean, float* dprev_var, float* dgamma, float* dbeta,
                                      mega_stream_t stream) {
  if (!dy || !x || !dx || !prev_mean || !count || !cummean || !cumrstd || !gamma || !dprev_mean || !dprev_var ||
      !dgamma || !dbeta)
    return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || L <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  const int G = (num_groups <= 0 || num_groups == D) ? D : num_groups;
  if (D % G != 0) return MEGA_ERR_SHAPE;
  if (G != D && !group_mean) return MEGA_ERR_NULL;
  if (G != D && D / G > 32 * kGF) return MEGA_ERR_UNSUPPORTED;
  const size_t es = elem_size(dtype);
  if (!aligned_to(dy, es) || !aligned_to(x, es) || !aligned_to(dx, es)) return MEGA_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(dgamma, 0, (size_t)D * sizeof(float), s) != cudaSuccess ||
      cudaMemsetAsync(dbeta, 0, (size_t)D * sizeof(float), s) != cudaSuccess)
    return check_launch("timestep_norm_bwd(memset)");
  TsnBwdArgs a{};
  a.dy = dy; a.x = x; a.dx = dx; a.B = B; a.L = L; a.D = D; a.G = G;
  a.gsb = gsb; a.gsl = gsl; a.gsd = gsd; a.xsb = xsb; a.xsl = xsl; a.xsd = xsd;
  a.dsb = dsb; a.dsl = dsl; a.dsd = dsd;
  a.dmean = dmean; a.dvar = dvar; a.prev_mean = prev_mean; a.count = (const long long*)count;
  a.cummean = cummean; a.cumrstd = cumrstd; a.group_mean = group_mean; a.gamma = gamma; a.mask = pad_mask;
  a.dprev_mean = dprev_mean; a.dprev_var = dprev_var; a.dgamma = dgamma; a.dbeta = dbeta;
  if (G == D) {
    TsnBwdStreamArgs sa{};
    sa.B = B; sa.L = L; sa.D = D; sa.dmean = dmean; sa.dvar = dvar; sa.prev_mean = prev_mean;
    sa.count = (const long long*)count; sa.gamma = gamma; sa.mask = pad_mask;
    sa.dprev_mean = dprev_mean; sa.dprev_var = dprev_var; sa.dgamma = dgamma; sa.dbeta = dbeta;
    if (tsn_bwd_stream_try(dtype, dy, x, dx, gsb, gsl, gsd, xsb, xsl, xsd, dsb, dsl, dsd, cummean, cumrstd, sa, s))
      return check_launch("timestep_norm_bwd(stream)");
    const unsigned grid = (unsigned)(((long long)B * D + 127) / 128);
    MEGA_DISPATCH_DTYPE(dtype, {
      if (pad_mask) launch(tsn_bwd_plain_kernel<T, true>, grid, 128, 0, stream, a);
      else launch(tsn_bwd_plain_kernel<T, false>, grid, 128, 0, stream, a);
    });
  } else {
    GroupStreamBwdArgs ga{};
    ga.B = B; ga.L = L; ga.D = D; ga.G = G; ga.dmean = dmean; ga.dvar = dvar; ga.prev_mean = prev_mean;
    ga.count = (const long long*)count; ga.cummean = cummean; ga.cumrstd = cumrstd; ga.group_mean = group_mean;
    ga.gamma = gamma; ga.mask = pad_mask;
    ga.dprev_mean = dprev_mean; ga.dprev_var = dprev_var; ga.dgamma = dgamma; ga.dbeta = dbeta;
    if (tsn_group_bwd_stream_try(dtype, dy, x, dx, gsb, gsl, gsd, xsb, xsl, xsd, dsb, dsl, dsd, ga, s))
      return check_launch("timestep_norm_bwd(group stream)");
    const unsigned grid = (unsigned)(((long long)B * G * 32 + 127) / 128);
    MEGA_DISPATCH_DTYPE(dtype, launch(tsn_bwd_group_kernel<T>, grid, 128, 0, stream, a));
  }
  return check_launch("timestep_norm_bwd");
}

extern "C" int mega_sequence_norm_bwd(const void* dy, const void* x, void* dx, int dtype, int B, int D, int L,
                                      int64_t gsb, int64_t gsd, int64_t gsl, int64_t xsb, int64_t xsd,
                                      int64_t xsl, int64_t dsb, int64_t dsd, int64_t dsl, const int64_t* count,
                                      const float* mean, const float* rstd, const float* gamma,
                                      const uint8_t* pad_mask, int num_groups, float* dgamma, float* dbeta,
                                      mega_stream_t stream) {
  if (!dy || !x || !dx || !count || !mean || !rstd || !gamma || !dgamma || !dbeta) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || L <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  const int G = (num_groups <= 0 || num_groups == D) ? D : num_groups;
  if (D % G != 0) return MEGA_ERR_SHAPE;
  const size_t es = elem_size(dtype);
  if (!aligned_to(dy, es) || !aligned_to(x, es) || !aligned_to(dx, es)) return MEGA_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(dgamma, 0, (size_t)D * sizeof(float), s) != cudaSuccess ||
      cudaMemsetAsync(dbeta, 0, (size_t)D * sizeof(float), s) != cudaSuccess)
    return check_launch("sequence_norm_bwd(memset)");
  SqnBwdArgs a{};
  a.dy = dy; a.x = x; a.dx = dx; a.B = B; a.D = D; a.L = L;
  a.gsb = gsb; a.gsd = gsd; a.gsl = gsl; a.xsb = xsb; a.xsd = xsd; a.xsl = xsl;
  a.dsb = dsb; a.dsd = dsd; a.dsl = dsl;
  a.count = (const long long*)count; a.mean = mean; a.rstd = rstd; a.gamma = gamma; a.mask = pad_mask;
  a.dgamma = dgamma; a.dbeta = dbeta;
  if (G != D) {
    SqnGroupBwdArgs ga{a, G};
    const size_t smem = (size_t)(D / G) * 2 * sizeof(float);
    if (smem > 48 * 1024) return MEGA_ERR_UNSUPPORTED;  // more than 6144 channels per group
    MEGA_DISPATCH_DTYPE(dtype, launch(sqn_bwd_group_kernel<T>, (unsigned)((long long)B * G), 256, smem, stream, ga));
    return check_launch("sequence_norm_bwd(group)");
  }
  MEGA_DISPATCH_DTYPE(dtype, launch(sqn_bwd_kernel<T>, (unsigned)((long long)B * D), 256, 0, stream, a));
  return check_launch("sequence_norm_bwd");
}
