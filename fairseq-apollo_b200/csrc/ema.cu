// EMA layer kernels: coefficients, kernel/bias materialisation, the diagonal-recurrence
// scan (causal, bidirectional, truncated, with carried state) and the decode step.
//
// The convolution y = k * x with k[l] = sum_n p_n gamma_n q_n^l is evaluated as the
// order-N diagonal recurrence h_t = q h_{t-1} + p x_t, y_t = sum_n gamma_n h_{n,t}:
// O(L) work per row, no length cap, one pass over x.
#include <type_traits>

#include "common.cuh"
#include "stream_cl.cuh"
#include "rowres.cuh"

namespace mega {

// ---------------------------------------------------------------------------
// coefficients / kernel / bias
// ---------------------------------------------------------------------------
template <typename T>
__global__ void ema_coeffs_kernel(const T* __restrict__ alpha, const T* __restrict__ delta,
                                  const T* __restrict__ beta, const T* __restrict__ gamma, int total,
                                  float scale, float* __restrict__ p, float* __restrict__ q,
                                  float* __restrict__ g) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float a = 1.0f / (1.0f + expf(-Elem<T>::ld(alpha + i)));
  float d = 1.0f / (1.0f + expf(-Elem<T>::ld(delta + i)));
  p[i] = a * Elem<T>::ld(beta + i);
  q[i] = 1.0f - a * d;
  g[i] = Elem<T>::ld(gamma + i) * scale;
}

// k[r,l] = sum_n p g exp(l log q)
__global__ void ema_kernel_kernel(const float* __restrict__ p, const float* __restrict__ q,
                                  const float* __restrict__ g, int K, int N, int L,
                                  float* __restrict__ out) {
  extern __shared__ float sm[];  // c[N], logq[N]
  int r = blockIdx.y;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    sm[n] = p[r * N + n] * g[r * N + n];
    sm[N + n] = logf(q[r * N + n]);
  }
  __syncthreads();
  int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= L) return;
  float acc = 0.f;
  for (int n = 0; n < N; ++n) acc += sm[n] * expf((float)l * sm[N + n]);
  out[(size_t)r * L + l] = acc;
}

// bias[b,d,l] = sum_n g q^(l+1) h[b,d,n]
__global__ void ema_bias_kernel(const float* __restrict__ q, const float* __restrict__ g,
                                const float* __restrict__ h, int D, int N, int L,
                                float* __restrict__ out) {
  extern __shared__ float sm[];  // c[N], logq[N]
  int row = blockIdx.y;          // b*D + d
  int d = row % D;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    sm[n] = g[d * N + n] * h[(size_t)row * N + n];
    sm[N + n] = logf(q[d * N + n]);
  }
  __syncthreads();
  int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= L) return;
  float acc = 0.f;
  for (int n = 0; n < N; ++n) acc += sm[n] * expf((float)(l + 1) * sm[N + n]);
  out[(size_t)row * L + l] = acc;
}

// ---------------------------------------------------------------------------
// scan
// ---------------------------------------------------------------------------
struct EmaArgs {
  const void* x;
  void* y;
  int B, D, L, N;
  long long xsb, xsd, xsl, ysb, ysd, ysl;
  const float *p, *q, *g, *omega;
  const unsigned char* mask;
  const float* h_in;
  float* h_out;
  int ksize;       // effective kernel support (>= L: untruncated)
  int dir;         // +1 causal pass, -1 anti-causal pass
  int shift;       // anti-causal pass starts at lag 1
  int accumulate;  // add to y instead of writing conv + omega*x
  int silu;
  int row_off;     // 0, or D for the anti-causal coefficient rows
};

enum { MODE_FAST = 0, MODE_STATE = 1, MODE_TRUNC = 2 };

// Per-thread pole state.  MODE_FAST/MODE_TRUNC keep s = h / p so one FMA updates a pole;
// MODE_STATE keeps the true h (needed to import/export states when p may be 0).
template <int NP, int MODE>
struct Poles {
  float q[NP], c[NP], s[NP];
  float aux[MODE == MODE_FAST ? 1 : NP];  // MODE_STATE: p ; MODE_TRUNC: q^ksize

  __device__ __forceinline__ void init(const EmaArgs& a, int row, int b, int d) {
#pragma unroll
    for (int n = 0; n < NP; ++n) {
      float pn = 0.f, qn = 0.f, gn = 0.f;
      if (n < a.N) {
        pn = __ldg(a.p + (size_t)row * a.N + n);
        qn = __ldg(a.q + (size_t)row * a.N + n);
        gn = __ldg(a.g + (size_t)row * a.N + n);
      }
      q[n] = qn;
      if (MODE == MODE_STATE) {
        c[n] = gn;
        aux[n] = pn;
        s[n] = (a.h_in != nullptr && n < a.N) ? __ldg(a.h_in + ((size_t)b * a.D + d) * a.N + n) : 0.f;
      } else {
        c[n] = pn * gn;
        s[n] = 0.f;
        if (MODE == MODE_TRUNC) aux[n] = (qn > 0.f) ? expf((float)a.ksize * logf(qn)) : 0.f;
      }
    }
  }
  // advance with input xm (already masked), xd = delayed input leaving the window (MODE_TRUNC)
  __device__ __forceinline__ void update(float xm, float xd) {
#pragma unroll
    for (int n = 0; n < NP; ++n) {
      if (MODE == MODE_STATE) {
        s[n] = fmaf(q[n], s[n], aux[n] * xm);
      } else if (MODE == MODE_TRUNC) {
        s[n] = fmaf(q[n], s[n], fmaf(-aux[n], xd, xm));
      } else {
        s[n] = fmaf(q[n], s[n], xm);
      }
    }
  }
  __device__ __forceinline__ float output() const {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int n = 0; n < NP; n += 2) {
      a0 = fmaf(c[n], s[n], a0);
      a1 = fmaf(c[n + 1], s[n + 1], a1);
    }
    return a0 + a1;
  }
  __device__ __forceinline__ void export_state(const EmaArgs& a, int b, int d) const {
    if (MODE == MODE_STATE && a.h_out != nullptr) {
#pragma unroll
      for (int n = 0; n < NP; ++n)
        if (n < a.N) a.h_out[((size_t)b * a.D + d) * a.N + n] = s[n];
    }
  }
};

// One thread per (batch, channel) row, channel fastest: coalesced when the channel stride is 1.
template <typename T, int NP, int MODE>
__global__ void __launch_bounds__(128) ema_scan_rows_kernel(EmaArgs a) {
  long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)a.B * a.D) return;
  const int d = (int)(gid % a.D);
  const int b = (int)(gid / a.D);
  Poles<NP, MODE> st;
  st.init(a, d + a.row_off, b, d);
  const T* xp = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ysb + d * a.ysd;
  const unsigned char* mp = a.mask ? a.mask + (size_t)b * a.L : nullptr;
  const float om = __ldg(a.omega + d);
  const int L = a.L;
  const bool fwd = a.dir > 0;
  const bool pre_output = (!fwd) && a.shift;  // anti-causal with lag-1 start: emit before update
  constexpr int U = 8;
  // The optional mask and the accumulate pass are compile-time inside the loop: run-time tests of
  // them between the loads of a batch serialise those loads.
  auto scan = [&](auto mask_tag, auto acc_tag) {
  constexpr bool kMask = decltype(mask_tag)::value, kAcc = decltype(acc_tag)::value;
  for (int t0 = 0; t0 < L; t0 += U) {
    float xv[U], xd[U], yo[U];
    bool mk[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u;
      const int tt = fwd ? t : L - 1 - t;
      xv[u] = 0.f; xd[u] = 0.f; yo[u] = 0.f; mk[u] = true;
      if (t < L) {
        xv[u] = Elem<T>::ld(xp + tt * a.xsl);
        mk[u] = kMask ? __ldg(mp + tt) != 0 : false;
        if (kAcc) yo[u] = Elem<T>::ld_shared(yp + tt * a.ysl);  // written by the causal pass: plain load
        if (MODE == MODE_TRUNC) {
          const int td = fwd ? tt - a.ksize : tt + a.ksize;
          if (td >= 0 && td < L && !(kMask && __ldg(mp + td) != 0)) xd[u] = Elem<T>::ld(xp + td * a.xsl);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u;
      if (t < L) {
        const int tt = fwd ? t : L - 1 - t;
        const float xm = mk[u] ? 0.f : xv[u];
        float conv;
        if (pre_output) {
          conv = st.output();
          st.update(xm, xd[u]);
        } else {
          st.update(xm, xd[u]);
          conv = st.output();
        }
        float v = kAcc ? (yo[u] + conv) : fmaf(om, xv[u], conv);
        if (a.silu) v = siluf_(v);
        Elem<T>::st(yp + tt * a.ysl, v);
      }
    }
  }
  };
  using std::true_type;
  using std::false_type;
  if (mp) {
    if (a.accumulate) scan(true_type{}, true_type{}); else scan(true_type{}, false_type{});
  } else {
    if (a.accumulate) scan(false_type{}, true_type{}); else scan(false_type{}, false_type{});
  }
  st.export_state(a, b, d);
}

// Length-contiguous rows: a warp owns 32 rows and moves 32x32 tiles through shared memory so
// that global accesses are contiguous along L while each lane scans its own row.
template <typename T, int NP>
__global__ void __launch_bounds__(128) ema_scan_lenlast_kernel(EmaArgs a) {
  __shared__ float tile[4][32][33];
  __shared__ float ytile[4][32][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long rows = (long long)a.B * a.D;
  const long long r0 = ((long long)blockIdx.x * 4 + w) * 32;
  if (r0 >= rows) return;
  const long long r = r0 + lane;
  const bool valid = r < rows;
  const int d = valid ? (int)(r % a.D) : 0;
  const int b = valid ? (int)(r / a.D) : 0;
  Poles<NP, MODE_FAST> st;
  st.init(a, d + a.row_off, b, d);
  const long long xoff = b * a.xsb + d * a.xsd;
  const long long yoff = b * a.ysb + d * a.ysd;
  const T* xg = reinterpret_cast<const T*>(a.x);
  T* yg = reinterpret_cast<T*>(a.y);
  const unsigned char* mp = (a.mask && valid) ? a.mask + (size_t)b * a.L : nullptr;
  const float om = valid ? __ldg(a.omega + d) : 0.f;
  const int L = a.L;
  const bool fwd = a.dir > 0;
  const bool pre_output = (!fwd) && a.shift;
  const int ntiles = (L + 31) / 32;
  for (int it = 0; it < ntiles; ++it) {
    const int t0 = (fwd ? it : ntiles - 1 - it) * 32;
    const int t = t0 + lane;
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
      const long long xo = __shfl_sync(0xffffffffu, xoff, i);
      const long long yo = __shfl_sync(0xffffffffu, yoff, i);
      const bool rv = (r0 + i) < rows && t < L;
      tile[w][i][lane] = rv ? Elem<T>::ld(xg + xo + t) : 0.f;
      if (a.accumulate) ytile[w][i][lane] = rv ? Elem<T>::ld(yg + yo + t) : 0.f;
    }
    __syncwarp();
    const int nt = min(32, L - t0);
#pragma unroll 4
    for (int jj = 0; jj < 32; ++jj) {
      const int j = fwd ? jj : 31 - jj;
      if (j < nt) {
        const float xr = tile[w][lane][j];
        const bool mk = mp != nullptr && mp[t0 + j] != 0;
        const float xm = mk ? 0.f : xr;
        float conv;
        if (pre_output) {
          conv = st.output();
          st.update(xm, 0.f);
        } else {
          st.update(xm, 0.f);
          conv = st.output();
        }
        float v = a.accumulate ? (ytile[w][lane][j] + conv) : fmaf(om, xr, conv);
        if (a.silu) v = siluf_(v);
        tile[w][lane][j] = v;
      }
    }
    __syncwarp();
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
      const long long yo = __shfl_sync(0xffffffffu, yoff, i);
      if ((r0 + i) < rows && t < L) Elem<T>::st(yg + yo + t, tile[w][i][lane]);
    }
    __syncwarp();
  }
}

// Decode step: one thread per (b, d).
template <typename T, int NP>
__global__ void __launch_bounds__(128) ema_step_kernel(const T* __restrict__ x, T* __restrict__ y, int B,
                                                       int D, int N, const float* __restrict__ p,
                                                       const float* __restrict__ q,
                                                       const float* __restrict__ g,
                                                       const float* __restrict__ omega,
                                                       const float* h_in, float* h_out, int silu) {
  long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)B * D) return;
  const int d = (int)(gid % D);
  const float xv = Elem<T>::ld(x + gid);
  float acc = 0.f;
#pragma unroll
  for (int n = 0; n < NP; ++n) {
    if (n < N) {
      const float hp = h_in ? h_in[gid * N + n] : 0.f;
      const float hn = fmaf(__ldg(q + d * N + n), hp, __ldg(p + d * N + n) * xv);
      h_out[gid * N + n] = hn;
      acc = fmaf(__ldg(g + d * N + n), hn, acc);
    }
  }
  float v = fmaf(__ldg(omega + d), xv, acc);
  if (silu) v = siluf_(v);
  Elem<T>::st(y + gid, v);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <typename T, int NP>
static void launch_scan(const EmaArgs& a, int mode, cudaStream_t s) {
  const long long rows = (long long)a.B * a.D;
  const bool lenlast = a.xsl == 1 && a.ysl == 1 && a.xsd != 1 && a.L >= 32;
  if (mode == MODE_FAST && lenlast) {
    const unsigned grid = (unsigned)((rows + 127) / 128);
    launch(ema_scan_lenlast_kernel<T, NP>, grid, 128, 0, s, a);
    return;
  }
  const unsigned grid = (unsigned)((rows + 127) / 128);
  if (mode == MODE_FAST) {
    launch(ema_scan_rows_kernel<T, NP, MODE_FAST>, grid, 128, 0, s, a);
  } else if (mode == MODE_STATE) {
    launch(ema_scan_rows_kernel<T, NP, MODE_STATE>, grid, 128, 0, s, a);
  } else {
    launch(ema_scan_rows_kernel<T, NP, MODE_TRUNC>, grid, 128, 0, s, a);
  }
}

int ema_fwd_simt(const EmaArgs& base, unsigned flags, int truncation, int dtype, cudaStream_t s) {
  EmaArgs a = base;
  const bool bidir = flags & MEGA_EMA_BIDIRECTIONAL;
  const bool trunc = truncation > 0 && truncation < a.L;
  a.ksize = trunc ? truncation : a.L;
  const int mode = trunc ? MODE_TRUNC : ((a.h_in || a.h_out) ? MODE_STATE : MODE_FAST);
  const int np = next_pow2_ndim(a.N);
  a.dir = 1; a.shift = 0; a.accumulate = 0; a.row_off = 0;
  a.silu = (!bidir && (flags & MEGA_EMA_SILU)) ? 1 : 0;
  MEGA_DISPATCH_DTYPE(dtype, MEGA_DISPATCH_NP(np, (launch_scan<T, NP>(a, mode, s))));
  if (bidir) {
    a.dir = -1; a.shift = (flags & MEGA_EMA_NO_SHIFT) ? 0 : 1; a.accumulate = 1; a.row_off = a.D;
    a.silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
    a.x = base.x;
    MEGA_DISPATCH_DTYPE(dtype, MEGA_DISPATCH_NP(np, (launch_scan<T, NP>(a, mode, s))));
  }
  return check_launch("ema_fwd");
}

}  // namespace mega

using namespace mega;

extern "C" int mega_ema_coeffs(const void* alpha, const void* delta, const void* beta, const void* gamma,
                               int param_dtype, int K, int N, float* p, float* q, float* gamma_hat,
                               mega_stream_t stream) {
  if (!alpha || !delta || !beta || !gamma || !p || !q || !gamma_hat) return MEGA_ERR_NULL;
  if (!valid_dtype(param_dtype)) return MEGA_ERR_DTYPE;
  if (K <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  const int total = K * N;
  const float scale = sqrtf(1.0f / (float)N);
  const unsigned grid = (total + 255) / 256;
  MEGA_DISPATCH_DTYPE(param_dtype,
                      launch(ema_coeffs_kernel<T>, grid, 256, 0, stream, (const T*)alpha,
                                  (const T*)delta, (const T*)beta, (const T*)gamma, total, scale, p, q,
                                  gamma_hat));
  return check_launch("ema_coeffs");
}

extern "C" int mega_ema_kernel(const float* p, const float* q, const float* gamma_hat, int K, int N, int L,
                               float* kernel_out, mega_stream_t stream) {
  if (!p || !q || !gamma_hat || !kernel_out) return MEGA_ERR_NULL;
  if (K <= 0 || L <= 0 || K > 65535) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  dim3 grid((L + 255) / 256, K);
  launch(ema_kernel_kernel, grid, 256, 2 * N * sizeof(float), stream, p, q, gamma_hat, K, N, L,
              kernel_out);
  return check_launch("ema_kernel");
}

extern "C" int mega_ema_bias(const float* q, const float* gamma_hat, const float* h, int B, int D, int N,
                             int L, float* bias_out, mega_stream_t stream) {
  if (!q || !gamma_hat || !h || !bias_out) return MEGA_ERR_NULL;
  if (B <= 0 || D <= 0 || L <= 0 || (long long)B * D > 65535) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  dim3 grid((L + 255) / 256, B * D);
  launch(ema_bias_kernel, grid, 256, 2 * N * sizeof(float), stream, q, gamma_hat, h, D, N, L,
              bias_out);
  return check_launch("ema_bias");
}

extern "C" int mega_ema_fwd(const void* x, void* y, int dtype, int B, int D, int L, int64_t xsb, int64_t xsd,
                            int64_t xsl, int64_t ysb, int64_t ysd, int64_t ysl, const float* p,
                            const float* q, const float* gamma_hat, const float* omega, int N,
                            const uint8_t* pad_mask, const float* h_in, float* h_out, unsigned flags,
                            int truncation, mega_stream_t stream) {
  if (!x || !y || !p || !q || !gamma_hat || !omega) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || D <= 0 || L <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  if (!aligned_to(x, elem_size(dtype)) || !aligned_to(y, elem_size(dtype))) return MEGA_ERR_ALIGN;
  const bool bidir = flags & MEGA_EMA_BIDIRECTIONAL;
  if (bidir && (h_in || h_out)) return MEGA_ERR_UNSUPPORTED;
  if (!bidir && truncation > 0 && truncation < L) return MEGA_ERR_UNSUPPORTED;
  if (x == y && (xsb != ysb || xsd != ysd || xsl != ysl)) return MEGA_ERR_STRIDE;
  if (bidir && x == y) return MEGA_ERR_UNSUPPORTED;  // second pass re-reads x
  EmaArgs a{};
  a.x = x; a.y = y; a.B = B; a.D = D; a.L = L; a.N = N;
  a.xsb = xsb; a.xsd = xsd; a.xsl = xsl; a.ysb = ysb; a.ysd = ysd; a.ysl = ysl;
  a.p = p; a.q = q; a.g = gamma_hat; a.omega = omega; a.mask = pad_mask; a.h_in = h_in; a.h_out = h_out;
  if (!h_in && !h_out && !(truncation > 0 && truncation < L) && xsl == 1 && ysl == 1 && xsd != 1) {
    RowArgs ra{};
    ra.x = x; ra.y = y; ra.B = B; ra.D = D; ra.L = L; ra.N = N;
    ra.xsb = xsb; ra.xsd = xsd; ra.ysb = ysb; ra.ysd = ysd;
    ra.p = p; ra.q = q; ra.g = gamma_hat; ra.omega = omega; ra.mask = pad_mask;
    ra.shift = (flags & MEGA_EMA_NO_SHIFT) ? 0 : 1;
    ra.silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
    if (rowres_try(dtype, ra, xsl, ysl, bidir, false, (cudaStream_t)stream)) return check_launch("ema_fwd(rowres)");
  }
  if (!bidir && x != y) {
    StreamArgs sa{};
    sa.B = B; sa.L = L; sa.D = D; sa.N = N;
    sa.p = p; sa.q = q; sa.g = gamma_hat; sa.omega = omega; sa.h_in = h_in; sa.h_out = h_out; sa.mask = pad_mask;
    sa.silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
    // (a state is exported and L is not a multiple of the tensor-core step of 32: head on the
    // tensor-core kernel, ragged tail on the streamed kernel, continuing from the head's state in place)
    const int Lh = L - L % 32;
    if (h_out && Lh > 0 && Lh < L && !pad_mask) {
      StreamArgs head = sa;
      head.L = Lh;
      if (mma_cl_try(dtype, x, y, nullptr, xsb, xsl, xsd, ysb, ysl, ysd, false, head, (cudaStream_t)stream)) {
        const size_t es = (size_t)elem_size(dtype);
        const void* xt = (const char*)x + (size_t)Lh * xsl * es;
        void* yt = (char*)y + (size_t)Lh * ysl * es;
        StreamArgs tail = sa;
        tail.L = L - Lh;
        tail.h_in = h_out;
        if (stream_cl_try(dtype, xt, yt, nullptr, xsb, xsl, xsd, ysb, ysl, ysd, false, true, tail, (cudaStream_t)stream))
          return check_launch("ema_fwd(mma head + stream tail)");
        a.x = xt; a.y = yt; a.L = L - Lh; a.h_in = h_out;
        return ema_fwd_simt(a, flags, truncation, dtype, (cudaStream_t)stream);
      }
    }
    if (mma_cl_try(dtype, x, y, nullptr, xsb, xsl, xsd, ysb, ysl, ysd, false, sa, (cudaStream_t)stream))
      return check_launch("ema_fwd(mma)");
    if (stream_cl_try(dtype, x, y, nullptr, xsb, xsl, xsd, ysb, ysl, ysd, false, true, sa, (cudaStream_t)stream))
      return check_launch("ema_fwd(stream)");
  }
  return ema_fwd_simt(a, flags, truncation, dtype, (cudaStream_t)stream);
}

extern "C" int mega_ema_step(const void* x, void* y, int dtype, int B, int D, const float* p, const float* q,
                             const float* gamma_hat, const float* omega, int N, const float* h_in,
                             float* h_out, unsigned flags, mega_stream_t stream) {
  if (!x || !y || !p || !q || !gamma_hat || !omega || !h_out) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || D <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  const int np = next_pow2_ndim(N);
  const unsigned grid = (unsigned)(((long long)B * D + 127) / 128);
  const int silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
  if (step_lanes_try(dtype, x, y, nullptr, B, D, N, nullptr, nullptr, nullptr, nullptr, nullptr, 0.f, p, q, gamma_hat,
                     omega, h_in, h_out, silu, stream))
    return check_launch("ema_step(lanes)");
  MEGA_DISPATCH_DTYPE(dtype, MEGA_DISPATCH_NP(np, launch(ema_step_kernel<T, NP>, grid, 128, 0, stream,
                                                              (const T*)x, (T*)y, B, D, N, p, q, gamma_hat,
                                                              omega, h_in, h_out, silu)));
  return check_launch("ema_step");
}
