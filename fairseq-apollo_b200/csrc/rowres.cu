// Row-resident EMA for length-contiguous activations ((B, D, L) memory): causal or bidirectional,
// optionally preceded by a fused per-channel SequenceNorm.
//
// One CTA of 256 threads owns one (batch, channel) row, keeps it in shared memory (fp32) and
// splits it into 256 contiguous segments.  Each thread (1) folds its segment into local pole
// states, (2) the CTA scans those states across segments (warp shuffles, then across warps),
// (3) each thread re-walks its segment from the correct incoming state and emits the outputs.
// The anti-causal half of a bidirectional layer runs the same three steps right to left into a
// second row buffer.  HBM sees the row once in and once out, whatever the number of passes.
#include <mutex>

#include "common.cuh"
#include "rowres.cuh"

namespace mega {


constexpr int kRowThreads = 256;
constexpr int kRowNP = 16;

__device__ __forceinline__ int padded(int i, int seg) { return i + i / seg; }

__device__ __forceinline__ float block_sum256(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < kRowThreads / 32; ++i) r += red[i];
  return r;
}

// Exclusive scan across the 256 segments of the affine maps s -> a s + loc (a = q^seg, the same
// for every segment).  On return st[n] holds the state entering this thread's segment.
// `reverse` scans right to left (for the anti-causal half).
__device__ __forceinline__ void carry_scan(float (&st)[kRowNP], const float (&aseg)[kRowNP], float* wtot,
                                           bool reverse) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int vl = reverse ? 31 - lane : lane;  // position of this lane in scan order
  float apow[kRowNP];
#pragma unroll
  for (int n = 0; n < kRowNP; ++n) apow[n] = aseg[n];
  // inclusive Hillis-Steele within the warp
#pragma unroll
  for (int dlt = 1; dlt < 32; dlt <<= 1) {
#pragma unroll
    for (int n = 0; n < kRowNP; ++n) {
      const float o = reverse ? __shfl_down_sync(0xffffffffu, st[n], dlt) : __shfl_up_sync(0xffffffffu, st[n], dlt);
      if (vl >= dlt) st[n] = fmaf(apow[n], o, st[n]);
      apow[n] *= apow[n];
    }
  }
  // apow now holds a^32.  Warp totals -> shared, then each warp folds in the warps before it.
  const int vw = reverse ? (kRowThreads / 32 - 1 - w) : w;
  if (vl == 31) {
#pragma unroll
    for (int n = 0; n < kRowNP; ++n) wtot[w * kRowNP + n] = st[n];
  }
  __syncthreads();
  float pre[kRowNP];  // state entering this warp
#pragma unroll
  for (int n = 0; n < kRowNP; ++n) pre[n] = 0.f;
  for (int k = 0; k < vw; ++k) {
    const int src = reverse ? (kRowThreads / 32 - 1 - k) : k;
#pragma unroll
    for (int n = 0; n < kRowNP; ++n) pre[n] = fmaf(apow[n], pre[n], wtot[src * kRowNP + n]);
  }
  // exclusive value for this lane: inclusive of the previous lane, plus a^(vl) * pre
#pragma unroll
  for (int n = 0; n < kRowNP; ++n) {
    float prev = reverse ? __shfl_down_sync(0xffffffffu, st[n], 1) : __shfl_up_sync(0xffffffffu, st[n], 1);
    if (vl == 0) prev = 0.f;
    // a^vl by binary powers of aseg
    float av = 1.f, b = aseg[n];
    int e = vl;
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      if (e & 1) av *= b;
      b *= b;
      e >>= 1;
    }
    st[n] = fmaf(av, pre[n], prev);
  }
  __syncthreads();
}

template <typename T, bool kBidir, bool kNorm>
__global__ void __launch_bounds__(kRowThreads) rowres_kernel(RowArgs a) {
  extern __shared__ float smf[];
  const int L = a.L, seg = a.seg;
  const int Lp = padded(kRowThreads * seg, seg) + 4;
  float* bx = smf;                       // row (raw or normalised x), padded per segment
  float* by = smf + Lp;                  // second buffer (bidirectional only)
  float* red = smf + (kBidir ? 2 : 1) * Lp;        // [8]
  float* wtot = red + 8;                           // [8][16]
  unsigned char* mk = reinterpret_cast<unsigned char*>(wtot + 8 * kRowNP);  // [256*seg]

  const int tid = threadIdx.x;
  const int row = blockIdx.x;
  const int d = row % a.D, b = row / a.D;
  const T* xg = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  T* yg = reinterpret_cast<T*>(a.y) + b * a.ysb + d * a.ysd;
  const unsigned char* mg = a.mask ? a.mask + (size_t)b * L : nullptr;
  const int Ltot = kRowThreads * seg;

  for (int i = tid; i < Ltot; i += kRowThreads) {
    const bool in = i < L;
    bx[padded(i, seg)] = in ? Elem<T>::ld(xg + i) : 0.f;
    mk[i] = in ? (mg ? mg[i] : 0) : 1;
  }
  __syncthreads();

  if (kNorm) {
    float s = 0.f, c = 0.f;
    for (int i = tid; i < L; i += kRowThreads)
      if (!mk[i]) { s += bx[padded(i, seg)]; c += 1.f; }
    const float cnt = block_sum256(c, red);
    const float mean = cnt > 0.f ? block_sum256(s, red) / cnt : 0.f;
    float v = 0.f;
    for (int i = tid; i < L; i += kRowThreads)
      if (!mk[i]) { const float dl = bx[padded(i, seg)] - mean; v = fmaf(dl, dl, v); }
    const float var = cnt > 0.f ? block_sum256(v, red) / cnt : 0.f;
    const float rstd = rsqrtf(var + a.eps);
    const float w = __ldg(a.ngamma + d), bb = __ldg(a.nbeta + d);
    for (int i = tid; i < L; i += kRowThreads) {
      const int pi = padded(i, seg);
      bx[pi] = mk[i] ? 0.f : fmaf((bx[pi] - mean) * rstd, w, bb);
    }
    if (tid == 0) {
      if (a.mean_out) a.mean_out[row] = mean;
      if (a.rstd_out) a.rstd_out[row] = rstd;
      if (a.count_out && d == 0) a.count_out[b] = (long long)(cnt + 0.5f);
    }
    __syncthreads();
  }

  const int t0 = tid * seg;
  const int base = padded(t0, seg);  // this thread's segment is contiguous from here
  const float om = __ldg(a.omega + d);

  // ------------------------------ causal half ----------------------------------------------
  {
    float q[kRowNP], c[kRowNP], st[kRowNP], aseg[kRowNP];
#pragma unroll
    for (int n = 0; n < kRowNP; ++n) {
      float pn = 0.f, qn = 0.f, gn = 0.f;
      if (n < a.N) {
        pn = __ldg(a.p + (size_t)d * a.N + n);
        qn = __ldg(a.q + (size_t)d * a.N + n);
        gn = __ldg(a.g + (size_t)d * a.N + n);
      }
      q[n] = qn; c[n] = pn * gn; st[n] = 0.f;
      aseg[n] = qn > 0.f ? __expf((float)seg * __logf(qn)) : 0.f;
    }
    for (int k = 0; k < seg; ++k) {
      const float xv = mk[t0 + k] ? 0.f : bx[base + k];
#pragma unroll
      for (int n = 0; n < kRowNP; ++n) st[n] = fmaf(q[n], st[n], xv);
    }
    carry_scan(st, aseg, wtot, false);
    float* out = kBidir ? by : bx;
    for (int k = 0; k < seg; ++k) {
      const float xr = bx[base + k];
      const float xv = mk[t0 + k] ? 0.f : xr;
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int n = 0; n < kRowNP; n += 2) {
        st[n] = fmaf(q[n], st[n], xv);
        st[n + 1] = fmaf(q[n + 1], st[n + 1], xv);
        a0 = fmaf(c[n], st[n], a0);
        a1 = fmaf(c[n + 1], st[n + 1], a1);
      }
      out[base + k] = fmaf(om, xr, a0 + a1);
    }
  }
  // ------------------------------ anti-causal half ------------------------------------------
  if (kBidir) {
    float q[kRowNP], c[kRowNP], st[kRowNP], aseg[kRowNP];
    const int r2 = d + a.D;
#pragma unroll
    for (int n = 0; n < kRowNP; ++n) {
      float pn = 0.f, qn = 0.f, gn = 0.f;
      if (n < a.N) {
        pn = __ldg(a.p + (size_t)r2 * a.N + n);
        qn = __ldg(a.q + (size_t)r2 * a.N + n);
        gn = __ldg(a.g + (size_t)r2 * a.N + n);
      }
      q[n] = qn; c[n] = pn * gn; st[n] = 0.f;
      aseg[n] = qn > 0.f ? __expf((float)seg * __logf(qn)) : 0.f;
    }
    for (int k = seg - 1; k >= 0; --k) {
      const float xv = mk[t0 + k] ? 0.f : bx[base + k];
#pragma unroll
      for (int n = 0; n < kRowNP; ++n) st[n] = fmaf(q[n], st[n], xv);
    }
    carry_scan(st, aseg, wtot, true);
    for (int k = seg - 1; k >= 0; --k) {
      const float xv = mk[t0 + k] ? 0.f : bx[base + k];
      float a0 = 0.f, a1 = 0.f;
      if (a.shift) {  // taps start at lag 1: emit from the state before this position enters
#pragma unroll
        for (int n = 0; n < kRowNP; n += 2) {
          a0 = fmaf(c[n], st[n], a0);
          a1 = fmaf(c[n + 1], st[n + 1], a1);
          st[n] = fmaf(q[n], st[n], xv);
          st[n + 1] = fmaf(q[n + 1], st[n + 1], xv);
        }
      } else {
#pragma unroll
        for (int n = 0; n < kRowNP; n += 2) {
          st[n] = fmaf(q[n], st[n], xv);
          st[n + 1] = fmaf(q[n + 1], st[n + 1], xv);
          a0 = fmaf(c[n], st[n], a0);
          a1 = fmaf(c[n + 1], st[n + 1], a1);
        }
      }
      by[base + k] += a0 + a1;
    }
  }
  __syncthreads();
  const float* out = kBidir ? by : bx;
  for (int i = tid; i < L; i += kRowThreads) {
    float v = out[padded(i, seg)];
    if (a.silu) v = siluf_(v);
    Elem<T>::st(yg + i, v);
  }
}

template <typename T, bool kBidir, bool kNorm>
static bool launch_rowres(const RowArgs& a, size_t smem, cudaStream_t s) {
  auto kern = rowres_kernel<T, kBidir, kNorm>;
  static std::once_flag once;
  static bool attr_ok = true;
  std::call_once(once, [&] {
    attr_ok = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) == cudaSuccess;
    cudaGetLastError();
  });
  if (!attr_ok) return false;
  launch(kern, dim3((unsigned)((long long)a.B * a.D)), dim3(kRowThreads), smem, (void*)s, a);
  return true;
}

// Tries the row-resident path: length stride 1 on both tensors, ndim <= 16, no carried state, no
// truncation, the row (two copies when bidirectional) fits in shared memory, at least 512 positions.
bool rowres_try(int dtype, const RowArgs& a_in, long long xsl, long long ysl, bool bidir, bool norm,
                cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (xsl != 1 || ysl != 1 || a_in.N > kRowNP || a_in.L < 512) return false;
  if ((long long)a_in.B * a_in.D > 0x7fffffffLL) return false;
  RowArgs a = a_in;
  int seg = (a.L + kRowThreads - 1) / kRowThreads;
  seg += seg & 1;
  a.seg = seg;
  const size_t lp = (size_t)kRowThreads * seg + kRowThreads + 4;
  const size_t smem = ((bidir ? 2 : 1) * lp + 8 + 8 * kRowNP) * sizeof(float) + (size_t)kRowThreads * seg + 16;
  if (smem > 220 * 1024) return false;
  bool ok = false;
  switch (dtype) {
#define MEGA_ROW_CASE(DT, TY)                                                                    \
  case DT:                                                                                       \
    if (bidir) ok = norm ? launch_rowres<TY, true, true>(a, smem, s) : launch_rowres<TY, true, false>(a, smem, s);   \
    else ok = norm ? launch_rowres<TY, false, true>(a, smem, s) : launch_rowres<TY, false, false>(a, smem, s);      \
    break;
    MEGA_ROW_CASE(MEGA_F32, float)
    MEGA_ROW_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_ROW_CASE(MEGA_F16, __half)
#undef MEGA_ROW_CASE
    default: return false;
  }
  return ok;
}

}  // namespace mega

using namespace mega;

extern "C" MEGA_API int mega_sqn_ema_fwd(const void* x, void* y, int dtype, int B, int D, int L, int64_t xsb,
                                         int64_t xsd, int64_t xsl, int64_t ysb, int64_t ysd, int64_t ysl,
                                         const float* norm_gamma, const float* norm_beta, double eps,
                                         int64_t* count_out, float* mean_out, float* rstd_out, const float* p,
                                         const float* q, const float* gamma_hat, const float* omega, int N,
                                         const uint8_t* pad_mask, unsigned flags, mega_stream_t stream) {
  if (!x || !y || !norm_gamma || !norm_beta || !p || !q || !gamma_hat || !omega) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (B <= 0 || D <= 0 || L <= 0) return MEGA_ERR_SHAPE;
  if (N < 1 || N > MEGA_MAX_NDIM) return MEGA_ERR_NDIM;
  if (!aligned_to(x, elem_size(dtype)) || !aligned_to(y, elem_size(dtype))) return MEGA_ERR_ALIGN;
  RowArgs a{};
  a.x = x; a.y = y; a.B = B; a.D = D; a.L = L; a.N = N;
  a.xsb = xsb; a.xsd = xsd; a.ysb = ysb; a.ysd = ysd;
  a.p = p; a.q = q; a.g = gamma_hat; a.omega = omega; a.mask = pad_mask;
  a.ngamma = norm_gamma; a.nbeta = norm_beta; a.eps = (float)eps;
  a.count_out = (long long*)count_out; a.mean_out = mean_out; a.rstd_out = rstd_out;
  a.shift = (flags & MEGA_EMA_NO_SHIFT) ? 0 : 1;
  a.silu = (flags & MEGA_EMA_SILU) ? 1 : 0;
  if (!rowres_try(dtype, a, xsl, ysl, (flags & MEGA_EMA_BIDIRECTIONAL) != 0, true, (cudaStream_t)stream))
    return MEGA_ERR_UNSUPPORTED;
  return check_launch("sqn_ema_fwd");
}
