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
#include "tma.cuh"
#include "rowres.cuh"

namespace mega {


constexpr int kRowNP = 16;

constexpr int kSegPad = 4;  // pad words after every segment: keeps segments 16-byte aligned and
                            // staggers them over the banks (segment pitch = seg + 4 words)

// index of element i in the padded row buffer; i / seg by multiplication with
// magic = ceil(2^32 / seg) (exact for i < 2^16, seg <= 256)
__device__ __forceinline__ int padded(int i, unsigned magic) {
  return i + kSegPad * (int)__umulhi((unsigned)i, magic);
}

template <int kT>
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < kT / 32; ++i) r += red[i];
  return r;
}

// Exclusive scan, across the 256 segments of a row, of the affine maps s -> a s + loc (a = q^seg,
// one per pole).  The 256 x 16 local states go through a shared table; thread j then owns pole
// j / (T/16) and a block of 16 consecutive segments, scans them sequentially, the 16 block totals are
// folded the same way, and every thread reads back the state entering its own segment.
// `vseg` is the position of this thread's segment in scan order (tid, or 255 - tid right-to-left).
template <int kT>
__device__ __forceinline__ void carry_scan(float (&st)[kRowNP], const float* qrow, int nq, int seg, int vseg,
                                           float* tab, float* tot) {
  constexpr int kBlocks = kT / 16;       // blocks of 16 segments per pole (= threads per pole)
  constexpr int kPitch = kBlocks * 17;   // table words per pole
  const int tid = threadIdx.x;
  // table entry of (pole n, segment position v): n * kPitch + (v / 16) * 17 + v % 16
  const int wslot = (vseg >> 4) * 17 + (vseg & 15);
#pragma unroll
  for (int n = 0; n < kRowNP; ++n) tab[n * kPitch + wslot] = st[n];
  const int n = tid / kBlocks, sb = tid % kBlocks;
  float a1 = 0.f;
  if (n < nq) {
    const float qn = __ldg(qrow + n);
    a1 = qn > 0.f ? __expf((float)seg * __logf(qn)) : 0.f;
  }
  __syncthreads();
  float* col = tab + n * kPitch + sb * 17;
  float run = 0.f;
#pragma unroll
  for (int s = 0; s < 16; ++s) {
    const float v = col[s];
    col[s] = run;
    run = fmaf(a1, run, v);
  }
  tot[n * (kBlocks + 1) + sb] = run;
  __syncthreads();
  float a16 = a1 * a1;
  a16 *= a16; a16 *= a16; a16 *= a16;
  float pre = 0.f;
  for (int k = 0; k < sb; ++k) pre = fmaf(a16, pre, tot[n * (kBlocks + 1) + k]);
#pragma unroll
  for (int s = 0; s < 16; ++s) {
    col[s] += pre;
    pre *= a1;
  }
  __syncthreads();
#pragma unroll
  for (int n2 = 0; n2 < kRowNP; ++n2) st[n2] = tab[n2 * kPitch + wslot];
  __syncthreads();
}

template <int kDir, bool kEmit, bool kAccum, bool kPreEmit>
__device__ __forceinline__ void walk_segment(float* src, float* dst, int base, int seg, const float (&q)[kRowNP],
                                             const float (&c)[kRowNP], float (&st)[kRowNP], float om) {
  // kDir = +1 left to right, -1 right to left; four positions per shared-memory access; two poles
  // per packed fp32x2 operation (the kernel is bound by issue slots, not by the FMA pipe)
  constexpr int kH = kRowNP / 2;
  f32x2 q2[kH], c2[kH], s2[kH];
#pragma unroll
  for (int n = 0; n < kH; ++n) {
    q2[n] = pack2(q[2 * n], q[2 * n + 1]);
    c2[n] = pack2(c[2 * n], c[2 * n + 1]);
    s2[n] = pack2(st[2 * n], st[2 * n + 1]);
  }
  const int nq4 = seg >> 2;
  for (int k4 = 0; k4 < nq4; ++k4) {
    const int off = base + 4 * (kDir > 0 ? k4 : nq4 - 1 - k4);
    const float4 xv4 = *reinterpret_cast<const float4*>(src + off);
    float xs[4] = {xv4.x, xv4.y, xv4.z, xv4.w};
    float ys[4];
    if (kAccum) {
      const float4 y4 = *reinterpret_cast<const float4*>(dst + off);
      ys[0] = y4.x; ys[1] = y4.y; ys[2] = y4.z; ys[3] = y4.w;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = kDir > 0 ? u : 3 - u;
      const float xv = xs[e];
      const f32x2 x2 = pack2(xv, xv);
      if (!kEmit) {
#pragma unroll
        for (int n = 0; n < kH; ++n) s2[n] = fma2(q2[n], s2[n], x2);
      } else {
        f32x2 a0 = pack2(0.f, 0.f), a1 = pack2(0.f, 0.f);
#pragma unroll
        for (int n = 0; n < kH; n += 2) {
          if (kPreEmit) {
            a0 = fma2(c2[n], s2[n], a0);
            a1 = fma2(c2[n + 1], s2[n + 1], a1);
          }
          s2[n] = fma2(q2[n], s2[n], x2);
          s2[n + 1] = fma2(q2[n + 1], s2[n + 1], x2);
          if (!kPreEmit) {
            a0 = fma2(c2[n], s2[n], a0);
            a1 = fma2(c2[n + 1], s2[n + 1], a1);
          }
        }
        float lo, hi;
        unpack2(add2(a0, a1), lo, hi);
        ys[e] = kAccum ? ys[e] + (lo + hi) : fmaf(om, xv, lo + hi);
      }
    }
    if (kEmit) *reinterpret_cast<float4*>(dst + off) = make_float4(ys[0], ys[1], ys[2], ys[3]);
  }
#pragma unroll
  for (int n = 0; n < kH; ++n) unpack2(s2[n], st[2 * n], st[2 * n + 1]);
}

template <typename T, bool kBidir, bool kNorm, int kT>
__global__ void __launch_bounds__(kT) rowres_kernel(RowArgs a) {
  constexpr int kRowThreads = kT;
  extern __shared__ __align__(16) float smf[];
  const int L = a.L, seg = a.seg;
  const unsigned magic = a.magic;
  const int Lp = kRowThreads * (seg + kSegPad);
  float* bx = smf;                                   // row (x zeroed at pads, or normalised x)
  float* by = smf + Lp;                              // second buffer (bidirectional only)
  float* tab = smf + (kBidir ? 2 : 1) * Lp;          // [16][272] carry table
  float* tot = tab + kRowNP * (kT / 16) * 17;        // [16][kT/16 + 1]
  float* red = tot + kRowNP * (kT / 16 + 1);         // [kT/32]
  unsigned char* mk = reinterpret_cast<unsigned char*>(red + kT / 32);  // [kT * seg]

  const int tid = threadIdx.x;
  const int row = blockIdx.x;
  const int d = row % a.D, b = row / a.D;
  const T* xg = reinterpret_cast<const T*>(a.x) + b * a.xsb + d * a.xsd;
  T* yg = reinterpret_cast<T*>(a.y) + b * a.ysb + d * a.ysd;
  const unsigned char* mg = a.mask ? a.mask + (size_t)b * L : nullptr;
  const int Ltot = kRowThreads * seg;

  // the row buffer holds x zeroed at padded positions (and beyond L); the residual of padded
  // positions, which uses the unmasked x, is added when the row is stored
  for (int i0 = tid; i0 < Ltot; i0 += 8 * kRowThreads) {
    float xv[8];
    unsigned char mv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {  // eight independent loads in flight per thread
      const int i = i0 + u * kRowThreads;
      const bool in = i < L;
      mv[u] = in ? (mg ? mg[i] : 0) : 1;
      xv[u] = in ? Elem<T>::ld(xg + i) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * kRowThreads;
      if (i < Ltot) {
        mk[i] = mv[u];
        bx[padded(i, magic)] = mv[u] ? 0.f : xv[u];
      }
    }
  }
  __syncthreads();

  const int t0 = tid * seg;
  const int base = tid * (seg + kSegPad);  // this thread's segment, contiguous and 16-byte aligned
  if (kNorm) {
    float s = 0.f, c = 0.f;
    for (int k = 0; k < seg; k += 4) {
      const float4 v4 = *reinterpret_cast<const float4*>(bx + base + k);  // padded positions hold 0
      s += (v4.x + v4.y) + (v4.z + v4.w);
      const uchar4 m4 = *reinterpret_cast<const uchar4*>(mk + t0 + k);
      c += (m4.x ? 0.f : 1.f) + (m4.y ? 0.f : 1.f) + (m4.z ? 0.f : 1.f) + (m4.w ? 0.f : 1.f);
    }
    const float cnt = block_sum<kT>(c, red);
    const float mean = cnt > 0.f ? block_sum<kT>(s, red) / cnt : 0.f;
    float v = 0.f;
    for (int k = 0; k < seg; k += 4) {
      const float4 v4 = *reinterpret_cast<const float4*>(bx + base + k);
      const uchar4 m4 = *reinterpret_cast<const uchar4*>(mk + t0 + k);
      const float d0 = m4.x ? 0.f : v4.x - mean, d1 = m4.y ? 0.f : v4.y - mean;
      const float d2 = m4.z ? 0.f : v4.z - mean, d3 = m4.w ? 0.f : v4.w - mean;
      v = fmaf(d0, d0, v); v = fmaf(d1, d1, v); v = fmaf(d2, d2, v); v = fmaf(d3, d3, v);
    }
    const float var = cnt > 0.f ? block_sum<kT>(v, red) / cnt : 0.f;
    const float rstd = rsqrtf(var + a.eps);
    const float w = __ldg(a.ngamma + d), bb = __ldg(a.nbeta + d);
    const float sc = rstd * w, sh = fmaf(-mean, sc, bb);
    for (int k = 0; k < seg; k += 4) {
      float4 v4 = *reinterpret_cast<const float4*>(bx + base + k);
      const uchar4 m4 = *reinterpret_cast<const uchar4*>(mk + t0 + k);
      v4.x = m4.x ? 0.f : fmaf(v4.x, sc, sh);
      v4.y = m4.y ? 0.f : fmaf(v4.y, sc, sh);
      v4.z = m4.z ? 0.f : fmaf(v4.z, sc, sh);
      v4.w = m4.w ? 0.f : fmaf(v4.w, sc, sh);
      *reinterpret_cast<float4*>(bx + base + k) = v4;
    }
    if (tid == 0) {
      if (a.mean_out) a.mean_out[row] = mean;
      if (a.rstd_out) a.rstd_out[row] = rstd;
      if (a.count_out && d == 0) a.count_out[b] = (long long)(cnt + 0.5f);
    }
  }

  const float om = __ldg(a.omega + d);

  // ------------------------------ causal half ----------------------------------------------
  {
    float q[kRowNP], c[kRowNP], st[kRowNP];
    const float* qrow = a.q + (size_t)d * a.N;
#pragma unroll
    for (int n = 0; n < kRowNP; ++n) {
      float pn = 0.f, qn = 0.f, gn = 0.f;
      if (n < a.N) {
        pn = __ldg(a.p + (size_t)d * a.N + n);
        qn = __ldg(qrow + n);
        gn = __ldg(a.g + (size_t)d * a.N + n);
      }
      q[n] = qn; c[n] = pn * gn; st[n] = 0.f;
    }
    walk_segment<1, false, false, false>(bx, bx, base, seg, q, c, st, om);
    carry_scan<kT>(st, qrow, a.N, seg, tid, tab, tot);
    walk_segment<1, true, false, false>(bx, kBidir ? by : bx, base, seg, q, c, st, om);
  }
  // ------------------------------ anti-causal half ------------------------------------------
  if (kBidir) {
    float q[kRowNP], c[kRowNP], st[kRowNP];
    const int r2 = d + a.D;
    const float* qrow = a.q + (size_t)r2 * a.N;
#pragma unroll
    for (int n = 0; n < kRowNP; ++n) {
      float pn = 0.f, qn = 0.f, gn = 0.f;
      if (n < a.N) {
        pn = __ldg(a.p + (size_t)r2 * a.N + n);
        qn = __ldg(qrow + n);
        gn = __ldg(a.g + (size_t)r2 * a.N + n);
      }
      q[n] = qn; c[n] = pn * gn; st[n] = 0.f;
    }
    walk_segment<-1, false, false, false>(bx, bx, base, seg, q, c, st, om);
    carry_scan<kT>(st, qrow, a.N, seg, kRowThreads - 1 - tid, tab, tot);
    if (a.shift)  // taps start at lag 1: emit from the state before the position enters
      walk_segment<-1, true, true, true>(bx, by, base, seg, q, c, st, om);
    else
      walk_segment<-1, true, true, false>(bx, by, base, seg, q, c, st, om);
  }
  __syncthreads();
  const float* out = kBidir ? by : bx;
  for (int i = tid; i < L; i += kRowThreads) {
    float v = out[padded(i, magic)];
    if (!kNorm && mk[i]) v = fmaf(om, Elem<T>::ld(xg + i), v);  // residual of the unmasked x at a pad
    if (a.silu) v = siluf_(v);
    Elem<T>::st(yg + i, v);
  }
}

template <typename T, bool kBidir, bool kNorm, int kT>
static bool launch_rowres(const RowArgs& a, size_t smem, cudaStream_t s) {
  auto kern = rowres_kernel<T, kBidir, kNorm, kT>;
  static std::once_flag once;
  static bool attr_ok = true;
  std::call_once(once, [&] {
    attr_ok = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) == cudaSuccess;
    cudaGetLastError();
  });
  if (!attr_ok) return false;
  launch(kern, dim3((unsigned)((long long)a.B * a.D)), dim3(kT), smem, (void*)s, a);
  g_last_kernel.store("rowres", std::memory_order_relaxed);
  return true;
}

static size_t rowres_smem(int threads, int seg, bool bidir) {
  const size_t lp = (size_t)threads * (seg + kSegPad);
  return ((bidir ? 2 : 1) * lp + kRowNP * (threads / 16) * 17 + kRowNP * (threads / 16 + 1) + threads / 32) * sizeof(float) +
         (size_t)threads * seg + 16;
}

// Tries the row-resident path: length stride 1 on both tensors, ndim <= 16, no carried state, no
// truncation, the row (two copies when bidirectional) fits in shared memory, at least 512 positions.
bool rowres_try(int dtype, const RowArgs& a_in, long long xsl, long long ysl, bool bidir, bool norm,
                cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (xsl != 1 || ysl != 1 || a_in.N > kRowNP || a_in.L < 512 || a_in.L > 65535) return false;
  if ((long long)a_in.B * a_in.D > 0x7fffffffLL) return false;
  RowArgs a = a_in;
  // 512 threads per row (16 warps per SM at one row per SM) once segments stay >= 16 positions
  int threads = a.L >= 8192 ? 512 : 256;
  int seg = (((a.L + threads - 1) / threads) + 3) & ~3;
  if (threads == 512 && rowres_smem(512, seg, bidir) > 220 * 1024) {
    threads = 256;
    seg = (((a.L + threads - 1) / threads) + 3) & ~3;
  }
  a.seg = seg;
  a.magic = (unsigned)((0x100000000ULL + seg - 1) / seg);
  const size_t smem = rowres_smem(threads, seg, bidir);
  if (smem > 220 * 1024) return false;
  bool ok = false;
  switch (dtype) {
#define MEGA_ROW_LAUNCH(TY, BI, NO) (threads == 512 ? launch_rowres<TY, BI, NO, 512>(a, smem, s) : launch_rowres<TY, BI, NO, 256>(a, smem, s))
#define MEGA_ROW_CASE(DT, TY)                                                                    \
  case DT:                                                                                       \
    if (bidir) ok = norm ? MEGA_ROW_LAUNCH(TY, true, true) : MEGA_ROW_LAUNCH(TY, true, false);   \
    else ok = norm ? MEGA_ROW_LAUNCH(TY, false, true) : MEGA_ROW_LAUNCH(TY, false, false);       \
    break;
    MEGA_ROW_CASE(MEGA_F32, float)
    MEGA_ROW_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_ROW_CASE(MEGA_F16, __half)
#undef MEGA_ROW_CASE
#undef MEGA_ROW_LAUNCH
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
