// Streamed backward kernels for channel-contiguous activations ((B, L, D) memory): TimestepNorm
// (per-feature) and the causal EMA.  Same data movement as the streamed forward kernels: a CTA
// owns kW adjacent channels of one sequence, tiles of kR timesteps arrive through a TMA ring
// (cp.async.bulk.tensor + mbarrier) and the input gradient leaves through TMA stores, so HBM sees
// whole row segments while every thread keeps its channel's recurrences in registers.
//
// TimestepNorm walks time backwards once.  The EMA makes two passes: forward in time for the
// parameter sums (states h, sensitivities s = dh/dq and r = dh/dp, no history stored), then
// backwards for the input gradient (lambda_t = g dy_t + q lambda_{t+1}).
#include <mutex>

#include "common.cuh"
#include "stream_bwd.cuh"
#include "tma.cuh"

namespace mega {

namespace {

constexpr int kW = 64;   // channels per CTA (= threads)
constexpr int kR = 32;   // timesteps per tile
constexpr int kS = 3;    // ring depth
constexpr int kNP = 16;  // poles held in registers
constexpr int kHead = 512;

// ---------------------------------------------------------------------------------------------
// TimestepNorm
// ---------------------------------------------------------------------------------------------
template <typename T>
struct TsnCfg {
  static constexpr int kTileT = kR * kW * (int)sizeof(T);   // x, dy, dx
  static constexpr int kTileF = kR * kW * 4;                // cumrstd
  static constexpr int kTileM = (kR + 1) * kW * 4;          // cummean, with the row before the tile
  static constexpr int kStage = 2 * kTileT + kTileF + kTileM;
  static constexpr int kSmem = kHead + kS * kStage + 2 * kTileT + 128;
};

template <typename T, bool kMask>
__global__ void __launch_bounds__(kW) tsn_bwd_stream_kernel(const __grid_constant__ CUtensorMap tmx,
                                                            const __grid_constant__ CUtensorMap tmg,
                                                            const __grid_constant__ CUtensorMap tmd,
                                                            const __grid_constant__ CUtensorMap tmm,
                                                            const __grid_constant__ CUtensorMap tmr,
                                                            TsnBwdStreamArgs a) {
  using C = TsnCfg<T>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  float* cbuf = reinterpret_cast<float*>(base);                      // [2][kR] 1/count per row, < 0: padded
  uint64_t* full = reinterpret_cast<uint64_t*>(base + 2 * kR * 4);   // [kS]
  unsigned char* stages = base + kHead;
  T* outs = reinterpret_cast<T*>(base + kHead + kS * C::kStage);     // [2][kR][kW]

  const int tid = threadIdx.x;
  const int d0 = blockIdx.x * kW;
  const int b = blockIdx.y;
  const int d = d0 + tid;
  const bool valid = d < a.D;
  const int dc = valid ? d : a.D - 1;
  const int L = a.L;
  const int nt = (L + kR - 1) / kR;

  auto issue = [&](int k) {  // k-th tile in processing order = tile nt-1-k of the sequence
    const int s = k % kS, i = nt - 1 - k;
    unsigned char* st = stages + (size_t)s * C::kStage;
    mbar_expect_tx(&full[s], C::kStage);
    tma_load_3d(st, &tmx, d0, i * kR, b, &full[s]);
    tma_load_3d(st + C::kTileT, &tmg, d0, i * kR, b, &full[s]);
    tma_load_3d(st + 2 * C::kTileT, &tmr, d0, i * kR, b, &full[s]);
    tma_load_3d(st + 2 * C::kTileT + C::kTileF, &tmm, d0, i * kR - 1, b, &full[s]);
  };
  if (tid == 0) {
    prefetch_tensormap(&tmx);
    prefetch_tensormap(&tmg);
    prefetch_tensormap(&tmd);
    prefetch_tensormap(&tmm);
    prefetch_tensormap(&tmr);
#pragma unroll
    for (int s = 0; s < kS; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0)
    for (int k = 0; k < kS && k < nt; ++k) issue(k);

  const float w = __ldg(a.gamma + dc);
  const float pm = a.prev_mean[(size_t)b * a.D + dc];
  float ug = a.dmean ? a.dmean[(size_t)b * a.D + dc] : 0.f;
  float vg = a.dvar ? a.dvar[(size_t)b * a.D + dc] : 0.f;
  float wg = 0.f, bg = 0.f;

  // warp 0 walks the count backwards and publishes 1/count per row of the next tile
  long long cnt_run = a.count[b];
  const unsigned char* mrow = kMask ? a.mask + (size_t)b * L : nullptr;
  auto publish = [&](int k, unsigned char mk_byte) {
    const int i = nt - 1 - k;
    const int t = i * kR + tid;
    const bool masked = (t >= L) || (kMask && mk_byte != 0);
    const unsigned vmask = __ballot_sync(0xffffffffu, !masked);
    const unsigned later = tid == 31 ? 0u : (vmask & (0xffffffffu << (tid + 1)));
    const float cf = rcp_approx((float)(cnt_run - __popc(later)));
    cbuf[(k & 1) * kR + tid] = masked ? -1.0f : cf;
    cnt_run -= __popc(vmask);
  };
  if (tid < 32) {
    const int t = (nt - 1) * kR + tid;
    publish(0, (kMask && t < L) ? mrow[t] : 0);
  }
  __syncthreads();

  for (int k = 0; k < nt; ++k) {
    const int s = k % kS;
    const uint32_t ph = (uint32_t)((k / kS) & 1);
    const int i = nt - 1 - k;
    const int o = k & 1;
    unsigned char mb_next = 0;
    if (kMask && tid < 32 && k + 1 < nt) {
      const int t = (i - 1) * kR + tid;
      if (t < L) mb_next = mrow[t];
    }
    const bool ok = mbar_wait(&full[s], ph);
    const unsigned char* st = stages + (size_t)s * C::kStage;
    const T* xt = reinterpret_cast<const T*>(st) + tid;
    const T* gt = reinterpret_cast<const T*>(st + C::kTileT) + tid;
    const float* rt = reinterpret_cast<const float*>(st + 2 * C::kTileT) + tid;
    const float* mt = reinterpret_cast<const float*>(st + 2 * C::kTileT + C::kTileF) + tid;  // row r+1 = step r
    T* ot = outs + (size_t)o * kR * kW + tid;
    const float* cf = cbuf + o * kR;
    const int rows = min(kR, L - i * kR);
#pragma unroll 8
    for (int rr = 0; rr < kR; ++rr) {
      const int r = kR - 1 - rr;
      if (r < rows) {
        const float coef = cf[r];
        const bool mk = coef < 0.f;
        const float x = Elem<T>::ld_shared(xt + r * kW), dy = Elem<T>::ld_shared(gt + r * kW);
        const float u = mt[(r + 1) * kW], rs = rt[r * kW];
        const float pu = (i == 0 && r == 0) ? pm : mt[r * kW];
        const float dyr = dy * rs, delta = x - u, xp = x - pu;
        const float dv = vg - 0.5f * dy * w * delta * (rs * rs * rs);
        const float du = ug - (w * dyr + coef * dv * xp);
        const float dx = w * dyr + dv * coef * (delta + xp) + coef * du;
        Elem<T>::st(ot + r * kW, mk ? 0.f : dx);
        ug = mk ? ug : (1.f - coef) * du - coef * delta * dv;
        vg = mk ? vg : (1.f - coef) * dv;
        wg = mk ? wg : fmaf(dyr, delta, wg);
        bg = mk ? bg : bg + dy;
      }
    }
    if (tid < 32 && k + 1 < nt) publish(k + 1, mb_next);
    fence_proxy_async();
    if (tid == 0) bulk_wait_read<0>();
    if (__syncthreads_or(!ok)) break;
    if (tid == 0) {
      tma_store_3d(&tmd, d0, i * kR, b, outs + (size_t)o * kR * kW);
      bulk_commit();
      if (k + kS < nt) issue(k + kS);
    }
  }
  if (tid == 0) bulk_wait<0>();
  if (valid) {
    a.dprev_mean[(size_t)b * a.D + d] = ug;
    a.dprev_var[(size_t)b * a.D + d] = vg;
    atomicAdd(a.dgamma + d, wg);
    atomicAdd(a.dbeta + d, bg);
  }
}

// ---------------------------------------------------------------------------------------------
// causal EMA
// ---------------------------------------------------------------------------------------------
template <typename T>
struct EmaCfg {
  static constexpr int kTileT = kR * kW * (int)sizeof(T);
  static constexpr int kStage = 2 * kTileT;  // pass A: x and dy; pass B uses the dy half only
  static constexpr int kSmem = kHead + kS * kStage + 2 * kTileT + 128;
};

template <typename T, bool kMask>
__global__ void __launch_bounds__(kW) ema_bwd_stream_kernel(const __grid_constant__ CUtensorMap tmx,
                                                            const __grid_constant__ CUtensorMap tmg,
                                                            const __grid_constant__ CUtensorMap tmd,
                                                            EmaBwdStreamArgs a) {
  using C = EmaCfg<T>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full_a = reinterpret_cast<uint64_t*>(base);       // [kS] pass A
  uint64_t* full_b = full_a + kS;                              // [kS] pass B
  unsigned char* stages = base + kHead;
  T* outs = reinterpret_cast<T*>(base + kHead + kS * C::kStage);

  const int tid = threadIdx.x;
  const int d0 = blockIdx.x * kW;
  const int b = blockIdx.y;
  const int d = d0 + tid;
  const bool valid = d < a.D;
  const int dc = valid ? d : a.D - 1;
  const int L = a.L;
  const int nt = (L + kR - 1) / kR;
  const unsigned char* mrow = kMask ? a.mask + (size_t)b * L : nullptr;

  if (tid == 0) {
    prefetch_tensormap(&tmx);
    prefetch_tensormap(&tmg);
    prefetch_tensormap(&tmd);
#pragma unroll
    for (int s = 0; s < kS; ++s) {
      mbar_init(&full_a[s], 1);
      mbar_init(&full_b[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  auto issue_a = [&](int i) {
    const int s = i % kS;
    unsigned char* st = stages + (size_t)s * C::kStage;
    mbar_expect_tx(&full_a[s], C::kStage);
    tma_load_3d(st, &tmx, d0, i * kR, b, &full_a[s]);
    tma_load_3d(st + C::kTileT, &tmg, d0, i * kR, b, &full_a[s]);
  };
  if (tid == 0)
    for (int i = 0; i < kS && i < nt; ++i) issue_a(i);

  // coefficients and states, two poles per packed register
  f32x2 q2[kNP / 2], p2[kNP / 2], g2[kNP / 2], h2[kNP / 2], s2[kNP / 2], r2[kNP / 2];
  f32x2 ag2[kNP / 2], aq2[kNP / 2], ap2[kNP / 2];
  const float om = __ldg(a.omega + dc);
  const size_t srow = ((size_t)b * a.D + dc) * a.N;
#pragma unroll
  for (int j = 0; j < kNP / 2; ++j) {
    float pv[2], qv[2], gv[2], hv[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int n = 2 * j + k;
      pv[k] = qv[k] = gv[k] = hv[k] = 0.f;
      if (n < a.N) {
        pv[k] = __ldg(a.p + (size_t)dc * a.N + n);
        qv[k] = __ldg(a.q + (size_t)dc * a.N + n);
        gv[k] = __ldg(a.g + (size_t)dc * a.N + n);
        if (a.h_in) hv[k] = __ldg(a.h_in + srow + n);
      }
    }
    q2[j] = pack2(qv[0], qv[1]);
    p2[j] = pack2(pv[0], pv[1]);
    g2[j] = pack2(gv[0], gv[1]);
    h2[j] = pack2(hv[0], hv[1]);
    s2[j] = r2[j] = ag2[j] = aq2[j] = ap2[j] = pack2(0.f, 0.f);
  }
  float aw = 0.f;

  // ---- pass A: forward in time, parameter sums ------------------------------------------------
  bool healthy = true;
  for (int i = 0; i < nt; ++i) {
    const int s = i % kS;
    const uint32_t ph = (uint32_t)((i / kS) & 1);
    const bool ok = mbar_wait(&full_a[s], ph);
    const unsigned char* st = stages + (size_t)s * C::kStage;
    const T* xt = reinterpret_cast<const T*>(st) + tid;
    const T* gt = reinterpret_cast<const T*>(st + C::kTileT) + tid;
    const int rows = min(kR, L - i * kR);
#pragma unroll 4
    for (int r = 0; r < kR; ++r) {
      if (r < rows) {
        const float xr = Elem<T>::ld_shared(xt + r * kW), dy = Elem<T>::ld_shared(gt + r * kW);
        aw = fmaf(dy, xr, aw);
        const float xm = (kMask && mrow[i * kR + r] != 0) ? 0.f : xr;
        const f32x2 x2 = pack2(xm, xm), d2 = pack2(dy, dy);
#pragma unroll
        for (int j = 0; j < kNP / 2; ++j) {
          s2[j] = fma2(q2[j], s2[j], h2[j]);
          h2[j] = fma2(q2[j], h2[j], mul2(p2[j], x2));
          r2[j] = fma2(q2[j], r2[j], x2);
          ag2[j] = fma2(d2, h2[j], ag2[j]);
          aq2[j] = fma2(d2, s2[j], aq2[j]);
          ap2[j] = fma2(d2, r2[j], ap2[j]);
        }
      }
    }
    if (__syncthreads_or(!ok)) {
      healthy = false;
      break;
    }
    if (tid == 0 && i + kS < nt) issue_a(i + kS);
  }
  if (!healthy) return;

  // gradients of the parameters (sum over the batch by atomic adds); lambda starts from the
  // gradient flowing into the returned state
  f32x2 lam2[kNP / 2];
#pragma unroll
  for (int j = 0; j < kNP / 2; ++j) {
    float dh[2] = {0.f, 0.f};
    float agv[2], aqv[2], apv[2], gv[2], sv[2], rv[2];
    unpack2(ag2[j], agv[0], agv[1]);
    unpack2(aq2[j], aqv[0], aqv[1]);
    unpack2(ap2[j], apv[0], apv[1]);
    unpack2(g2[j], gv[0], gv[1]);
    unpack2(s2[j], sv[0], sv[1]);
    unpack2(r2[j], rv[0], rv[1]);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int n = 2 * j + k;
      if (n < a.N) {
        if (a.dh_out) dh[k] = __ldg(a.dh_out + srow + n);
        if (valid) {
          atomicAdd(a.dg + (size_t)d * a.N + n, agv[k]);
          atomicAdd(a.dp + (size_t)d * a.N + n, fmaf(gv[k], apv[k], dh[k] * rv[k]));
          atomicAdd(a.dq + (size_t)d * a.N + n, fmaf(gv[k], aqv[k], dh[k] * sv[k]));
        }
      }
    }
    lam2[j] = pack2(dh[0], dh[1]);
  }
  if (valid) atomicAdd(a.domega + d, aw);

  // ---- pass B: backwards in time, input gradient -----------------------------------------------
  __syncthreads();  // every thread is done with the pass-A stages
  auto issue_b = [&](int k) {
    const int s = k % kS, i = nt - 1 - k;
    mbar_expect_tx(&full_b[s], C::kTileT);
    tma_load_3d(stages + (size_t)s * C::kStage + C::kTileT, &tmg, d0, i * kR, b, &full_b[s]);
  };
  if (tid == 0)
    for (int k = 0; k < kS && k < nt; ++k) issue_b(k);
  for (int k = 0; k < nt; ++k) {
    const int s = k % kS;
    const uint32_t ph = (uint32_t)((k / kS) & 1);
    const int i = nt - 1 - k;
    const int o = k & 1;
    const bool ok = mbar_wait(&full_b[s], ph);
    const T* gt = reinterpret_cast<const T*>(stages + (size_t)s * C::kStage + C::kTileT) + tid;
    T* ot = outs + (size_t)o * kR * kW + tid;
    const int rows = min(kR, L - i * kR);
#pragma unroll 4
    for (int rr = 0; rr < kR; ++rr) {
      const int r = kR - 1 - rr;
      if (r < rows) {
        const float dy = Elem<T>::ld_shared(gt + r * kW);
        const f32x2 d2 = pack2(dy, dy);
        f32x2 acc0 = pack2(0.f, 0.f), acc1 = pack2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kNP / 2; j += 2) {
          const f32x2 l0 = fma2(g2[j], d2, lam2[j]), l1 = fma2(g2[j + 1], d2, lam2[j + 1]);
          acc0 = fma2(p2[j], l0, acc0);
          acc1 = fma2(p2[j + 1], l1, acc1);
          lam2[j] = mul2(q2[j], l0);
          lam2[j + 1] = mul2(q2[j + 1], l1);
        }
        float lo, hi;
        unpack2(add2(acc0, acc1), lo, hi);
        const bool mk = kMask && mrow[i * kR + r] != 0;
        Elem<T>::st(ot + r * kW, fmaf(om, dy, mk ? 0.f : lo + hi));
      }
    }
    fence_proxy_async();
    if (tid == 0) bulk_wait_read<0>();
    if (__syncthreads_or(!ok)) break;
    if (tid == 0) {
      tma_store_3d(&tmd, d0, i * kR, b, outs + (size_t)o * kR * kW);
      bulk_commit();
      if (k + kS < nt) issue_b(k + kS);
    }
  }
  if (tid == 0) bulk_wait<0>();
  if (valid && a.dh_in) {
#pragma unroll
    for (int j = 0; j < kNP / 2; ++j) {
      float lo, hi;
      unpack2(lam2[j], lo, hi);
      if (2 * j < a.N) a.dh_in[srow + 2 * j] = lo;
      if (2 * j + 1 < a.N) a.dh_in[srow + 2 * j + 1] = hi;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// causal complex EMA.  Two threads per channel (8 complex poles each, two poles per packed
// register); the pair reads the same shared-memory element and joins its halves of dx by a shuffle.
// ---------------------------------------------------------------------------------------------
constexpr int kCT = 2 * kW;  // threads per CTA of the complex kernel
constexpr int kCP = 4;       // packed pole pairs per thread

template <typename T, bool kMask>
__global__ void __launch_bounds__(kCT) cema_bwd_stream_kernel(const __grid_constant__ CUtensorMap tmx,
                                                              const __grid_constant__ CUtensorMap tmg,
                                                              const __grid_constant__ CUtensorMap tmd,
                                                              EmaBwdStreamArgs a) {
  using C = EmaCfg<T>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full_a = reinterpret_cast<uint64_t*>(base);
  uint64_t* full_b = full_a + kS;
  unsigned char* stages = base + kHead;
  T* outs = reinterpret_cast<T*>(base + kHead + kS * C::kStage);

  const int tid = threadIdx.x;
  const int ch = tid >> 1, half = tid & 1;
  const int d0 = blockIdx.x * kW;
  const int b = blockIdx.y;
  const int d = d0 + ch;
  const bool valid = d < a.D;
  const int dc = valid ? d : a.D - 1;
  const int L = a.L;
  const int nt = (L + kR - 1) / kR;
  const unsigned char* mrow = kMask ? a.mask + (size_t)b * L : nullptr;

  if (tid == 0) {
    prefetch_tensormap(&tmx);
    prefetch_tensormap(&tmg);
    prefetch_tensormap(&tmd);
#pragma unroll
    for (int s = 0; s < kS; ++s) {
      mbar_init(&full_a[s], 1);
      mbar_init(&full_b[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  auto issue_a = [&](int i) {
    const int s = i % kS;
    unsigned char* st = stages + (size_t)s * C::kStage;
    mbar_expect_tx(&full_a[s], C::kStage);
    tma_load_3d(st, &tmx, d0, i * kR, b, &full_a[s]);
    tma_load_3d(st + C::kTileT, &tmg, d0, i * kR, b, &full_a[s]);
  };
  if (tid == 0)
    for (int i = 0; i < kS && i < nt; ++i) issue_a(i);

  f32x2 qr2[kCP], qi2[kCP], nqi2[kCP], p2[kCP], gr2[kCP], gi2[kCP];
  f32x2 hr2[kCP], hi2[kCP], sr2[kCP], si2[kCP], rr2[kCP], ri2[kCP];
  f32x2 ahr[kCP], ahi[kCP], asr[kCP], asi[kCP], arr[kCP], ari[kCP];
  const float om = __ldg(a.omega + dc);
  const f32x2 zero2 = pack2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < kCP; ++j) {
    float pv[2], qrv[2], qiv[2], grv[2], giv[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int n = half * 2 * kCP + 2 * j + k;
      pv[k] = qrv[k] = qiv[k] = grv[k] = giv[k] = 0.f;
      if (n < a.N) {
        const size_t c = (size_t)dc * a.N + n;
        pv[k] = __ldg(a.p + c);
        qrv[k] = __ldg(a.q + 2 * c);
        qiv[k] = __ldg(a.q + 2 * c + 1);
        grv[k] = __ldg(a.g + 2 * c);
        giv[k] = __ldg(a.g + 2 * c + 1);
      }
    }
    p2[j] = pack2(pv[0], pv[1]);
    qr2[j] = pack2(qrv[0], qrv[1]);
    qi2[j] = pack2(qiv[0], qiv[1]);
    nqi2[j] = pack2(-qiv[0], -qiv[1]);
    gr2[j] = pack2(grv[0], grv[1]);
    gi2[j] = pack2(giv[0], giv[1]);
    hr2[j] = hi2[j] = sr2[j] = si2[j] = rr2[j] = ri2[j] = zero2;
    ahr[j] = ahi[j] = asr[j] = asi[j] = arr[j] = ari[j] = zero2;
  }
  float aw = 0.f;

  // ---- pass A: forward in time ---------------------------------------------------------------
  bool healthy = true;
  for (int i = 0; i < nt; ++i) {
    const int s = i % kS;
    const uint32_t ph = (uint32_t)((i / kS) & 1);
    const bool ok = mbar_wait(&full_a[s], ph);
    const unsigned char* st = stages + (size_t)s * C::kStage;
    const T* xt = reinterpret_cast<const T*>(st) + ch;
    const T* gt = reinterpret_cast<const T*>(st + C::kTileT) + ch;
    const int rows = min(kR, L - i * kR);
#pragma unroll 2
    for (int r = 0; r < kR; ++r) {
      if (r < rows) {
        const float xr = Elem<T>::ld_shared(xt + r * kW), dy = Elem<T>::ld_shared(gt + r * kW);
        aw = fmaf(dy, xr, aw);
        const float xm = (kMask && mrow[i * kR + r] != 0) ? 0.f : xr;
        const f32x2 x2 = pack2(xm, xm), d2 = pack2(dy, dy);
#pragma unroll
        for (int j = 0; j < kCP; ++j) {
          const f32x2 nsr = fma2(qr2[j], sr2[j], fma2(nqi2[j], si2[j], hr2[j]));
          const f32x2 nsi = fma2(qi2[j], sr2[j], fma2(qr2[j], si2[j], hi2[j]));
          const f32x2 nhr = fma2(qr2[j], hr2[j], fma2(nqi2[j], hi2[j], mul2(p2[j], x2)));
          const f32x2 nhi = fma2(qi2[j], hr2[j], mul2(qr2[j], hi2[j]));
          const f32x2 nrr = fma2(qr2[j], rr2[j], fma2(nqi2[j], ri2[j], x2));
          const f32x2 nri = fma2(qi2[j], rr2[j], mul2(qr2[j], ri2[j]));
          sr2[j] = nsr; si2[j] = nsi; hr2[j] = nhr; hi2[j] = nhi; rr2[j] = nrr; ri2[j] = nri;
          ahr[j] = fma2(d2, nhr, ahr[j]); ahi[j] = fma2(d2, nhi, ahi[j]);
          asr[j] = fma2(d2, nsr, asr[j]); asi[j] = fma2(d2, nsi, asi[j]);
          arr[j] = fma2(d2, nrr, arr[j]); ari[j] = fma2(d2, nri, ari[j]);
        }
      }
    }
    if (__syncthreads_or(!ok)) {
      healthy = false;
      break;
    }
    if (tid == 0 && i + kS < nt) issue_a(i + kS);
  }
  if (!healthy) return;

  f32x2 lr2[kCP], li2[kCP];
#pragma unroll
  for (int j = 0; j < kCP; ++j) {
    float v[12];
    unpack2(ahr[j], v[0], v[1]); unpack2(ahi[j], v[2], v[3]); unpack2(asr[j], v[4], v[5]);
    unpack2(asi[j], v[6], v[7]); unpack2(arr[j], v[8], v[9]); unpack2(ari[j], v[10], v[11]);
    float grv[2], giv[2];
    unpack2(gr2[j], grv[0], grv[1]);
    unpack2(gi2[j], giv[0], giv[1]);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int n = half * 2 * kCP + 2 * j + k;
      if (n < a.N && valid) {
        const size_t c = (size_t)d * a.N + n;
        atomicAdd(a.dg + 2 * c, v[0 + k]);
        atomicAdd(a.dg + 2 * c + 1, -v[2 + k]);
        atomicAdd(a.dp + c, grv[k] * v[8 + k] - giv[k] * v[10 + k]);
        atomicAdd(a.dq + 2 * c, grv[k] * v[4 + k] - giv[k] * v[6 + k]);
        atomicAdd(a.dq + 2 * c + 1, -(grv[k] * v[6 + k] + giv[k] * v[4 + k]));
      }
    }
    lr2[j] = li2[j] = zero2;
  }
  if (valid && half == 0) atomicAdd(a.domega + d, aw);

  // ---- pass B: backwards in time ---------------------------------------------------------------
  __syncthreads();
  auto issue_b = [&](int k) {
    const int s = k % kS, i = nt - 1 - k;
    mbar_expect_tx(&full_b[s], C::kTileT);
    tma_load_3d(stages + (size_t)s * C::kStage + C::kTileT, &tmg, d0, i * kR, b, &full_b[s]);
  };
  if (tid == 0)
    for (int k = 0; k < kS && k < nt; ++k) issue_b(k);
  for (int k = 0; k < nt; ++k) {
    const int s = k % kS;
    const uint32_t ph = (uint32_t)((k / kS) & 1);
    const int i = nt - 1 - k;
    const int o = k & 1;
    const bool ok = mbar_wait(&full_b[s], ph);
    const T* gt = reinterpret_cast<const T*>(stages + (size_t)s * C::kStage + C::kTileT) + ch;
    T* ot = outs + (size_t)o * kR * kW + ch;
    const int rows = min(kR, L - i * kR);
#pragma unroll 4
    for (int rr = 0; rr < kR; ++rr) {
      const int r = kR - 1 - rr;
      if (r < rows) {
        const float dy = Elem<T>::ld_shared(gt + r * kW);
        const f32x2 d2 = pack2(dy, dy);
        f32x2 acc = zero2;
#pragma unroll
        for (int j = 0; j < kCP; ++j) {
          const f32x2 cr = fma2(gr2[j], d2, lr2[j]), ci = fma2(gi2[j], d2, li2[j]);
          acc = fma2(p2[j], cr, acc);
          lr2[j] = fma2(qr2[j], cr, mul2(nqi2[j], ci));
          li2[j] = fma2(qi2[j], cr, mul2(qr2[j], ci));
        }
        float lo, hi;
        unpack2(acc, lo, hi);
        float part = lo + hi;
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        const bool mk = kMask && mrow[i * kR + r] != 0;
        if (half == 0) Elem<T>::st(ot + r * kW, fmaf(om, dy, mk ? 0.f : part));
      }
    }
    fence_proxy_async();
    if (tid == 0) bulk_wait_read<0>();
    if (__syncthreads_or(!ok)) break;
    if (tid == 0) {
      tma_store_3d(&tmd, d0, i * kR, b, outs + (size_t)o * kR * kW);
      bulk_commit();
      if (k + kS < nt) issue_b(k + kS);
    }
  }
  if (tid == 0) bulk_wait<0>();
}

template <typename K>
static bool set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
}

}  // namespace

bool tsn_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                        long long gsd, long long xsb, long long xsl, long long xsd, long long dsb, long long dsl,
                        long long dsd, const float* cummean, const float* cumrstd, const TsnBwdStreamArgs& a,
                        cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (gsd != 1 || xsd != 1 || dsd != 1 || a.B > 65535 || a.D < 8) return false;
  CUtensorMap tx, tg, td, tm, tr;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&tg, dtype, dy, a.D, a.L, a.B, gsl, gsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&td, dtype, dx, a.D, a.L, a.B, dsl, dsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&tm, MEGA_F32, cummean, a.D, a.L, a.B, a.D, (long long)a.L * a.D, kW, kR + 1, 1,
                          CU_TENSOR_MAP_SWIZZLE_NONE))
    return false;
  if (!make_tensor_map_3d(&tr, MEGA_F32, cumrstd, a.D, a.L, a.B, a.D, (long long)a.L * a.D, kW, kR, 1,
                          CU_TENSOR_MAP_SWIZZLE_NONE))
    return false;
  dim3 grid((a.D + kW - 1) / kW, a.B);
  bool ok = true;
  switch (dtype) {
#define MEGA_TSN_BWD_CASE(DT, TY)                                                                  \
  case DT: {                                                                                       \
    static std::once_flag once;                                                                    \
    static bool attr_ok = true;                                                                    \
    std::call_once(once, [&] {                                                                     \
      attr_ok = set_smem(tsn_bwd_stream_kernel<TY, true>, TsnCfg<TY>::kSmem) &&                    \
                set_smem(tsn_bwd_stream_kernel<TY, false>, TsnCfg<TY>::kSmem);                     \
    });                                                                                            \
    if (!attr_ok) { cudaGetLastError(); return false; }                                            \
    if (a.mask) launch(tsn_bwd_stream_kernel<TY, true>, grid, dim3(kW), (size_t)TsnCfg<TY>::kSmem, (void*)s, tx, \
                       tg, td, tm, tr, a);                                                         \
    else launch(tsn_bwd_stream_kernel<TY, false>, grid, dim3(kW), (size_t)TsnCfg<TY>::kSmem, (void*)s, tx, tg, \
                td, tm, tr, a);                                                                    \
  } break;
    MEGA_TSN_BWD_CASE(MEGA_F32, float)
    MEGA_TSN_BWD_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_TSN_BWD_CASE(MEGA_F16, __half)
#undef MEGA_TSN_BWD_CASE
    default: ok = false;
  }
  return ok;
}

bool ema_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                        long long gsd, long long xsb, long long xsl, long long xsd, long long dsb, long long dsl,
                        long long dsd, const EmaBwdStreamArgs& a, cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (gsd != 1 || xsd != 1 || dsd != 1 || a.B > 65535 || a.D < 8 || a.N > kNP) return false;
  CUtensorMap tx, tg, td;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&tg, dtype, dy, a.D, a.L, a.B, gsl, gsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&td, dtype, dx, a.D, a.L, a.B, dsl, dsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  dim3 grid((a.D + kW - 1) / kW, a.B);
  bool ok = true;
  switch (dtype) {
#define MEGA_EMA_BWD_CASE(DT, TY)                                                                  \
  case DT: {                                                                                       \
    static std::once_flag once;                                                                    \
    static bool attr_ok = true;                                                                    \
    std::call_once(once, [&] {                                                                     \
      attr_ok = set_smem(ema_bwd_stream_kernel<TY, true>, EmaCfg<TY>::kSmem) &&                    \
                set_smem(ema_bwd_stream_kernel<TY, false>, EmaCfg<TY>::kSmem);                     \
    });                                                                                            \
    if (!attr_ok) { cudaGetLastError(); return false; }                                            \
    if (a.mask) launch(ema_bwd_stream_kernel<TY, true>, grid, dim3(kW), (size_t)EmaCfg<TY>::kSmem, (void*)s, tx, \
                       tg, td, a);                                                                 \
    else launch(ema_bwd_stream_kernel<TY, false>, grid, dim3(kW), (size_t)EmaCfg<TY>::kSmem, (void*)s, tx, tg,   \
                td, a);                                                                            \
  } break;
    MEGA_EMA_BWD_CASE(MEGA_F32, float)
    MEGA_EMA_BWD_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_EMA_BWD_CASE(MEGA_F16, __half)
#undef MEGA_EMA_BWD_CASE
    default: ok = false;
  }
  return ok;
}

bool cema_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                         long long gsd, long long xsb, long long xsl, long long xsd, long long dsb, long long dsl,
                         long long dsd, const EmaBwdStreamArgs& a, cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (gsd != 1 || xsd != 1 || dsd != 1 || a.B > 65535 || a.D < 8 || a.N > 4 * kCP) return false;
  CUtensorMap tx, tg, td;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&tg, dtype, dy, a.D, a.L, a.B, gsl, gsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&td, dtype, dx, a.D, a.L, a.B, dsl, dsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  dim3 grid((a.D + kW - 1) / kW, a.B);
  bool ok = true;
  switch (dtype) {
#define MEGA_CEMA_BWD_CASE(DT, TY)                                                                 \
  case DT: {                                                                                       \
    static std::once_flag once;                                                                    \
    static bool attr_ok = true;                                                                    \
    std::call_once(once, [&] {                                                                     \
      attr_ok = set_smem(cema_bwd_stream_kernel<TY, true>, EmaCfg<TY>::kSmem) &&                   \
                set_smem(cema_bwd_stream_kernel<TY, false>, EmaCfg<TY>::kSmem);                    \
    });                                                                                            \
    if (!attr_ok) { cudaGetLastError(); return false; }                                            \
    if (a.mask) launch(cema_bwd_stream_kernel<TY, true>, grid, dim3(kCT), (size_t)EmaCfg<TY>::kSmem, (void*)s, \
                       tx, tg, td, a);                                                             \
    else launch(cema_bwd_stream_kernel<TY, false>, grid, dim3(kCT), (size_t)EmaCfg<TY>::kSmem, (void*)s, tx,  \
                tg, td, a);                                                                        \
  } break;
    MEGA_CEMA_BWD_CASE(MEGA_F32, float)
    MEGA_CEMA_BWD_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_CEMA_BWD_CASE(MEGA_F16, __half)
#undef MEGA_CEMA_BWD_CASE
    default: ok = false;
  }
  return ok;
}

cudaError_t stream_bwd_read_device_error(int* v, bool reset) { return read_device_error(v, reset); }

}  // namespace mega
