// Streamed grouped TimestepNorm (forward and backward) for channel-contiguous activations.
//
// The grouped norm pools the statistics of the D / G channels of a group at every step, then
// combines them over time.  Only that combination is serial, and it is tiny (one value per step
// and group), so a tile of kR steps is handled in three phases: (1) all (step, group) moments of
// the tile in parallel — a warp per row, lanes across channels, shuffle reductions; (2) one thread
// per group walks the kR steps of the running Welford combination; (3) one thread per channel
// normalises.  Tiles move through the same TMA ring as the other streamed kernels.  Group sizes
// 8, 16, 32 or 64 channels (a CTA owns 64 channels = whole groups); other sizes use the generic
// kernel.
#include <mutex>

#include "common.cuh"
#include "stream_bwd.cuh"
#include "tma.cuh"

namespace mega {

namespace {

constexpr int kW = 64;  // channels per CTA (= threads)
constexpr int kR = 32;  // timesteps per tile
constexpr int kS = 3;   // ring depth
constexpr int kMaxG = 8;  // groups per CTA at the smallest group size
constexpr int kHead = 128;

// sum over the lanes of a group: segments of `width` lanes (width = min(gs, 32))
__device__ __forceinline__ float seg_sum(float v, int width) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    if (o < width) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
struct GCfg {
  static constexpr int kTileT = kR * kW * (int)sizeof(T);
  // forward: x ring + 2 output tiles; backward: (x, dy) ring + 2 output tiles
  static constexpr int kSmemFwd = kHead + kS * kTileT + 2 * kTileT + 128;
  static constexpr int kSmemBwd = kHead + kS * 2 * kTileT + 2 * kTileT + 128;
};

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
template <typename T, bool kMask, bool kSave>
__global__ void __launch_bounds__(kW) tsn_group_stream_kernel(const __grid_constant__ CUtensorMap tmx,
                                                              const __grid_constant__ CUtensorMap tmy,
                                                              GroupStreamArgs a) {
  using C = GCfg<T>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full = reinterpret_cast<uint64_t*>(base);
  T* xs = reinterpret_cast<T*>(base + kHead);
  T* ys = reinterpret_cast<T*>(base + kHead + kS * C::kTileT);
  __shared__ float gmean[kR][kMaxG], gvar[kR][kMaxG];   // moments of (row, group); then mean / rstd to apply

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int d0 = blockIdx.x * kW;
  const int b = blockIdx.y;
  const int d = d0 + tid;
  const bool valid = d < a.D;
  const int dc = valid ? d : a.D - 1;
  const int L = a.L;
  const int nt = (L + kR - 1) / kR;
  const int gs = a.D / a.G;
  const int ng = kW / gs;          // groups per CTA
  const int g0 = d0 / gs;          // first group of this CTA
  const int width = gs < 32 ? gs : 32;
  const float inv_gs = 1.f / (float)gs;

  if (tid == 0) {
    prefetch_tensormap(&tmx);
    prefetch_tensormap(&tmy);
#pragma unroll
    for (int s = 0; s < kS; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0)
    for (int i = 0; i < kS && i < nt; ++i) {
      mbar_expect_tx(&full[i], C::kTileT);
      tma_load_3d(xs + (size_t)i * kR * kW, &tmx, d0, i * kR, b, &full[i]);
    }

  const float w = __ldg(a.gamma + dc), bb = __ldg(a.beta + dc);
  const int my_g = tid / gs;       // group (within the CTA) of this thread's channel
  // phase-2 threads (tid < ng) carry the running statistics of group g0 + tid
  const bool owner = tid < ng && g0 + tid < a.G;
  float mean = 0.f, var = 1.f;
  int seen = 0;
  const long long cnt0 = a.prev_count[b];
  const float cnt0f = (float)cnt0;
  if (owner) {
    mean = a.prev_mean[(size_t)b * a.G + g0 + tid];
    var = a.prev_var[(size_t)b * a.G + g0 + tid];
  }
  const unsigned char* mrow = kMask ? a.mask + (size_t)b * L : nullptr;

  for (int i = 0; i < nt; ++i) {
    const int s = i % kS;
    const uint32_t ph = (uint32_t)((i / kS) & 1);
    const int o = i & 1;
    const bool ok = mbar_wait(&full[s], ph);
    const T* xt = xs + (size_t)s * kR * kW;
    T* yt = ys + (size_t)o * kR * kW;
    const int rows = min(kR, L - i * kR);
    // ---- phase 1: moments of every (row, group) of the tile ------------------------------------
    for (int r = warp; r < rows; r += kW / 32) {
      const float x0 = Elem<T>::ld_shared(xt + r * kW + lane), x1 = Elem<T>::ld_shared(xt + r * kW + 32 + lane);
      float m0, m1v;
      if (gs == 64) {
        m0 = m1v = seg_sum(x0 + x1, 32) * inv_gs;
      } else {
        m0 = seg_sum(x0, width) * inv_gs;
        m1v = seg_sum(x1, width) * inv_gs;
      }
      const float e0 = x0 - m0, e1 = x1 - m1v;
      float v0, v1;
      if (gs == 64) {
        v0 = v1 = seg_sum(e0 * e0 + e1 * e1, 32) * inv_gs;
      } else {
        v0 = seg_sum(e0 * e0, width) * inv_gs;
        v1 = seg_sum(e1 * e1, width) * inv_gs;
      }
      if ((lane & (width - 1)) == 0) {
        if (gs == 64) {
          gmean[r][0] = m0;
          gvar[r][0] = v0;
        } else {
          const int ga = lane / gs, gb = (32 + lane) / gs;
          gmean[r][ga] = m0;
          gvar[r][ga] = v0;
          gmean[r][gb] = m1v;
          gvar[r][gb] = v1;
        }
      }
    }
    __syncthreads();
    // ---- phase 2: running combination over the rows, one thread per group ---------------------
    if (owner) {
      for (int r = 0; r < rows; ++r) {
        const int t = i * kR + r;
        const float gm = gmean[r][tid], gv = gvar[r][tid];
        // WelfordCombine(count, mean, var, 1, gm, gv)  (fairseq/csrc/utils.h:67-76)
        const float cprev = cnt0f + (float)seen;
        const float c2 = rcp_approx(cprev + 1.f), c1 = cprev * c2;
        const float dl = gm - mean;
        const float m1 = c1 * mean + c2 * gm;
        const float m2 = c1 * var + c2 * gv + (c1 * dl) * (c2 * dl);
        const float rstd = rsqrt_approx(m2 + a.eps);
        const bool mk = kMask && mrow[t] != 0;
        if (!mk) {
          mean = m1;
          var = m2;
          ++seen;
        }
        gmean[r][tid] = m1;                     // what phase 3 applies
        gvar[r][tid] = mk ? -1.f : rstd;        // negative: padded step
        if (kSave) {
          const size_t idx = ((size_t)b * L + t) * a.G + g0 + tid;
          a.group_mean[idx] = gm;
          a.cummean[idx] = mean;
          a.cumrstd[idx] = rstd;
        }
      }
    }
    __syncthreads();
    // ---- phase 3: normalise, one thread per channel ------------------------------------------
#pragma unroll 8
    for (int r = 0; r < kR; ++r) {
      if (r < rows) {
        const float m1 = gmean[r][my_g], rs = gvar[r][my_g];
        const float xv = Elem<T>::ld_shared(xt + r * kW + tid);
        Elem<T>::st(yt + r * kW + tid, rs < 0.f ? 0.f : fmaf((xv - m1) * rs, w, bb));
      }
    }
    fence_proxy_async();
    if (tid == 0) bulk_wait_read<0>();
    if (__syncthreads_or(!ok)) break;
    if (tid == 0) {
      tma_store_3d(&tmy, d0, i * kR, b, yt);
      bulk_commit();
      if (i + kS < nt) {
        mbar_expect_tx(&full[s], C::kTileT);
        tma_load_3d(xs + (size_t)s * kR * kW, &tmx, d0, (i + kS) * kR, b, &full[s]);
      }
    }
  }
  if (tid == 0) bulk_wait<0>();
  if (owner) {
    a.mean_out[(size_t)b * a.G + g0 + tid] = mean;
    a.var_out[(size_t)b * a.G + g0 + tid] = var;
    if (g0 + tid == 0) a.count_out[b] = cnt0 + seen;
  }
}

// ---------------------------------------------------------------------------------------------
// backward (fairseq/csrc/ops/timestep_norm.cc:318-446), tiles walked from the end
// ---------------------------------------------------------------------------------------------
template <typename T, bool kMask>
__global__ void __launch_bounds__(kW) tsn_group_bwd_stream_kernel(const __grid_constant__ CUtensorMap tmx,
                                                                  const __grid_constant__ CUtensorMap tmg,
                                                                  const __grid_constant__ CUtensorMap tmd,
                                                                  GroupStreamBwdArgs a) {
  using C = GCfg<T>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full = reinterpret_cast<uint64_t*>(base);
  unsigned char* stages = base + kHead;                        // [kS][x tile, dy tile]
  T* outs = reinterpret_cast<T*>(base + kHead + kS * 2 * C::kTileT);
  __shared__ float su[kR + 1][kMaxG];                          // cummean of steps t0-1 .. t0+kR-1
  __shared__ float sr[kR][kMaxG], sx[kR][kMaxG];               // cumrstd, group_mean
  __shared__ float sds[kR][kMaxG], sdb[kR][kMaxG];             // reductions; then dux, dvx
  __shared__ float scf[kR];                                    // per row: 1 / count, < 0: padded

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int d0 = blockIdx.x * kW;
  const int b = blockIdx.y;
  const int d = d0 + tid;
  const bool valid = d < a.D;
  const int dc = valid ? d : a.D - 1;
  const int L = a.L;
  const int nt = (L + kR - 1) / kR;
  const int gs = a.D / a.G;
  const int ng = kW / gs;
  const int g0 = d0 / gs;
  const int width = gs < 32 ? gs : 32;
  const float cg = 1.f / (float)gs;

  auto issue = [&](int k) {
    const int s = k % kS, i = nt - 1 - k;
    unsigned char* st = stages + (size_t)s * 2 * C::kTileT;
    mbar_expect_tx(&full[s], 2 * C::kTileT);
    tma_load_3d(st, &tmx, d0, i * kR, b, &full[s]);
    tma_load_3d(st + C::kTileT, &tmg, d0, i * kR, b, &full[s]);
  };
  if (tid == 0) {
    prefetch_tensormap(&tmx);
    prefetch_tensormap(&tmg);
    prefetch_tensormap(&tmd);
#pragma unroll
    for (int s = 0; s < kS; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0)
    for (int k = 0; k < kS && k < nt; ++k) issue(k);

  const float w = valid ? __ldg(a.gamma + dc) : 0.f;
  // lanes of phase 1 need the scale of both channels they read
  const float w0 = (d0 + lane < a.D) ? __ldg(a.gamma + d0 + lane) : 0.f;
  const float w1 = (d0 + 32 + lane < a.D) ? __ldg(a.gamma + d0 + 32 + lane) : 0.f;
  const int my_g = tid / gs;
  const bool owner = tid < ng && g0 + tid < a.G;
  float ug = 0.f, vg = 0.f;
  if (owner) {
    ug = a.dmean ? a.dmean[(size_t)b * a.G + g0 + tid] : 0.f;
    vg = a.dvar ? a.dvar[(size_t)b * a.G + g0 + tid] : 0.f;
  }
  float wg = 0.f, bg = 0.f;
  long long cnt_run = a.count[b];  // count after the last step of the current tile
  const unsigned char* mrow = kMask ? a.mask + (size_t)b * L : nullptr;

  for (int k = 0; k < nt; ++k) {
    const int s = k % kS;
    const uint32_t ph = (uint32_t)((k / kS) & 1);
    const int i = nt - 1 - k;
    const int o = k & 1;
    const int t0 = i * kR;
    const int rows = min(kR, L - t0);
    // saved statistics of the tile (small: one value per step and group) and the step counts
    for (int idx = tid; idx < (kR + 1) * ng; idx += kW) {
      const int r = idx / ng, g = idx % ng;       // r = 0 is step t0 - 1
      const int t = t0 - 1 + r;
      float v = 0.f;
      if (g0 + g < a.G) {
        if (t < 0) v = a.prev_mean[(size_t)b * a.G + g0 + g];
        else if (t < L) v = __ldg(a.cummean + ((size_t)b * L + t) * a.G + g0 + g);
      }
      su[r][g] = v;
      if (r < kR) {
        const int tt = t0 + r;
        const bool in = tt < L && g0 + g < a.G;
        sr[r][g] = in ? __ldg(a.cumrstd + ((size_t)b * L + tt) * a.G + g0 + g) : 0.f;
        sx[r][g] = in ? __ldg(a.group_mean + ((size_t)b * L + tt) * a.G + g0 + g) : 0.f;
      }
    }
    if (tid < 32) {  // counts, walking backwards: lane r = step t0 + r
      const int t = t0 + tid;
      const bool masked = (t >= L) || (kMask && mrow[t] != 0);
      const unsigned vmask = __ballot_sync(0xffffffffu, !masked);
      const unsigned later = tid == 31 ? 0u : (vmask & (0xffffffffu << (tid + 1)));
      scf[tid] = masked ? -1.f : (float)(cnt_run - __popc(later));   // the count itself (>= 1)
      cnt_run -= __popc(vmask);
    }
    const bool ok = mbar_wait(&full[s], ph);
    __syncthreads();
    const unsigned char* st = stages + (size_t)s * 2 * C::kTileT;
    const T* xt = reinterpret_cast<const T*>(st);
    const T* gt = reinterpret_cast<const T*>(st + C::kTileT);
    T* ot = outs + (size_t)o * kR * kW;
    // ---- phase 1: ds = sum dy (x - u) w, db = sum dy w over the channels of each (row, group) --
    for (int r = warp; r < rows; r += kW / 32) {
      const float x0 = Elem<T>::ld_shared(xt + r * kW + lane), x1 = Elem<T>::ld_shared(xt + r * kW + 32 + lane);
      const float y0 = Elem<T>::ld_shared(gt + r * kW + lane), y1 = Elem<T>::ld_shared(gt + r * kW + 32 + lane);
      const int ga = gs == 64 ? 0 : lane / gs, gb = gs == 64 ? 0 : (32 + lane) / gs;
      const float p0 = y0 * w0, p1 = y1 * w1;
      const float a0 = p0 * (x0 - su[r + 1][ga]), a1 = p1 * (x1 - su[r + 1][gb]);
      float ds0, ds1, db0, db1;
      if (gs == 64) {
        ds0 = ds1 = seg_sum(a0 + a1, 32);
        db0 = db1 = seg_sum(p0 + p1, 32);
      } else {
        ds0 = seg_sum(a0, width);
        ds1 = seg_sum(a1, width);
        db0 = seg_sum(p0, width);
        db1 = seg_sum(p1, width);
      }
      if ((lane & (width - 1)) == 0) {
        sds[r][ga] = ds0;
        sdb[r][ga] = db0;
        if (gs != 64) {
          sds[r][gb] = ds1;
          sdb[r][gb] = db1;
        }
      }
    }
    __syncthreads();
    // ---- phase 2: reverse walk of the statistics' gradients, one thread per group --------------
    if (owner) {
      for (int r = rows - 1; r >= 0; --r) {
        const float cnt = scf[r];
        if (cnt < 0.f) {
          sds[r][tid] = 0.f;
          sdb[r][tid] = 0.f;
          continue;
        }
        const float c2 = 1.f / cnt, c1 = (cnt - 1.f) * c2;
        const float rs = sr[r][tid], ux = sx[r][tid], pu = su[r][tid];
        const float du = ug - rs * sdb[r][tid];
        const float dv = vg - 0.5f * (rs * rs * rs) * sds[r][tid];
        const float cross = 2.f * c1 * c2 * dv * (ux - pu);
        sds[r][tid] = c2 * du + cross;   // dux
        sdb[r][tid] = c2 * dv;           // dvx
        ug = c1 * du - cross;
        vg = c1 * dv;
      }
    }
    __syncthreads();
    // ---- phase 3: dx and the per-channel sums, one thread per channel ---------------------------
#pragma unroll 8
    for (int r = 0; r < kR; ++r) {
      if (r < rows) {
        const bool mk = scf[r] < 0.f;
        const float x = Elem<T>::ld_shared(xt + r * kW + tid), dy = Elem<T>::ld_shared(gt + r * kW + tid);
        const float rs = sr[r][my_g], ux = sx[r][my_g], u = su[r + 1][my_g];
        const float dx = dy * rs * w + sds[r][my_g] * cg + 2.f * sdb[r][my_g] * cg * (x - ux);
        Elem<T>::st(ot + r * kW + tid, mk ? 0.f : dx);
        wg = mk ? wg : fmaf(dy * (x - u), rs, wg);
        bg = mk ? bg : bg + dy;
      }
    }
    fence_proxy_async();
    if (tid == 0) bulk_wait_read<0>();
    if (__syncthreads_or(!ok)) break;
    if (tid == 0) {
      tma_store_3d(&tmd, d0, t0, b, ot);
      bulk_commit();
      if (k + kS < nt) issue(k + kS);
    }
  }
  if (tid == 0) bulk_wait<0>();
  if (owner) {
    a.dprev_mean[(size_t)b * a.G + g0 + tid] = ug;
    a.dprev_var[(size_t)b * a.G + g0 + tid] = vg;
  }
  if (valid) {
    atomicAdd(a.dgamma + d, wg);
    atomicAdd(a.dbeta + d, bg);
  }
}

template <typename K>
static bool set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
}

static bool group_size_ok(int D, int G) {
  if (G <= 0 || D % G != 0) return false;
  const int gs = D / G;
  return gs == 8 || gs == 16 || gs == 32 || gs == 64;
}

}  // namespace

bool tsn_group_stream_try(int dtype, const void* x, void* y, long long xsb, long long xsl, long long xsd,
                          long long ysb, long long ysl, long long ysd, const GroupStreamArgs& a, cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (xsd != 1 || ysd != 1 || a.B > 65535 || !group_size_ok(a.D, a.G) || x == y) return false;
  CUtensorMap tx, ty;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&ty, dtype, y, a.D, a.L, a.B, ysl, ysb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  dim3 grid((a.D + kW - 1) / kW, a.B);
  const bool save = a.cummean != nullptr;
  switch (dtype) {
#define MEGA_GROUP_FWD_CASE(DT, TY)                                                                     \
  case DT: {                                                                                            \
    static std::once_flag once;                                                                         \
    static bool attr_ok = true;                                                                         \
    std::call_once(once, [&] {                                                                          \
      attr_ok = set_smem(tsn_group_stream_kernel<TY, true, true>, GCfg<TY>::kSmemFwd) &&                \
                set_smem(tsn_group_stream_kernel<TY, true, false>, GCfg<TY>::kSmemFwd) &&               \
                set_smem(tsn_group_stream_kernel<TY, false, true>, GCfg<TY>::kSmemFwd) &&               \
                set_smem(tsn_group_stream_kernel<TY, false, false>, GCfg<TY>::kSmemFwd);                \
    });                                                                                                 \
    if (!attr_ok) { cudaGetLastError(); return false; }                                                 \
    const size_t sm = (size_t)GCfg<TY>::kSmemFwd;                                                       \
    if (a.mask && save) launch(tsn_group_stream_kernel<TY, true, true>, grid, dim3(kW), sm, (void*)s, tx, ty, a);   \
    else if (a.mask) launch(tsn_group_stream_kernel<TY, true, false>, grid, dim3(kW), sm, (void*)s, tx, ty, a);     \
    else if (save) launch(tsn_group_stream_kernel<TY, false, true>, grid, dim3(kW), sm, (void*)s, tx, ty, a);       \
    else launch(tsn_group_stream_kernel<TY, false, false>, grid, dim3(kW), sm, (void*)s, tx, ty, a);    \
  } break;
    MEGA_GROUP_FWD_CASE(MEGA_F32, float)
    MEGA_GROUP_FWD_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_GROUP_FWD_CASE(MEGA_F16, __half)
#undef MEGA_GROUP_FWD_CASE
    default: return false;
  }
  return true;
}

bool tsn_group_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                              long long gsd, long long xsb, long long xsl, long long xsd, long long dsb,
                              long long dsl, long long dsd, const GroupStreamBwdArgs& a, cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (gsd != 1 || xsd != 1 || dsd != 1 || a.B > 65535 || !group_size_ok(a.D, a.G)) return false;
  CUtensorMap tx, tg, td;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&tg, dtype, dy, a.D, a.L, a.B, gsl, gsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  if (!make_tensor_map_3d(&td, dtype, dx, a.D, a.L, a.B, dsl, dsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
  dim3 grid((a.D + kW - 1) / kW, a.B);
  switch (dtype) {
#define MEGA_GROUP_BWD_CASE(DT, TY)                                                                     \
  case DT: {                                                                                            \
    static std::once_flag once;                                                                         \
    static bool attr_ok = true;                                                                         \
    std::call_once(once, [&] {                                                                          \
      attr_ok = set_smem(tsn_group_bwd_stream_kernel<TY, true>, GCfg<TY>::kSmemBwd) &&                  \
                set_smem(tsn_group_bwd_stream_kernel<TY, false>, GCfg<TY>::kSmemBwd);                   \
    });                                                                                                 \
    if (!attr_ok) { cudaGetLastError(); return false; }                                                 \
    const size_t sm = (size_t)GCfg<TY>::kSmemBwd;                                                       \
    if (a.mask) launch(tsn_group_bwd_stream_kernel<TY, true>, grid, dim3(kW), sm, (void*)s, tx, tg, td, a);  \
    else launch(tsn_group_bwd_stream_kernel<TY, false>, grid, dim3(kW), sm, (void*)s, tx, tg, td, a);   \
  } break;
    MEGA_GROUP_BWD_CASE(MEGA_F32, float)
    MEGA_GROUP_BWD_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_GROUP_BWD_CASE(MEGA_F16, __half)
#undef MEGA_GROUP_BWD_CASE
    default: return false;
  }
  return true;
}

cudaError_t stream_group_read_device_error(int* v, bool reset) { return read_device_error(v, reset); }

}  // namespace mega
