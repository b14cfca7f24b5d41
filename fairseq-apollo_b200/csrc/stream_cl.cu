// Streamed channel-contiguous kernels: TimestepNorm, causal EMA, or both fused, for activations
// whose channel stride is 1 ((B, L, D) and time-major (L, B, D) memory).
//
// One CTA owns kW adjacent channels of one sequence and walks the sequence in tiles of kR
// timesteps.  Tiles arrive through a kS-deep TMA ring (cp.async.bulk.tensor + mbarrier), results
// leave through TMA stores from a double-buffered staging tile, so HBM sees whole 128 B / 256 B
// row segments while every thread keeps its channel's Welford state and pole states in registers.
// The pole update and the output projection use packed fp32x2 FMAs.
#include <mutex>

#include "common.cuh"
#include "tma.cuh"
#include "stream_cl.cuh"
#include "stream_bwd.cuh"

namespace mega {

// ---------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    cudaGetLastError();
  });
  return fn;
}

bool make_tensor_map_3d(CUtensorMap* out, int dtype, const void* base, uint64_t dim0, uint64_t dim1,
                        uint64_t dim2, int64_t stride1, int64_t stride2, uint32_t box0, uint32_t box1,
                        uint32_t box2, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const int es = elem_size(dtype);
  if (!aligned_to(base, 16)) return false;
  if (stride1 <= 0 || stride2 <= 0) return false;
  if ((stride1 * es) % 16 != 0 || (stride2 * es) % 16 != 0) return false;
  if ((uint64_t)box0 * es % 16 != 0 || box0 > 256 || box1 > 256 || box2 > 256) return false;
  CUtensorMapDataType dt = dtype == MEGA_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == MEGA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[3] = {dim0, dim1, dim2};
  cuuint64_t strides[2] = {(cuuint64_t)stride1 * es, (cuuint64_t)stride2 * es};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------

constexpr int kW = 64;  // channels per CTA (= threads)
constexpr int kR = 32;  // timesteps per tile
constexpr int kNP = 16; // poles held in registers (ndim <= 16, padded with inert poles)

template <typename T>
struct StreamCfg {
  static constexpr int kS = sizeof(T) == 2 ? 4 : 3;  // input ring depth
  static constexpr int kTile = kR * kW * (int)sizeof(T);
  static constexpr int kHead = 512;  // coefficient double buffer + barriers, keeps tiles 128 B aligned
  static constexpr int kTileF = kR * kW * 4;  // fp32 tiles of the training saves
  static constexpr int smem_bytes(bool has_xn, bool save = false) {
    return kHead + kTile * (kS + 2 + (has_xn ? 2 : 0)) + (save ? 4 * kTileF : 0) + 128;
  }
};

template <typename T, bool kNorm, bool kEma, bool kState, bool kCplx, bool kSave>
__global__ void __launch_bounds__(kW) stream_cl_kernel(const __grid_constant__ CUtensorMap tmx,
                                                       const __grid_constant__ CUtensorMap tmy,
                                                       const __grid_constant__ CUtensorMap tmn,
                                                       const __grid_constant__ CUtensorMap tmm,
                                                       const __grid_constant__ CUtensorMap tmr, StreamArgs a) {
  constexpr int kS = StreamCfg<T>::kS;
  constexpr int kTile = StreamCfg<T>::kTile;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  constexpr int kHead = StreamCfg<T>::kHead;
  float* cbuf = reinterpret_cast<float*>(base);                        // [2][kR]
  uint64_t* full = reinterpret_cast<uint64_t*>(base + 2 * kR * 4);     // [kS]
  T* xs = reinterpret_cast<T*>(base + kHead);                          // [kS][kR][kW]
  T* ys = reinterpret_cast<T*>(base + kHead + kS * kTile);             // [2][kR][kW]
  T* ns = reinterpret_cast<T*>(base + kHead + (kS + 2) * kTile);       // [2][kR][kW], only with has_xn
  // training saves (norm-only mode): running mean and rstd per step, fp32 [2][kR][kW] each
  float* cms = reinterpret_cast<float*>(base + kHead + (kS + 2) * kTile);
  float* crs = cms + 2 * kR * kW;

  const int tid = threadIdx.x;
  const int d0 = blockIdx.x * kW;
  const int b = blockIdx.y;
  const int d = d0 + tid;
  const bool valid = d < a.D;
  const int dc = valid ? d : a.D - 1;
  const int L = a.L;
  const int nt = (L + kR - 1) / kR;

  if (tid == 0) {
    prefetch_tensormap(&tmx);
    prefetch_tensormap(&tmy);
    if (a.has_xn) prefetch_tensormap(&tmn);
#pragma unroll
    for (int s = 0; s < kS; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0) {
    for (int s = 0; s < kS && s < nt; ++s) {
      mbar_expect_tx(&full[s], kTile);
      tma_load_3d(xs + (size_t)s * kR * kW, &tmx, d0, s * kR, b, &full[s]);
    }
  }

  // per-channel constants and running state
  f32x2 q2[kNP / 2], c2[kNP / 2], s2[kNP / 2], p2[kState ? kNP / 2 : 1];
  // complex poles: q2 / c2 / s2 hold the real parts, these the imaginary parts (nq2i = -Im q,
  // nc2i = -Im gamma: y = Re(gamma h) = gr hr - gi hi)
  f32x2 nq2i[kCplx ? kNP / 2 : 1], q2i[kCplx ? kNP / 2 : 1], nc2i[kCplx ? kNP / 2 : 1], s2i[kCplx ? kNP / 2 : 1];
  float om = 0.f;
  if (kEma && kCplx) {
    om = __ldg(a.omega + dc);
#pragma unroll
    for (int j = 0; j < kNP / 2; ++j) {
      float pv[2], qr[2], qi[2], gr[2], gi[2], hr[2], hi[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int n = 2 * j + k;
        pv[k] = qr[k] = qi[k] = gr[k] = gi[k] = hr[k] = hi[k] = 0.f;
        if (n < a.N) {
          const size_t c = (size_t)dc * a.N + n;
          pv[k] = __ldg(a.p + c);
          qr[k] = __ldg(a.q + 2 * c);
          qi[k] = __ldg(a.q + 2 * c + 1);
          gr[k] = __ldg(a.g + 2 * c);
          gi[k] = __ldg(a.g + 2 * c + 1);
          if (kState && a.h_in) {
            const size_t sidx = ((size_t)b * a.D + dc) * a.N + n;
            hr[k] = __ldg(a.h_in + 2 * sidx);
            hi[k] = __ldg(a.h_in + 2 * sidx + 1);
          }
        }
      }
      q2[j] = pack2(qr[0], qr[1]);
      q2i[j] = pack2(qi[0], qi[1]);
      nq2i[j] = pack2(-qi[0], -qi[1]);
      if (kState) {  // true states, input gain applied per step
        c2[j] = pack2(gr[0], gr[1]);
        nc2i[j] = pack2(-gi[0], -gi[1]);
        p2[j] = pack2(pv[0], pv[1]);
        s2[j] = pack2(hr[0], hr[1]);
        s2i[j] = pack2(hi[0], hi[1]);
      } else {       // states scaled by 1 / p: the gain moves into the output weights
        c2[j] = pack2(pv[0] * gr[0], pv[1] * gr[1]);
        nc2i[j] = pack2(-pv[0] * gi[0], -pv[1] * gi[1]);
        s2[j] = pack2(0.f, 0.f);
        s2i[j] = pack2(0.f, 0.f);
      }
    }
  } else if (kEma) {
    om = __ldg(a.omega + dc);
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
          if (kState && a.h_in) hv[k] = __ldg(a.h_in + ((size_t)b * a.D + dc) * a.N + n);
        }
      }
      q2[j] = pack2(qv[0], qv[1]);
      if (kState) {
        c2[j] = pack2(gv[0], gv[1]);
        p2[j] = pack2(pv[0], pv[1]);
        s2[j] = pack2(hv[0], hv[1]);
      } else {
        c2[j] = pack2(pv[0] * gv[0], pv[1] * gv[1]);
        s2[j] = pack2(0.f, 0.f);
      }
    }
  }
  float mean = 0.f, var = 1.f, w = 1.f, bb = 0.f;
  if (kNorm) {
    mean = a.prev_mean[(size_t)b * a.D + dc];
    var = a.prev_var[(size_t)b * a.D + dc];
    w = __ldg(a.gamma + dc);
    bb = __ldg(a.beta + dc);
  }

  // warp 0 keeps the running count and publishes, per timestep of the next tile, the Welford
  // coefficient 1/count (negative = padded step)
  long long cnt_run = kNorm ? a.prev_count[b] + a.count_offset : 0;
  const unsigned char* mrow = a.mask ? a.mask + (size_t)b * L : nullptr;
  auto publish = [&](int tile, unsigned char mk_byte) {
    // called by warp 0 (kR == 32 lanes); lane r handles timestep tile*kR + r
    const int t = tile * kR + tid;
    const bool masked = (t >= L) || (mk_byte != 0);
    const unsigned vmask = __ballot_sync(0xffffffffu, !masked);
    const int upto = __popc(vmask & (0xffffffffu >> (31 - tid)));
    const float cf = __frcp_rn((float)(cnt_run + upto));
    cbuf[(tile & 1) * kR + tid] = masked ? -1.0f : cf;
    cnt_run += __popc(vmask);
  };
  if (tid < 32) {
    const int t = tid;
    unsigned char mb = (mrow && t < L) ? mrow[t] : 0;
    publish(0, mb);
  }
  __syncthreads();

  for (int i = 0; i < nt; ++i) {
    const int s = i % kS;
    const uint32_t ph = (uint32_t)((i / kS) & 1);
    const int o = i & 1;
    // prefetch the padding flags of the next tile (consumed after the row loop)
    unsigned char mb_next = 0;
    if (tid < 32 && mrow) {
      const int t = (i + 1) * kR + tid;
      if (t < L) mb_next = mrow[t];
    }
    const bool ok = mbar_wait(&full[s], ph);
    const T* xt = xs + (size_t)s * kR * kW + tid;
    T* yt = ys + (size_t)o * kR * kW + tid;
    T* ntile = ns + (size_t)o * kR * kW + tid;
    const float* cf = cbuf + o * kR;
    const int rows = min(kR, L - i * kR);
#pragma unroll 8
    for (int r = 0; r < kR; ++r) {
      if (r < rows) {
        const float xr = Elem<T>::ld_shared(xt + r * kW);
        const float coef = cf[r];
        const bool mk = coef < 0.f;
        float xn;
        if (kNorm) {
          const float d1 = xr - mean;
          const float m1 = fmaf(coef, d1, mean);
          const float dm = xr - m1;
          const float d2 = fmaf(d1, dm, -var);
          const float m2 = fmaf(coef, d2, var);
          const float rstd = rsqrtf(m2 + a.eps);
          xn = mk ? 0.f : fmaf(dm * rstd, w, bb);
          mean = mk ? mean : m1;
          var = mk ? var : m2;
          if (kSave) {  // the running mean after this step (unchanged by a padded step)
            cms[(o * kR + r) * kW + tid] = mean;
            crs[(o * kR + r) * kW + tid] = rstd;
          }
          if (!kEma || a.has_xn) Elem<T>::st((kEma ? ntile : yt) + r * kW, xn);
        } else {
          xn = mk ? 0.f : xr;
        }
        if (kEma) {
          const f32x2 x2 = pack2(xn, xn);
          f32x2 acc0 = pack2(0.f, 0.f), acc1 = pack2(0.f, 0.f);
          if (kCplx) {
#pragma unroll
            for (int j = 0; j < kNP / 2; ++j) {
              // h' = q h + p x (complex); y += Re(gamma h')
              const f32x2 in2 = kState ? mul2(p2[j], x2) : x2;
              const f32x2 nr = fma2(q2[j], s2[j], fma2(nq2i[j], s2i[j], in2));
              const f32x2 ni = fma2(q2i[j], s2[j], mul2(q2[j], s2i[j]));
              s2[j] = nr;
              s2i[j] = ni;
              acc0 = fma2(c2[j], nr, acc0);
              acc1 = fma2(nc2i[j], ni, acc1);
            }
          } else {
#pragma unroll
          for (int j = 0; j < kNP / 2; j += 2) {
            if (kState) {
              s2[j] = fma2(q2[j], s2[j], mul2(p2[j], x2));
              s2[j + 1] = fma2(q2[j + 1], s2[j + 1], mul2(p2[j + 1], x2));
            } else {
              s2[j] = fma2(q2[j], s2[j], x2);
              s2[j + 1] = fma2(q2[j + 1], s2[j + 1], x2);
            }
            acc0 = fma2(c2[j], s2[j], acc0);
            acc1 = fma2(c2[j + 1], s2[j + 1], acc1);
          }
          }
          float lo, hi;
          unpack2(add2(acc0, acc1), lo, hi);
          float v = fmaf(om, kNorm ? xn : xr, lo + hi);
          if (a.silu) v = siluf_(v);
          Elem<T>::st(yt + r * kW, v);
        }
      }
    }
    if (tid < 32 && i + 1 < nt) publish(i + 1, mb_next);
    fence_proxy_async();
    if (tid == 0) bulk_wait_read<0>();
    if (__syncthreads_or(!ok)) break;
    if (tid == 0) {
      tma_store_3d(&tmy, d0, i * kR, b, ys + (size_t)o * kR * kW);
      if (kNorm && kEma && a.has_xn) tma_store_3d(&tmn, d0, i * kR, b, ns + (size_t)o * kR * kW);
      if (kSave) {
        tma_store_3d(&tmm, d0, i * kR, b, cms + (size_t)o * kR * kW);
        tma_store_3d(&tmr, d0, i * kR, b, crs + (size_t)o * kR * kW);
      }
      bulk_commit();
      if (i + kS < nt) {
        mbar_expect_tx(&full[s], kTile);
        tma_load_3d(xs + (size_t)s * kR * kW, &tmx, d0, (i + kS) * kR, b, &full[s]);
      }
    }
  }
  if (tid == 0) bulk_wait<0>();

  if (valid) {
    if (kNorm) {
      a.mean_out[(size_t)b * a.D + d] = mean;
      a.var_out[(size_t)b * a.D + d] = var;
    }
    if (kEma && kState && kCplx && a.h_out) {
#pragma unroll
      for (int j = 0; j < kNP / 2; ++j) {
        float rl, rh, il, ih;
        unpack2(s2[j], rl, rh);
        unpack2(s2i[j], il, ih);
        const size_t sidx = ((size_t)b * a.D + d) * a.N + 2 * j;
        if (2 * j < a.N) {
          a.h_out[2 * sidx] = rl;
          a.h_out[2 * sidx + 1] = il;
        }
        if (2 * j + 1 < a.N) {
          a.h_out[2 * sidx + 2] = rh;
          a.h_out[2 * sidx + 3] = ih;
        }
      }
    } else if (kEma && kState && a.h_out) {
#pragma unroll
      for (int j = 0; j < kNP / 2; ++j) {
        float lo, hi;
        unpack2(s2[j], lo, hi);
        if (2 * j < a.N) a.h_out[((size_t)b * a.D + d) * a.N + 2 * j] = lo;
        if (2 * j + 1 < a.N) a.h_out[((size_t)b * a.D + d) * a.N + 2 * j + 1] = hi;
      }
    }
  }
  if (kNorm && blockIdx.x == 0 && tid == 0) a.count_out[b] = cnt_run;
}

// ---------------------------------------------------------------------------
// host launcher
// ---------------------------------------------------------------------------
template <typename T, bool kNorm, bool kEma, bool kState, bool kCplx = false, bool kSave = false>
static bool launch_one(const CUtensorMap& tx, const CUtensorMap& ty, const CUtensorMap& tn, const StreamArgs& a,
                       cudaStream_t s, const CUtensorMap* tm = nullptr, const CUtensorMap* tr = nullptr) {
  auto kern = stream_cl_kernel<T, kNorm, kEma, kState, kCplx, kSave>;
  const int smem = StreamCfg<T>::smem_bytes(a.has_xn != 0, kSave);
  static std::once_flag once;
  static bool attr_ok = true;
  std::call_once(once, [&] {
    attr_ok = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   StreamCfg<T>::smem_bytes(true, kSave)) == cudaSuccess;
  });
  if (!attr_ok) {
    cudaGetLastError();
    return false;
  }
  dim3 grid((a.D + kW - 1) / kW, a.B);
  launch(kern, grid, dim3(kW), (size_t)smem, (void*)s, tx, ty, tn, tm ? *tm : ty, tr ? *tr : ty, a);
  g_last_kernel.store("stream_cl", std::memory_order_relaxed);
  return true;
}

// Tries the streamed path; returns false (nothing launched) when the call is outside its envelope:
// channel stride must be 1, ndim <= 16, 16-byte aligned bases and strides, B <= 65535.
bool stream_cl_try(int dtype, const void* x, void* y, void* xn, long long xsb, long long xsl, long long xsd,
                   long long ysb, long long ysl, long long ysd, bool norm, bool ema, const StreamArgs& a_in,
                   cudaStream_t s) {
  if (g_options[OPT_DISABLE_STREAM].load() != 0) return false;
  if (xsd != 1 || ysd != 1) return false;
  if (ema && a_in.N > kNP) return false;
  if (a_in.B > 65535 || a_in.D < 8) return false;
  StreamArgs a = a_in;
  a.has_xn = (xn != nullptr && norm && ema) ? 1 : 0;
  CUtensorMap tx, ty, tn;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
    return false;
  if (!make_tensor_map_3d(&ty, dtype, y, a.D, a.L, a.B, ysl, ysb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
    return false;
  tn = ty;
  if (a.has_xn &&
      !make_tensor_map_3d(&tn, dtype, xn, a.D, a.L, a.B, ysl, ysb, kW, kR, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
    return false;
  const bool state = ema && (a.h_in || a.h_out);
  const bool save = norm && !ema && a.cummean != nullptr && a.cumrstd != nullptr;
  CUtensorMap tm, tr;
  if (save) {
    if (!make_tensor_map_3d(&tm, MEGA_F32, a.cummean, a.D, a.L, a.B, a.D, (long long)a.L * a.D, kW, kR, 1,
                            CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !make_tensor_map_3d(&tr, MEGA_F32, a.cumrstd, a.D, a.L, a.B, a.D, (long long)a.L * a.D, kW, kR, 1,
                            CU_TENSOR_MAP_SWIZZLE_NONE))
      return false;
  }
  bool ok = false;
  switch (dtype) {
#define MEGA_STREAM_CASE(DT, TY)                                                        \
  case DT:                                                                              \
    if (ema && a.cplx) {                                                                \
      if (norm) ok = state ? launch_one<TY, true, true, true, true>(tx, ty, tn, a, s)   \
                           : launch_one<TY, true, true, false, true>(tx, ty, tn, a, s); \
      else ok = state ? launch_one<TY, false, true, true, true>(tx, ty, tn, a, s)       \
                      : launch_one<TY, false, true, false, true>(tx, ty, tn, a, s);     \
    } else if (norm && ema) ok = state ? launch_one<TY, true, true, true>(tx, ty, tn, a, s)    \
                                : launch_one<TY, true, true, false>(tx, ty, tn, a, s);  \
    else if (ema) ok = state ? launch_one<TY, false, true, true>(tx, ty, tn, a, s)      \
                             : launch_one<TY, false, true, false>(tx, ty, tn, a, s);    \
    else if (save) ok = launch_one<TY, true, false, false, false, true>(tx, ty, tn, a, s, &tm, &tr); \
    else ok = launch_one<TY, true, false, false>(tx, ty, tn, a, s);                     \
    break;
    MEGA_STREAM_CASE(MEGA_F32, float)
    MEGA_STREAM_CASE(MEGA_BF16, __nv_bfloat16)
    MEGA_STREAM_CASE(MEGA_F16, __half)
#undef MEGA_STREAM_CASE
    default: return false;
  }
  return ok;
}

}  // namespace mega

extern "C" MEGA_API int mega_debug_device_error(int* host_value, int reset) {
  if (!host_value) return MEGA_ERR_NULL;
  int v = 0;
  int v2 = 0;
  if (mega::read_device_error(&v, reset != 0) != cudaSuccess) return mega::check_launch("device_error");
  if (mega::mma_cl_read_device_error(&v2, reset != 0) != cudaSuccess) return mega::check_launch("device_error");
  int v3 = 0;
  if (mega::stream_bwd_read_device_error(&v3, reset != 0) != cudaSuccess) return mega::check_launch("device_error");
  v2 |= v3;
  if (mega::stream_group_read_device_error(&v3, reset != 0) != cudaSuccess) return mega::check_launch("device_error");
  v2 |= v3;
  *host_value = v | v2;
  return MEGA_OK;
}
