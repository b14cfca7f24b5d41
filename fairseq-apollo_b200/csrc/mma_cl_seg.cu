// The segmented form of the tensor-core kernel (mma_cl_kernel.cuh): its scratch in device memory and
// its launches.
#include "mma_cl_kernel.cuh"

namespace mega {

namespace {

// ---- segmented form (kPs): scratch and launch ---------------------------------------------------
// The hand-off of the pole states between the runs of a strip (when the call has no h_out) and the
// work counter with the items' flags live in fixed device arrays of this library; nothing is
// allocated.  Calls that use them must not overlap: a call on another stream than the one before
// first waits (on the device) for that one's event.
constexpr size_t kHandoffFloats = size_t(4) << 20;  // 16 MiB: pole states of B x D x ndim <= 4 Mi values
constexpr size_t kHandoffStats = size_t(512) << 10;  // 2 MiB: running sums (two values) of B x D <= 256 Ki channels
constexpr size_t kMatrixBytes = size_t(12) << 20;   // 12 MiB: the matrices of 144 tiles of 64 channels
constexpr int kSchedItems = 16384;
static __device__ __align__(256) unsigned char g_matrices[kMatrixBytes];
static __device__ __align__(256) float g_handoff[kHandoffFloats];
static __device__ __align__(256) float g_handoff_stats[kHandoffStats];
static __device__ __align__(256) int g_sched[2 + kSchedItems];   // counter, one flag per item, "a wait ran out"

struct SegScratch {
  bool tried = false, ok = false;
  float* handoff = nullptr;
  float* stats = nullptr;
  unsigned char* matrices = nullptr;
  int* sched = nullptr;
  bool ev_tried = false;
  cudaEvent_t done = nullptr;   // made on first use by a caller that orders its calls across streams
  cudaStream_t last = nullptr;
  bool used = false;
};
static std::mutex g_seg_mutex;
static SegScratch g_seg[16];

// (g_seg_mutex held) scratch of the current device, or nullptr; with_event: also the event that orders
// calls on different streams
static SegScratch* seg_scratch(bool with_event) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  SegScratch& sc = g_seg[dev];
  if (!sc.tried) {
    sc.tried = true;
    bool ok = cudaGetSymbolAddress((void**)&sc.handoff, g_handoff) == cudaSuccess;
    ok = ok && cudaGetSymbolAddress((void**)&sc.stats, g_handoff_stats) == cudaSuccess;
    ok = ok && cudaGetSymbolAddress((void**)&sc.matrices, g_matrices) == cudaSuccess;
    ok = ok && cudaGetSymbolAddress((void**)&sc.sched, g_sched) == cudaSuccess;
    if (!ok) cudaGetLastError();
    sc.ok = ok;
  }
  if (sc.ok && with_event && !sc.ev_tried) {
    sc.ev_tried = true;
    if (cudaEventCreateWithFlags(&sc.done, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      sc.done = nullptr;
    }
  }
  if (with_event && sc.done == nullptr) return nullptr;
  return sc.ok ? &sc : nullptr;
}

// Runs the call as n_seg runs per strip, one CTA per (run, tile, group of sequences).  False (nothing launched) when the
// call does not fit the scratch, the stream is being captured, or the set-up failed.
// order_streams: a call on another stream than the scratch's last user first waits for that one's event
// (the automatic path); without it the caller keeps calls that use the scratch from overlapping.
template <bool kNorm, bool kSilu, bool kEma = true>
static bool launch_segmented(int dtype, const void* x, void* y, long long xsb, long long xsl, long long ysb,
                             long long ysl, const StreamArgs& a_in, int n_seg, cudaStream_t s,
                             bool order_streams = true) {
  static_assert(kEma || (kNorm && !kSilu), "without the EMA: TimestepNorm alone");
  constexpr int kCg = 8;
  using C = Cfg<kCg, false, false, 1, 1, false>;
  StreamArgs a = a_in;
  const int nsteps = (a.L + kStep - 1) / kStep;
  if ((n_seg != 2 && n_seg != 4 && n_seg != 8) || nsteps % n_seg != 0) return false;
  a.n_seg = n_seg;
  a.seg_steps = nsteps / n_seg;
  a.tiles_d = (a.D + C::kCh - 1) / C::kCh;
  const long long items = (long long)a.tiles_d * ((a.B + kSeq - 1) / kSeq) * n_seg;
  if (items > kSchedItems) return false;
  a.n_items = (int)items;
  if (kEma && !a.h_out && (size_t)a.B * a.D * a.N > kHandoffFloats) return false;
  if (kNorm && (size_t)a.B * a.D * 2 > kHandoffStats) return false;
  if ((size_t)a.tiles_d * (C::kOffKp - C::kOffT) > kMatrixBytes) return false;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return false;
  }
  CUtensorMap tx, ty;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, C::kCh, kStep, kSeq, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
  if (!make_tensor_map_3d(&ty, dtype, y, a.D, a.L, a.B, ysl, ysb, C::kCh, kStep, kSeq, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
  auto kern = tsn_ema_mma_kernel<kNorm, kCg, kSilu, 1, false, kEma, false, 1, false, false, kNorm ? 3 : 1>;
  auto builder = tsn_ema_mma_kernel<(kNorm && kEma), kCg, false, 1, false, true, false, 1, false, false, 2>;
  std::lock_guard<std::mutex> lock(g_seg_mutex);
  SegScratch* sc = seg_scratch(order_streams);
  if (sc == nullptr) return false;
  a.handoff_h = sc->handoff;
  a.handoff_s = sc->stats;
  a.matrices = sc->matrices;
  a.sched = sc->sched;
  if (order_streams && sc->used && sc->last != s && cudaStreamWaitEvent(s, sc->done, 0) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (cudaMemsetAsync(sc->sched, 0, sizeof(int) * (size_t)(2 + a.n_items), s) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (!kNorm) launch(builder, dim3((unsigned)a.tiles_d), dim3(kCg * 32), (size_t)C::kSmemBytes, (void*)s, tx, ty, ty, a);
  launch(kern, dim3((unsigned)a.n_items), dim3(kCg * 32), (size_t)C::kSmemBytes, (void*)s, tx, ty, ty, a);
  if (order_streams) {
    cudaEventRecord(sc->done, s);
    sc->last = s;
    sc->used = true;
  }
  static const std::string base = std::string("tsn_ema_mma tile=8 warps_per_column=1 pipe=1") + (kNorm ? " norm" : "") +
                                  (kEma ? " ema" : "") + " segmented runs=";
  static const std::string names[3] = {base + "2", base + "4", base + "8"};
  g_last_kernel.store(names[n_seg == 2 ? 0 : n_seg == 4 ? 1 : 2].c_str(), std::memory_order_relaxed);
  return true;
}

}  // namespace

// The segmented form in n_seg runs for the call (norm: TimestepNorm in front; ema: a.N > 0), or false
// (nothing launched) when the call does not fit its envelope or its scratch.
bool mma_cl_segmented(int dtype, const void* x, void* y, long long xsb, long long xsl, long long ysb, long long ysl,
                      bool norm, const StreamArgs& a, int n_seg, cudaStream_t s) {
  const bool ema = a.N > 0;
  if (!ema) return norm && !a.silu && launch_segmented<true, false, false>(dtype, x, y, xsb, xsl, ysb, ysl, a, n_seg, s);
  if (norm)
    return a.silu ? launch_segmented<true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a, n_seg, s)
                  : launch_segmented<true, false>(dtype, x, y, xsb, xsl, ysb, ysl, a, n_seg, s);
  return a.silu ? launch_segmented<false, true>(dtype, x, y, xsb, xsl, ysb, ysl, a, n_seg, s)
                : launch_segmented<false, false>(dtype, x, y, xsb, xsl, ysb, ysl, a, n_seg, s);
}

// The segmented form on request (mega_tsn_ema_fwd_runs): the normalising kernel in `runs` runs or
// nothing.  Uses only the fixed device arrays above (no event either).
bool mma_cl_runs(int dtype, const void* x, void* y, long long xsb, long long xsl, long long xsd, long long ysb,
                 long long ysl, long long ysd, const StreamArgs& a_arg, int runs, cudaStream_t s) {
  if (dtype != MEGA_BF16 || xsd != 1 || ysd != 1) return false;
  if (a_arg.mask != nullptr || a_arg.cplx || a_arg.N < 1 || a_arg.N > 16 || a_arg.B < 4 || a_arg.L >= (1 << 24) ||
      a_arg.D < 8 || (a_arg.L % kStep) != 0 || (a_arg.B + kSeq - 1) / kSeq > 65535)
    return false;
  StreamArgs a = a_arg;
  const int lim = g_options[OPT_WAIT_LIMIT].load();
  a.wait_limit = lim > 0 ? (long long)lim : 4000000000LL;
  a.withhold_step = -1;
  return a.silu ? launch_segmented<true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a, runs, s, false)
                : launch_segmented<true, false>(dtype, x, y, xsb, xsl, ysb, ysl, a, runs, s, false);
}

cudaError_t mma_cl_seg_read_device_error(int* v, bool reset) { return read_device_error(v, reset); }

}  // namespace mega
