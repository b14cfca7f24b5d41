// Dispatch of the tensor-core kernel (mma_cl_kernel.cuh): which form of it a call takes.  The
// segmented forms are launched from mma_cl_seg.cu, a translation unit of its own because the register
// allocation that suits their step loop (ptxas --register-usage-level) does not suit the others; for the
// same reason the forms with tiles narrower than 56 channels are launched from mma_cl_narrow.cu.
#include "mma_cl_kernel.cuh"

namespace mega {

// Envelope: bf16, channel stride 1, ndim <= 16, a padding mask only with real poles, a
// normalised-copy output (strided like y) only together with the normalisation and distinct from x
// and y, B >= 4 (rows of the MMAs are sequences) unless the pipelined form applies, L < 2^24, and L
// a multiple of 32 when a state is exported.  Returns false, launching nothing, outside of it.
bool mma_cl_try(int dtype, const void* x, void* y, void* xn, long long xsb, long long xsl, long long xsd,
                long long ysb, long long ysl, long long ysd, bool norm, const StreamArgs& a_arg, cudaStream_t s) {
  if (g_options[OPT_DISABLE_MMA].load() != 0) return false;
  StreamArgs a_in = a_arg;
  {
    const int lim = g_options[OPT_WAIT_LIMIT].load(), wh = g_options[OPT_WITHHOLD_LOAD].load();
    a_in.wait_limit = lim > 0 ? (long long)lim : 4000000000LL;
    a_in.withhold_step = wh > 0 ? wh : -1;
  }
  if (dtype != MEGA_BF16 || xsd != 1 || ysd != 1) return false;
  // a padding mask: real poles only
  const bool masked = a_in.mask != nullptr;
  if (masked && a_in.cplx) return false;
  const bool want_xn = xn != nullptr;  // second output: the normalised activations, strided like y
  if (want_xn && (!norm || xn == y || xn == x)) return false;
  const bool ema = a_in.N > 0;  // N = 0: TimestepNorm alone
  if (!ema && (!norm || want_xn || a_in.silu || a_in.h_in || a_in.h_out)) return false;
  const int forced = g_options[OPT_MMA_TILE].load();
  const bool forced_pipe = forced == 222 || forced == 224 || forced == 422 || forced == 124;
  // fewer than 4 sequences leave most rows of the MMAs empty: only the pipelined form, which fills the SMs
  // from the sequence length, is then worth more than the SIMT kernels
  const bool can_pipe = ema && !want_xn && !a_in.cplx && !(a_in.mask != nullptr);
  if (a_in.N > 16 || a_in.N < 0 || (a_in.B < 4 && !(forced_pipe || (forced == 0 && can_pipe))) ||
      a_in.L >= (1 << 24) || a_in.D < 8)
    return false;
  if (a_in.h_out && (a_in.L % kStep) != 0) return false;
  if ((a_in.B + kSeq - 1) / kSeq > 65535) return false;
  // Tile width.  Large problems: 64 channels, or 56 when that fills the 148 SMs in fewer or
  // fuller waves (one CTA per SM; e.g. D = 2048 with 64 sequences: 37 x 8 = 296 CTAs = two full
  // waves).  Problems too small to give every SM a wide tile: 32 or 16 channels per CTA, so
  // that the few (8 sequences x 8 channels) strips there are spread over the SMs; a strip is
  // a serial chain along the sequence, so its speed depends on how few warps share its SM.
  // With the normalisation (three quarters of a step's instructions) such problems take the
  // 16-channel tile with two warps per column: a warp then walks 4 channels per step, e.g.
  // B = 16, L = 4096, D = 1024: 0.29 -> 0.17 ms; B = 8, L = 8192, D = 1024: 0.55 -> 0.30 ms.
  const long long seq_groups = (a_in.B + kSeq - 1) / kSeq;
  auto ctas = [&](int ch) -> long long { return ((a_in.D + ch - 1) / ch) * seq_groups; };
  auto waves_cost = [&](int ch) -> double {
    const long long waves = (ctas(ch) + 147) / 148;
    return (double)waves * ch;  // time ~ waves x work per CTA
  };
  int tile = g_options[OPT_MMA_TILE].load();
  // segmented form (64-channel tile, the sequence in 2, 4 or 8 runs): real EMA, no second output, no mask
  if (tile == 82 || tile == 84 || tile == 88) {
    const int n_seg = tile - 80;
    tile = 0;
    if (can_pipe && a_in.B >= 4) {
      if (mma_cl_segmented(dtype, x, y, xsb, xsl, ysb, ysl, norm, a_in, n_seg, s)) return true;
    } else if (!ema && norm && !masked && a_in.B >= 4) {  // TimestepNorm alone
      if (mma_cl_segmented(dtype, x, y, xsb, xsl, ysb, ysl, true, a_in, n_seg, s)) return true;
    }
  }
  // pipelined forms (real EMA, with or without the normalisation, no second output)
  if ((tile == 222 || tile == 224 || tile == 422 || tile == 124) && (a_in.cplx || !ema || want_xn || masked)) tile = 0;
  if (tile == 71 && (a_in.cplx || !ema || want_xn || masked)) tile = 0;
  if (tile != 2 && tile != 4 && tile != 7 && tile != 8 && tile != 22 && tile != 222 && tile != 224 && tile != 422 &&
      tile != 124 && tile != 71) {
    // (the EMA alone is closer to the memory bound and prefers the 128-byte rows of the 64-channel
    // tile: 1.71 against 2.02 ms at B = 64, L = 16384, D = 2048, unless 56 channels save a wave)
    if (ctas(64) >= 148 || ctas(56) >= 148) {
      tile = waves_cost(56) * (norm ? 1.0 : 1.15) < waves_cost(64) ? 7 : 8;
      // More than one wave: whole waves waste the SMs that the last one leaves idle.  The segmented
      // form takes ceil(items x runs / SMs) / runs waves of 64-channel steps instead (a step of the
      // 56- and of the 64-channel tile take about the same time); it pays when that saves 4 %.
      if (can_pipe && a_in.B >= 4 && ctas(64) > 148) {
        const int nsteps = (a_in.L + kStep - 1) / kStep;
        const double plain = (double)((ctas(tile == 7 ? 56 : 64) + 147) / 148);
        int best = 0;
        double best_cost = plain * 0.96;
        for (int n_seg = 2; n_seg <= 8; n_seg *= 2) {
          if (nsteps % n_seg != 0 || nsteps / n_seg < 64) continue;
          const double cost = (double)((ctas(64) * n_seg + 147) / 148) / n_seg * 1.02;
          if (cost < best_cost) {
            best_cost = cost;
            best = n_seg;
          }
        }
        if (best != 0) {
          if (mma_cl_segmented(dtype, x, y, xsb, xsl, ysb, ysl, norm, a_in, best, s)) return true;
        }
      }
    }
    else if (can_pipe && (ctas(16) <= 148 || a_in.B < 4))
      // too few strips for the SMs: four groups of warps per 16-channel strip set, pipelined along the
      // sequence (B = 8, L = 32768, D = 2048: 1.21 -> 1.05 ms; B = 16, L = 4096, D = 1024: 0.168 -> 0.143 ms;
      // the EMA alone on that shape: 0.153 -> 0.102 ms)
      tile = 224;
    else if (norm) tile = 22;  // 16 channels, two warps per column: twice the strips, half as long a step
    else tile = ctas(32) >= 111 ? 4 : 2;
  }
  // The tile code as the forms allow it; everything narrower than 56 channels (and the complex forms, which
  // always run the 16-channel tile) is launched from mma_cl_narrow.cu.
  if (masked || want_xn) tile = (tile == 7 || tile == 8) ? 7 : 22;
  else if (!ema && (tile == 2 || tile == 4)) tile = 22;
  if (a_in.cplx || !(tile == 7 || tile == 8 || tile == 71))
    return mma_cl_narrow(tile, dtype, x, y, xn, xsb, xsl, ysb, ysl, norm, a_in, s);
  if (masked) {  // 56-channel tile
    if (!norm)  // the EMA alone
      return a_in.silu ? launch_variant<false, 7, true, 1, false, true, false, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)
                       : launch_variant<false, 7, false, 1, false, true, false, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s);
#define MEGA_MASKED(SILU, XN, EMA) \
  launch_variant<true, 7, SILU, 1, XN, EMA, false, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl)
    if (!ema) return MEGA_MASKED(false, false, false);
    if (want_xn) return a_in.silu ? MEGA_MASKED(true, true, true) : MEGA_MASKED(false, true, true);
    return a_in.silu ? MEGA_MASKED(true, false, true) : MEGA_MASKED(false, false, true);
#undef MEGA_MASKED
  }
  if (!ema) {
    // more than one wave of wide tiles: the segmented form, as for the fused pair
    if (a_in.B >= 4 && ctas(64) > 148 && g_options[OPT_MMA_TILE].load() == 0) {
      const int nsteps = (a_in.L + kStep - 1) / kStep;
      const double plain = (double)((ctas(tile == 7 ? 56 : 64) + 147) / 148);
      int best = 0;
      double best_cost = plain * 0.96;
      for (int n_seg = 2; n_seg <= 8; n_seg *= 2) {
        if (nsteps % n_seg != 0 || nsteps / n_seg < 64) continue;
        const double cost = (double)((ctas(64) * n_seg + 147) / 148) / n_seg * 1.02;
        if (cost < best_cost) {
          best_cost = cost;
          best = n_seg;
        }
      }
      if (best != 0 && mma_cl_segmented(dtype, x, y, xsb, xsl, ysb, ysl, true, a_in, best, s)) return true;
    }
    return tile == 7 ? launch_variant<true, 7, false, 1, false, false>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)
                     : launch_variant<true, 8, false, 1, false, false>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s);
  }
  if (want_xn)  // 56-channel tiles (the 64-channel tile has no room for the two extra buffers)
    return a_in.silu ? launch_variant<true, 7, true, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl)
                     : launch_variant<true, 7, false, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl);
#define MEGA_MMA_VARIANT(NORM, SILU)                                                           \
  (tile == 71 ? launch_variant<NORM, 7, SILU, 1, false, true, false, 1, false, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s) \
   : tile == 7 ? launch_variant<NORM, 7, SILU>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)        \
               : launch_variant<NORM, 8, SILU>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s))
  if (norm) return a_in.silu ? MEGA_MMA_VARIANT(true, true) : MEGA_MMA_VARIANT(true, false);
  return a_in.silu ? MEGA_MMA_VARIANT(false, true) : MEGA_MMA_VARIANT(false, false);
#undef MEGA_MMA_VARIANT
}

cudaError_t mma_cl_read_device_error(int* v, bool reset) {
  int v2 = 0;
  cudaError_t e = read_device_error(v, reset);
  if (e == cudaSuccess) e = mma_cl_seg_read_device_error(&v2, reset);
  if (e == cudaSuccess && *v == 0) *v = v2;
  if (e == cudaSuccess) e = mma_cl_narrow_read_device_error(&v2, reset);
  if (e == cudaSuccess && *v == 0) *v = v2;
  return e;
}

}  // namespace mega
