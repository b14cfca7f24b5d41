// The forms of the tensor-core kernel (mma_cl_kernel.cuh) with tiles narrower than 56 channels, and the
// complex forms (always 16 channels): launches only, the choice of the form is made in mma_cl.cu.  A
// translation unit of its own because these forms run ~2 % faster with a low ptxas register usage level.
#include "mma_cl_kernel.cuh"

namespace mega {

// `tile` as mma_cl_try settled it: 22 for masked / normalised-copy / TimestepNorm-alone calls, else one of
// 2, 4, 22, 222, 224, 422, 124 (any value with complex poles).
bool mma_cl_narrow(int tile, int dtype, const void* x, void* y, void* xn, long long xsb, long long xsl, long long ysb,
                   long long ysl, bool norm, const StreamArgs& a_in, cudaStream_t s) {
  const bool masked = a_in.mask != nullptr;
  const bool want_xn = xn != nullptr;
  const bool ema = a_in.N > 0;
  if (a_in.cplx) {
    // complex poles (fused TimestepNorm -> MultiHeadComplexEMA): the matrices of a channel take
    // 2.4 KB, so the 16-channel tile with two warps per column (three CTAs per SM) serves all sizes
    if (!ema || masked) return false;
    if (!norm)  // the complex layer alone
      return a_in.silu ? launch_variant<false, 2, true, 2, false, true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)
                       : launch_variant<false, 2, false, 2, false, true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s);
    if (want_xn)
      return a_in.silu ? launch_variant<true, 2, true, 2, true, true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl)
                       : launch_variant<true, 2, false, 2, true, true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl);
    return a_in.silu ? launch_variant<true, 2, true, 2, false, true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)
                     : launch_variant<true, 2, false, 2, false, true, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s);
  }
  if (masked) {  // the 16-channel two-warp tile
    if (!norm)  // the EMA alone
      return a_in.silu ? launch_variant<false, 2, true, 2, false, true, false, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)
                       : launch_variant<false, 2, false, 2, false, true, false, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s);
#define MEGA_MASKED(SILU, XN, EMA) \
  launch_variant<true, 2, SILU, 2, XN, EMA, false, 1, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl)
    if (!ema) return MEGA_MASKED(false, false, false);
    if (want_xn) return a_in.silu ? MEGA_MASKED(true, true, true) : MEGA_MASKED(false, true, true);
    return a_in.silu ? MEGA_MASKED(true, false, true) : MEGA_MASKED(false, false, true);
#undef MEGA_MASKED
  }
  if (!ema) return launch_variant<true, 2, false, 2, false, false>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s);
  if (want_xn)
    return a_in.silu ? launch_variant<true, 2, true, 2, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl)
                     : launch_variant<true, 2, false, 2, true>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s, xn, ysb, ysl);
#define MEGA_MMA_VARIANT(NORM, SILU)                                                           \
  (tile == 222 ? launch_variant<NORM, 2, SILU, 2, false, true, false, 2>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s) \
   : tile == 224 ? launch_variant<NORM, 2, SILU, 2, false, true, false, 4>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s) \
   : tile == 422 ? launch_variant<NORM, 4, SILU, 2, false, true, false, 2>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s) \
   : tile == 124 ? launch_variant<NORM, 1, SILU, 2, false, true, false, 4>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s) \
   : tile == 22  ? launch_variant<NORM, 2, SILU, 2>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)     \
   : tile == 4 ? launch_variant<NORM, 4, SILU>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s)        \
               : launch_variant<NORM, 2, SILU>(dtype, x, y, xsb, xsl, ysb, ysl, a_in, s))
  if (norm) return a_in.silu ? MEGA_MMA_VARIANT(true, true) : MEGA_MMA_VARIANT(true, false);
  return a_in.silu ? MEGA_MMA_VARIANT(false, true) : MEGA_MMA_VARIANT(false, false);
#undef MEGA_MMA_VARIANT
}

cudaError_t mma_cl_narrow_read_device_error(int* v, bool reset) { return read_device_error(v, reset); }

}  // namespace mega
