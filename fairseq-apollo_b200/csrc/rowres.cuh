// Interface of the row-resident length-contiguous EMA kernels (rowres.cu).
#pragma once
#include <cuda_runtime.h>

namespace mega {

struct RowArgs {
  const void* x;
  void* y;
  int B, D, L, N;
  long long xsb, xsd, ysb, ysd;
  const float *p, *q, *g, *omega;        // (K, N) coefficient rows, K = D or 2D
  const unsigned char* mask;             // (B, L) or null
  const float *ngamma, *nbeta;           // SequenceNorm affine (effective scale), or null
  float eps;
  long long* count_out;                  // SequenceNorm outputs (optional)
  float *mean_out, *rstd_out;
  int shift, silu;
  int seg;                               // elements per thread (multiple of 4)
  unsigned magic;                        // ceil(2^32 / seg)
};

// Tries the row-resident path: length stride 1 on both tensors, ndim <= 16, the row (two copies
// when bidirectional) fits in shared memory, at least 512 positions.  Returns false, launching
// nothing, otherwise.  `norm` fuses a per-channel SequenceNorm in front of the EMA.
bool rowres_try(int dtype, const RowArgs& a, long long xsl, long long ysl, bool bidir, bool norm, cudaStream_t s);

}  // namespace mega
