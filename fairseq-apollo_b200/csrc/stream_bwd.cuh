// Interface of the streamed backward kernels (stream_bwd.cu): channel-contiguous activations only.
#pragma once
#include <cuda_runtime.h>

namespace mega {

struct TsnBwdStreamArgs {
  int B, L, D;
  const float *dmean, *dvar, *prev_mean;  // (B, D); dmean / dvar may be NULL
  const long long* count;                 // (B) final counts
  const float* gamma;
  const unsigned char* mask;
  float *dprev_mean, *dprev_var, *dgamma, *dbeta;
};

struct EmaBwdStreamArgs {
  int B, L, D, N;
  const float *p, *q, *g, *omega;
  const unsigned char* mask;
  const float *h_in, *dh_out;
  float *dp, *dq, *dg, *domega, *dh_in;
};

// Each returns false, having launched nothing, outside its envelope (channel stride != 1, bases or
// strides not 16-byte aligned, more than 65535 sequences, ndim > 16 for the EMA).
bool tsn_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                        long long gsd, long long xsb, long long xsl, long long xsd, long long dsb, long long dsl,
                        long long dsd, const float* cummean, const float* cumrstd, const TsnBwdStreamArgs& a,
                        cudaStream_t s);
bool ema_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                        long long gsd, long long xsb, long long xsl, long long xsd, long long dsb, long long dsl,
                        long long dsd, const EmaBwdStreamArgs& a, cudaStream_t s);
// Complex layer: q, g of the arguments are interleaved (re, im) (D, N, 2), dq / dg likewise; h_in,
// dh_out, dh_in are not used.
bool cema_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                         long long gsd, long long xsb, long long xsl, long long xsd, long long dsb, long long dsl,
                         long long dsd, const EmaBwdStreamArgs& a, cudaStream_t s);
cudaError_t stream_bwd_read_device_error(int* v, bool reset);

// ---- streamed grouped TimestepNorm (stream_group.cu): group sizes 8, 16, 32, 64 ---------------
struct GroupStreamArgs {
  int B, L, D, G;
  const long long* prev_count;
  const float *prev_mean, *prev_var;  // (B, G)
  const float *gamma, *beta;
  const unsigned char* mask;
  float eps;
  long long* count_out;
  float *mean_out, *var_out;                  // (B, G)
  float *cummean, *cumrstd, *group_mean;      // (B, L, G) training saves, or all NULL
};
struct GroupStreamBwdArgs {
  int B, L, D, G;
  const float *dmean, *dvar, *prev_mean;      // (B, G); dmean / dvar may be NULL
  const long long* count;
  const float *cummean, *cumrstd, *group_mean;
  const float* gamma;
  const unsigned char* mask;
  float *dprev_mean, *dprev_var, *dgamma, *dbeta;
};
bool tsn_group_stream_try(int dtype, const void* x, void* y, long long xsb, long long xsl, long long xsd,
                          long long ysb, long long ysl, long long ysd, const GroupStreamArgs& a, cudaStream_t s);
bool tsn_group_bwd_stream_try(int dtype, const void* dy, const void* x, void* dx, long long gsb, long long gsl,
                              long long gsd, long long xsb, long long xsl, long long xsd, long long dsb,
                              long long dsl, long long dsd, const GroupStreamBwdArgs& a, cudaStream_t s);
cudaError_t stream_group_read_device_error(int* v, bool reset);

}  // namespace mega
