// Interface of the streamed channel-contiguous kernels (stream_cl.cu).
#pragma once
#include <cuda_runtime.h>

namespace mega {

struct StreamArgs {
  int B, L, D, N;
  const long long* prev_count;
  const float *prev_mean, *prev_var, *gamma, *beta;
  float eps;
  long long* count_out;
  float *mean_out, *var_out;
  const float *p, *q, *g, *omega;
  const float* h_in;
  float* h_out;
  const unsigned char* mask;
  int silu;
  int has_xn;
  float *cummean, *cumrstd;  // training saves of the norm-only mode, (B, L, D) fp32 contiguous, or NULL
  int cplx;  // complex poles: q, g are interleaved (re, im) (K, N, 2); states (B, D, N, 2)
  // set by the tensor-core path itself (callers leave them alone)
  long long wait_limit;  // SM cycles after which a bounded wait gives up
  int withhold_step;     // test aid: step whose tile is never loaded, or -1
  long long count_offset;  // added to prev_count (a call that continues another call's positions)
  // segmented form of the tensor-core path (mma_cl_seg.cu): the sequence is cut into n_seg runs of seg_steps
  // steps; a work item is (run, tile of channels, group of sequences), taken from sched[0] in order
  int n_seg, seg_steps, n_items, tiles_d;
  float* handoff_h;  // pole states between the runs of a strip, laid out like h_out
  float* handoff_s;  // running sum and squared deviations (B, D, 2) between the runs
  unsigned char* matrices;  // per tile of channels: the tile's matrices as the kernel holds them in shared memory
  int* sched;        // [0]: next work item; [1 + item]: set once the item's statistics and states are written;
                     // [1 + n_items]: set when a wait of this launch ran out
};

// Tries the streamed TMA path for TimestepNorm (norm), causal EMA (ema) or both fused.  Returns
// false, having launched nothing, when the call is outside its envelope (channel stride != 1,
// ndim > 16, bases or strides not 16-byte aligned, more than 65535 sequences).
bool stream_cl_try(int dtype, const void* x, void* y, void* xn, long long xsb, long long xsl, long long xsd,
                   long long ysb, long long ysl, long long ysd, bool norm, bool ema, const StreamArgs& a,
                   cudaStream_t s);

// Tries the tensor-core path (mma_cl.cu): bf16, channel stride 1, ndim <= 16 (its envelope is
// stated at the definition).  Same contract as stream_cl_try.
bool mma_cl_try(int dtype, const void* x, void* y, void* xn, long long xsb, long long xsl, long long xsd,
                long long ysb, long long ysl, long long ysd, bool norm, const StreamArgs& a, cudaStream_t s);
// The segmented form of the tensor-core path with the given number of runs (2, 4 or 8), or false
// (nothing launched) when the call is outside its envelope or its scratch.
bool mma_cl_runs(int dtype, const void* x, void* y, long long xsb, long long xsl, long long xsd, long long ysb,
                 long long ysl, long long ysd, const StreamArgs& a, int runs, cudaStream_t s);
// (mma_cl_seg.cu) the segmented form of the tensor-core kernel in n_seg runs, or false (nothing launched)
bool mma_cl_segmented(int dtype, const void* x, void* y, long long xsb, long long xsl, long long ysb, long long ysl,
                      bool norm, const StreamArgs& a, int n_seg, cudaStream_t s);
cudaError_t mma_cl_seg_read_device_error(int* v, bool reset);
// (mma_cl_narrow.cu) launches of the forms with tiles narrower than 56 channels and of the complex forms
bool mma_cl_narrow(int tile, int dtype, const void* x, void* y, void* xn, long long xsb, long long xsl, long long ysb,
                   long long ysl, bool norm, const StreamArgs& a, cudaStream_t s);
cudaError_t mma_cl_narrow_read_device_error(int* v, bool reset);
cudaError_t mma_cl_read_device_error(int* v, bool reset);

}  // namespace mega
