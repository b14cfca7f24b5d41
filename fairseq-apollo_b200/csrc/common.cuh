// Shared device/host helpers for the mega_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "mega_b200.h"

namespace mega {

// ---- launch bookkeeping ---------------------------------------------------
extern std::atomic<uint64_t> g_launches;
extern thread_local char g_cuda_err[256];
extern std::atomic<int> g_options[8];
enum { OPT_DISABLE_STREAM = 0, OPT_DISABLE_MMA = 1, OPT_MMA_TILE = 2, OPT_WAIT_LIMIT = 3, OPT_WITHHOLD_LOAD = 4 };
// Name of the kernel family of the most recent launch (test aid): launch() sets "other", the
// launchers of the named families overwrite it right after.
extern std::atomic<const char*> g_last_kernel;
int check_launch(const char* what);

// Single-token step with N / 4 lanes per (sequence, channel) (csrc/fused.cu): TimestepNorm update
// when count is given, then the pole update; false (nothing launched) when N is not 4, 8, 16 or 32
// or a state / coefficient pointer is not 16-byte aligned.
bool step_lanes_try(int dtype, const void* x, void* y, void* xn_out, int B, int D, int N, const long long* count,
                    float* mean, float* var, const float* gamma, const float* beta, float eps, const float* p,
                    const float* q, const float* g, const float* omega, const float* h_in, float* h_out, int silu,
                    void* stream, long long* count_next = nullptr);

template <typename... KArgs, typename... Args>
static inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, void* stream,
                          Args... args) {
  // Above the default 48 KB the dynamic shared-memory size is an opt-in attribute of the kernel ON
  // THE CURRENT DEVICE; setting it at every such launch (microseconds, these launches run for
  // hundreds) keeps a process that drives several GPUs correct.
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  kernel<<<grid, block, smem, (cudaStream_t)stream>>>(static_cast<KArgs>(args)...);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  g_last_kernel.store("other", std::memory_order_relaxed);
}

// ---- element I/O ------------------------------------------------------------
template <typename T>
struct Elem;

// `ldv`: the same read-only load as `ld`, issued through a volatile asm statement so that the
// compiler keeps a batch of independent loads together at the top of an unrolled block instead
// of sinking each one to its use (kernels with few resident warps hide latency per thread).
template <>
struct Elem<float> {
  static __device__ __forceinline__ float ld(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ float ldv(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
  }
  static __device__ __forceinline__ float ld_shared(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) {
    return __bfloat162float(__ldg(p));
  }
  static __device__ __forceinline__ float ldv(const __nv_bfloat16* p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __uint_as_float((unsigned)v << 16);
  }
  static __device__ __forceinline__ float ld_shared(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
  }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float ld(const __half* p) { return __half2float(__ldg(p)); }
  static __device__ __forceinline__ float ldv(const __half* p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __half2float(__ushort_as_half(v));
  }
  static __device__ __forceinline__ float ld_shared(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void st(__half* p, float v) { *p = __float2half_rn(v); }
};

// MUFU approximations (about 1 ulp): no slow path, no subroutine call in a serial loop
__device__ __forceinline__ float rcp_approx(float v) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float rsqrt_approx(float v) {
  float r;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + __expf(-v)); }
__device__ __forceinline__ float siluf_(float v) { return v / (1.0f + __expf(-v)); }
// silu(v) = v * sigmoid(v) = h + h * tanh(h), h = v / 2: one MUFU op (tanh.approx, relative error
// about 2^-11) and two FP32 ops.  For kernels whose output is rounded to bf16 / fp16 anyway.
__device__ __forceinline__ float silu_tanh(float v) {
  const float h = 0.5f * v;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}

static inline int elem_size(int dtype) { return dtype == MEGA_F32 ? 4 : 2; }

static inline bool valid_dtype(int dtype) {
  return dtype == MEGA_F32 || dtype == MEGA_BF16 || dtype == MEGA_F16;
}

static inline bool aligned_to(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

static inline int next_pow2_ndim(int n) {
  int v = 2;
  while (v < n) v <<= 1;
  return v;
}

// Dispatch helpers: call f.template operator()<T>() for the activation dtype.
#define MEGA_DISPATCH_DTYPE(dtype, ...)                 \
  switch (dtype) {                                      \
    case MEGA_F32: { using T = float; __VA_ARGS__; } break;           \
    case MEGA_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;  \
    case MEGA_F16: { using T = __half; __VA_ARGS__; } break;          \
    default: return MEGA_ERR_DTYPE;                     \
  }

#define MEGA_DISPATCH_NP(np, ...)                       \
  switch (np) {                                         \
    case 2: { constexpr int NP = 2; __VA_ARGS__; } break;   \
    case 4: { constexpr int NP = 4; __VA_ARGS__; } break;   \
    case 8: { constexpr int NP = 8; __VA_ARGS__; } break;   \
    case 16: { constexpr int NP = 16; __VA_ARGS__; } break; \
    case 32: { constexpr int NP = 32; __VA_ARGS__; } break; \
    default: return MEGA_ERR_NDIM;                      \
  }

}  // namespace mega
