// Process-wide bookkeeping of the C ABI: status strings, launch counter, last CUDA error.
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace mega {

std::atomic<uint64_t> g_launches{0};
thread_local char g_cuda_err[256] = "";
std::atomic<int> g_options[8];
std::atomic<const char*> g_last_kernel{"none"};

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return MEGA_OK;
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return MEGA_ERR_CUDA;
}

}  // namespace mega

extern "C" const char* mega_status_string(int status) {
  switch (status) {
    case MEGA_OK: return "ok";
    case MEGA_ERR_NULL: return "a required pointer is NULL";
    case MEGA_ERR_DTYPE: return "unknown activation dtype";
    case MEGA_ERR_SHAPE: return "non-positive or inconsistent extent";
    case MEGA_ERR_STRIDE: return "unsupported stride combination";
    case MEGA_ERR_ALIGN: return "pointer not aligned for its element type";
    case MEGA_ERR_NDIM: return "ndim outside 1..32";
    case MEGA_ERR_UNSUPPORTED: return "request not supported by this build";
    case MEGA_ERR_CUDA: return "CUDA launch failed";
    default: return "unknown status";
  }
}

extern "C" const char* mega_last_cuda_error(void) { return mega::g_cuda_err; }
extern "C" int mega_abi_version(void) { return MEGA_ABI_VERSION; }
extern "C" uint64_t mega_launch_count(void) { return mega::g_launches.load(); }

extern "C" MEGA_API const char* mega_debug_last_kernel(void) { return mega::g_last_kernel.load(); }

extern "C" MEGA_API int mega_set_option(int key, int value) {
  if (key < 0 || key >= 8) return MEGA_ERR_SHAPE;
  mega::g_options[key].store(value);
  return MEGA_OK;
}
