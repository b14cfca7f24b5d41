// Attention-weight softmax of the Mega block: softmax over the last axis of the (.., C_q, C_k)
// score tensor with an optional causal mask (row r keeps its first C_k - C_q + r + 1 columns) and
// its backward.  One CTA per row; the row stays in registers between the three steps (maximum,
// sum of exponentials, normalise), so HBM sees one read and one write per element.
#include "common.cuh"

namespace mega {

namespace {

constexpr int kT = 128;  // threads per row

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* shm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();  // shm may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) shm[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = shm[0];
#pragma unroll
  for (int w = 1; w < kT / 32; ++w) r = is_max ? fmaxf(r, shm[w]) : r + shm[w];
  return r;
}

// DropKey (dropout on the attention scores before the softmax): column c of row `row` is dropped
// when word c % 4 of Philox4x32-10(counter = (c / 4, row, offset), key = seed) is below the
// threshold, so the mask depends on (seed, offset, row, column) only, not on the launch shape.
struct DropKey {
  unsigned long long seed, offset;
  unsigned threshold;  // dropout * 2^32 (a column is dropped when its 32 random bits are below it)
};

__device__ __forceinline__ uint4 philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0,
                                               unsigned k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}
__device__ __forceinline__ uint4 dropkey_words(const DropKey& dk, long long row, int col_group) {
  return philox4x32_10((unsigned)col_group, (unsigned)row, (unsigned)dk.offset, (unsigned)(dk.offset >> 32),
                       (unsigned)dk.seed, (unsigned)(dk.seed >> 32));
}

// 16-byte vector access: kV elements of type T
template <typename T>
struct Vec {
  static constexpr int kV = 16 / (int)sizeof(T);
  static __device__ __forceinline__ void load(const T* p, float (&v)[kV]) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < kV; ++k) v[k] = Elem<T>::ld_shared(e + k);
  }
  static __device__ __forceinline__ void store(T* p, const float (&v)[kV]) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int k = 0; k < kV; ++k) Elem<T>::st(e + k, v[k]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

// Vectorised rows (inner a multiple of the vector width, 16-byte aligned rows): kN vectors per
// thread, vector j of thread t covers columns (t + j * kT) * kV ...
template <typename T, int kN, bool kDrop>
__global__ void __launch_bounds__(kT) attn_softmax_fwd_vec_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                  long long outer, int inner, int causal,
                                                                  DropKey dk) {
  constexpr int kV = Vec<T>::kV;
  __shared__ float shm[kT / 32];
  const long long row = blockIdx.x;
  const int r = (int)(row % outer);
  const int n = causal ? (int)(inner - outer + r + 1) : inner;
  const T* xr = x + row * inner;
  T* yr = y + row * inner;
  float v[kN][kV];
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < kN; ++j) {
    const int c = (threadIdx.x + j * kT) * kV;
    if (c < n) {  // vectors wholly past the kept columns are not read at all
      Vec<T>::load(xr + c, v[j]);
      if (kDrop) {
#pragma unroll
        for (int k4 = 0; k4 < kV; k4 += 4) {
          const uint4 w = dropkey_words(dk, row, (c + k4) >> 2);
          if (w.x < dk.threshold) v[j][k4 + 0] = -INFINITY;
          if (w.y < dk.threshold) v[j][k4 + 1] = -INFINITY;
          if (w.z < dk.threshold) v[j][k4 + 2] = -INFINITY;
          if (w.w < dk.threshold) v[j][k4 + 3] = -INFINITY;
        }
      }
#pragma unroll
      for (int k = 0; k < kV; ++k) {
        if (c + k >= n) v[j][k] = -INFINITY;
        m = fmaxf(m, v[j][k]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < kV; ++k) v[j][k] = -INFINITY;
    }
  }
  m = block_reduce(m, true, shm);
  const bool dead = m == -INFINITY;
  float d = 0.f;
#pragma unroll
  for (int j = 0; j < kN; ++j)
#pragma unroll
    for (int k = 0; k < kV; ++k) {
      v[j][k] = dead ? 0.f : __expf(v[j][k] - m);
      d += v[j][k];
    }
  d = block_reduce(d, false, shm);
  const float inv = d == 0.f ? 0.f : 1.f / d;
#pragma unroll
  for (int j = 0; j < kN; ++j) {
    const int c = (threadIdx.x + j * kT) * kV;
    if (c < inner) {
#pragma unroll
      for (int k = 0; k < kV; ++k) v[j][k] *= inv;
      Vec<T>::store(yr + c, v[j]);
    }
  }
}

template <typename T, int kN>
__global__ void __launch_bounds__(kT) attn_softmax_bwd_vec_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                                  T* __restrict__ dx, long long outer, int inner,
                                                                  int causal) {
  constexpr int kV = Vec<T>::kV;
  __shared__ float shm[kT / 32];
  const long long row = blockIdx.x;
  const int r = (int)(row % outer);
  const int n = causal ? (int)(inner - outer + r + 1) : inner;
  const T* gr = dy + row * inner;
  const T* yr = y + row * inner;
  T* dr = dx + row * inner;
  float yv[kN][kV], gv[kN][kV];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kN; ++j) {
    const int c = (threadIdx.x + j * kT) * kV;
    if (c < n) {
      Vec<T>::load(yr + c, yv[j]);
      Vec<T>::load(gr + c, gv[j]);
#pragma unroll
      for (int k = 0; k < kV; ++k) {
        if (c + k >= n) yv[j][k] = 0.f;
        s = fmaf(yv[j][k], gv[j][k], s);
      }
    } else {
#pragma unroll
      for (int k = 0; k < kV; ++k) yv[j][k] = gv[j][k] = 0.f;
    }
  }
  s = block_reduce(s, false, shm);
#pragma unroll
  for (int j = 0; j < kN; ++j) {
    const int c = (threadIdx.x + j * kT) * kV;
    if (c < inner) {
      float o[kV];
#pragma unroll
      for (int k = 0; k < kV; ++k) o[k] = yv[j][k] * (gv[j][k] - s);
      Vec<T>::store(dr + c, o);
    }
  }
}

// kE elements per thread, element j of thread t is column t + j * kT (coalesced)
template <typename T, int kE, bool kDrop>
__global__ void __launch_bounds__(kT) attn_softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                              long long outer, int inner, int causal, DropKey dk) {
  __shared__ float shm[kT / 32];
  const long long row = blockIdx.x;
  const int r = (int)(row % outer);
  const int n = causal ? (int)(inner - outer + r + 1) : inner;  // columns kept (may be <= 0)
  const T* xr = x + row * inner;
  T* yr = y + row * inner;
  float v[kE];
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < kE; ++j) {
    const int c = threadIdx.x + j * kT;
    v[j] = c < n ? Elem<T>::ld(xr + c) : -INFINITY;
    if (kDrop && c < n) {
      const uint4 w = dropkey_words(dk, row, c >> 2);
      const unsigned bits = (c & 3) == 0 ? w.x : (c & 3) == 1 ? w.y : (c & 3) == 2 ? w.z : w.w;
      if (bits < dk.threshold) v[j] = -INFINITY;
    }
    m = fmaxf(m, v[j]);
  }
  m = block_reduce(m, true, shm);
  if (m == -INFINITY) {  // every kept score is -inf (or nothing is kept): the row is all zeros
#pragma unroll
    for (int j = 0; j < kE; ++j) {
      const int c = threadIdx.x + j * kT;
      if (c < inner) Elem<T>::st(yr + c, 0.f);
    }
    return;
  }
  float d = 0.f;
#pragma unroll
  for (int j = 0; j < kE; ++j) {
    v[j] = __expf(v[j] - m);  // exp(-inf) = 0 for masked columns
    d += v[j];
  }
  d = block_reduce(d, false, shm);
  const float inv = d == 0.f ? 0.f : 1.f / d;
#pragma unroll
  for (int j = 0; j < kE; ++j) {
    const int c = threadIdx.x + j * kT;
    if (c < inner) Elem<T>::st(yr + c, v[j] * inv);
  }
}

// dx = y * (dy - sum_k dy_k y_k) on the kept columns, 0 elsewhere
template <typename T, int kE>
__global__ void __launch_bounds__(kT) attn_softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                              T* __restrict__ dx, long long outer, int inner,
                                                              int causal) {
  __shared__ float shm[kT / 32];
  const long long row = blockIdx.x;
  const int r = (int)(row % outer);
  const int n = causal ? (int)(inner - outer + r + 1) : inner;
  const T* gr = dy + row * inner;
  const T* yr = y + row * inner;
  T* dr = dx + row * inner;
  float yv[kE], gv[kE];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kE; ++j) {
    const int c = threadIdx.x + j * kT;
    yv[j] = c < n ? Elem<T>::ld(yr + c) : 0.f;
    gv[j] = c < n ? Elem<T>::ld(gr + c) : 0.f;
    s = fmaf(yv[j], gv[j], s);
  }
  s = block_reduce(s, false, shm);
#pragma unroll
  for (int j = 0; j < kE; ++j) {
    const int c = threadIdx.x + j * kT;
    if (c < inner) Elem<T>::st(dr + c, yv[j] * (gv[j] - s));
  }
}

}  // namespace

}  // namespace mega

using namespace mega;

// vectors per thread for the vectorised kernels: rows up to kT * kN * kV elements
#define MEGA_ATTN_DISPATCH_VEC(KERNEL, EXTRA, ...)                                                   \
  MEGA_DISPATCH_DTYPE(dtype, {                                                                       \
    constexpr int kV = Vec<T>::kV;                                                                   \
    if (inner <= 1 * kT * kV) launch(KERNEL<T, 1 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);          \
    else if (inner <= 2 * kT * kV) launch(KERNEL<T, 2 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);     \
    else if (inner <= 4 * kT * kV) launch(KERNEL<T, 4 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);     \
    else if (inner <= 8 * kT * kV) launch(KERNEL<T, 8 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);     \
    else launch(KERNEL<T, 16 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);                              \
  })

static bool vec_ok(int dtype, int inner, const void* a, const void* b, const void* c) {
  const int kv = 16 / elem_size(dtype);
  return inner % kv == 0 && aligned_to(a, 16) && aligned_to(b, 16) && (c == nullptr || aligned_to(c, 16));
}

#define MEGA_ATTN_DISPATCH(KERNEL, EXTRA, ...)                                                       \
  MEGA_DISPATCH_DTYPE(dtype, {                                                                       \
    if (inner <= 8 * kT) launch(KERNEL<T, 8 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);               \
    else if (inner <= 16 * kT) launch(KERNEL<T, 16 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);        \
    else if (inner <= 32 * kT) launch(KERNEL<T, 32 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);        \
    else launch(KERNEL<T, 64 EXTRA>, grid, kT, 0, stream, __VA_ARGS__);                              \
  })
#define MEGA_COMMA ,

static int attention_softmax_fwd_impl(const void* x, void* y, int dtype, int64_t batch, int64_t outer, int inner,
                                      int causal, bool drop, DropKey dk, mega_stream_t stream) {
  if (!x || !y) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (batch <= 0 || outer <= 0 || inner <= 0) return MEGA_ERR_SHAPE;
  if (inner > 64 * kT) return MEGA_ERR_UNSUPPORTED;  // rows longer than 8192 scores
  if (batch * outer > 2147483647LL) return MEGA_ERR_SHAPE;
  const unsigned grid = (unsigned)(batch * outer);
  if (vec_ok(dtype, inner, x, y, nullptr)) {
    if (drop) {
      MEGA_ATTN_DISPATCH_VEC(attn_softmax_fwd_vec_kernel, MEGA_COMMA true, (const T*)x, (T*)y, (long long)outer, inner,
                             causal, dk);
    } else {
      MEGA_ATTN_DISPATCH_VEC(attn_softmax_fwd_vec_kernel, MEGA_COMMA false, (const T*)x, (T*)y, (long long)outer,
                             inner, causal, dk);
    }
    return check_launch("attention_softmax_fwd(vec)");
  }
  if (drop) {
    MEGA_ATTN_DISPATCH(attn_softmax_fwd_kernel, MEGA_COMMA true, (const T*)x, (T*)y, (long long)outer, inner, causal,
                       dk);
  } else {
    MEGA_ATTN_DISPATCH(attn_softmax_fwd_kernel, MEGA_COMMA false, (const T*)x, (T*)y, (long long)outer, inner, causal,
                       dk);
  }
  return check_launch("attention_softmax_fwd");
}

extern "C" int mega_attention_softmax_fwd(const void* x, void* y, int dtype, int64_t batch, int64_t outer,
                                          int inner, int causal, mega_stream_t stream) {
  return attention_softmax_fwd_impl(x, y, dtype, batch, outer, inner, causal, false, DropKey{0, 0, 0}, stream);
}

extern "C" int mega_attention_dropkey_softmax_fwd(const void* x, void* y, int dtype, int64_t batch, int64_t outer,
                                                  int inner, int causal, double dropout, uint64_t seed,
                                                  uint64_t offset, mega_stream_t stream) {
  if (!(dropout >= 0.0) || dropout >= 1.0) return MEGA_ERR_UNSUPPORTED;
  DropKey dk;
  dk.seed = seed;
  dk.offset = offset;
  dk.threshold = (unsigned)(dropout * 4294967296.0);
  return attention_softmax_fwd_impl(x, y, dtype, batch, outer, inner, causal, dk.threshold != 0, dk, stream);
}

extern "C" int mega_attention_softmax_bwd(const void* dy, const void* y, void* dx, int dtype, int64_t batch,
                                          int64_t outer, int inner, int causal, mega_stream_t stream) {
  if (!dy || !y || !dx) return MEGA_ERR_NULL;
  if (!valid_dtype(dtype)) return MEGA_ERR_DTYPE;
  if (batch <= 0 || outer <= 0 || inner <= 0) return MEGA_ERR_SHAPE;
  if (inner > 64 * kT) return MEGA_ERR_UNSUPPORTED;
  if (batch * outer > 2147483647LL) return MEGA_ERR_SHAPE;
  const unsigned grid = (unsigned)(batch * outer);
  if (vec_ok(dtype, inner, dy, y, dx)) {
    MEGA_ATTN_DISPATCH_VEC(attn_softmax_bwd_vec_kernel, , (const T*)dy, (const T*)y, (T*)dx, (long long)outer, inner,
                           causal);
    return check_launch("attention_softmax_bwd(vec)");
  }
  MEGA_ATTN_DISPATCH(attn_softmax_bwd_kernel, , (const T*)dy, (const T*)y, (T*)dx, (long long)outer, inner, causal);
  return check_launch("attention_softmax_bwd");
}
