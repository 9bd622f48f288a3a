// Fused softmax cross-entropy over large vocabularies: logits[rows, V] (bf16 or fp32) and integer
// labels -> per-row loss and log-sum-exp (forward); dlogits = (softmax - onehot) * dloss (backward).
// Replaces log_softmax + nll_loss (keras/src/backend/torch/nn.py:936-982) and their fp32 upcast copies.
#include "common.cuh"

constexpr int XE_THREADS = 512;

// `ld` is the row pitch in elements (>= V).  When rows start 16-byte aligned (`vec` = 1: base pointer aligned and the pitch a
// multiple of 16 bytes) the body is read and written as 16-byte vectors; the tail and unaligned inputs use scalar accesses.
// Backward also zeroes the columns [V, Vz) of each row: a padded logits buffer gets a gradient that a padded GEMM can consume.
template <typename T>
struct XeVec {
  static constexpr int N = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void xe_load(const T* p, float* v) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  if constexpr (sizeof(T) == 2) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  } else {
    const float* f = reinterpret_cast<const float*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = f[j];
  }
}

template <typename T>
__device__ __forceinline__ void xe_store(T* p, const float* v) {
  uint4 raw;
  if constexpr (sizeof(T) == 2) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  } else {
    float* f = reinterpret_cast<float*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] = v[j];
  }
  *reinterpret_cast<uint4*>(p) = raw;
}

__device__ __forceinline__ void xe_online(float v, float& m, float& s) {
  if (v > m) {
    s = s * __expf(m - v) + 1.f;
    m = v;
  } else {
    s += __expf(v - m);
  }
}

template <typename T>
__global__ void __launch_bounds__(XE_THREADS) xent_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                                              float* __restrict__ loss, float* __restrict__ lse_out, int V, long long ld, int vec) {
  __shared__ float red[32];
  constexpr int VN = XeVec<T>::N;
  const long long row = blockIdx.x;
  const T* l = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  const int body = vec ? (V / VN) * VN : 0;
  for (int i = threadIdx.x * VN; i < body; i += XE_THREADS * VN) {
    float v[VN];
    xe_load<T>(l + i, v);
    float vm = v[0];
#pragma unroll
    for (int j = 1; j < VN; ++j) vm = fmaxf(vm, v[j]);
    if (vm > m) {
      s *= __expf(m - vm);
      m = vm;
    }
#pragma unroll
    for (int j = 0; j < VN; ++j) s += __expf(v[j] - m);
  }
  for (int i = body + threadIdx.x; i < V; i += XE_THREADS) xe_online(to_f32<T>(l[i]), m, s);
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float lse = gm + logf(s);
    const long long t = labels[row];
    lse_out[row] = lse;
    loss[row] = (t >= 0 && t < V) ? lse - to_f32<T>(l[t]) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(XE_THREADS) xent_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                                              const float* __restrict__ lse, const float* __restrict__ dloss, T* __restrict__ dlogits,
                                                              int V, long long ld, int Vz, int vec) {
  constexpr int VN = XeVec<T>::N;
  const long long row = blockIdx.x;
  const T* l = logits + row * ld;
  T* d = dlogits + row * ld;
  const float r_lse = lse[row];
  const long long t = labels[row];
  const bool valid = t >= 0 && t < V;
  const float g = valid ? dloss[row] : 0.f;
  const int body = vec ? (V / VN) * VN : 0;
  for (int i = threadIdx.x * VN; i < body; i += XE_THREADS * VN) {
    float v[VN];
    xe_load<T>(l + i, v);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      float p = __expf(v[j] - r_lse);
      if (i + j == t) p -= 1.f;
      v[j] = p * g;
    }
    xe_store<T>(d + i, v);
  }
  for (int i = body + threadIdx.x; i < Vz; i += XE_THREADS) {
    float p = 0.f;
    if (i < V) {
      p = __expf(to_f32<T>(l[i]) - r_lse);
      if (i == t) p -= 1.f;
    }
    d[i] = from_f32<T>(p * g);
  }
}

KB_API int kb200_xent_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long rows, int V, long long ld, int dtype,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int esize = dtype == 1 ? 2 : 4;
  const int vec = (((uintptr_t)logits & 15) == 0 && (ld * esize) % 16 == 0) ? 1 : 0;
  if (dtype == 1)
    xent_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, labels, loss, lse, V, ld, vec);
  else
    xent_fwd_kernel<float><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const float*)logits, labels, loss, lse, V, ld, vec);
  KB_CHECK_LAUNCH("xent_fwd");
  return 0;
}

// `zero_to` (V <= zero_to <= ld): columns [V, zero_to) of every dlogits row are written as zeros.
KB_API int kb200_xent_bwd(const void* logits, const long long* labels, const float* lse, const float* dloss, void* dlogits, long long rows, int V,
                          long long ld, int zero_to, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int esize = dtype == 1 ? 2 : 4;
  const int vec = ((((uintptr_t)logits | (uintptr_t)dlogits) & 15) == 0 && (ld * esize) % 16 == 0) ? 1 : 0;
  if (zero_to < V) zero_to = V;
  if (dtype == 1)
    xent_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, labels, lse, dloss, (__nv_bfloat16*)dlogits, V,
                                                                                ld, zero_to, vec);
  else
    xent_bwd_kernel<float><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const float*)logits, labels, lse, dloss, (float*)dlogits, V, ld, zero_to, vec);
  KB_CHECK_LAUNCH("xent_bwd");
  return 0;
}
