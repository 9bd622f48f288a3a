// Fused softmax cross-entropy over large vocabularies: logits[rows, V] (bf16 or fp32) and integer
// labels -> per-row loss and log-sum-exp (forward); dlogits = (softmax - onehot) * dloss (backward).
// Replaces log_softmax + nll_loss (keras/src/backend/torch/nn.py:936-982) and their fp32 upcast copies.
#include "common.cuh"

constexpr int XE_THREADS = 512;

template <typename T>
__global__ void __launch_bounds__(XE_THREADS) xent_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                                              float* __restrict__ loss, float* __restrict__ lse_out, int V) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* l = logits + row * V;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < V; i += XE_THREADS) {
    const float v = to_f32<T>(l[i]);
    if (v > m) {
      s = s * __expf(m - v) + 1.f;
      m = v;
    } else {
      s += __expf(v - m);
    }
  }
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
                                                              int V) {
  const long long row = blockIdx.x;
  const T* l = logits + row * V;
  T* d = dlogits + row * V;
  const float r_lse = lse[row], g = dloss[row];
  const long long t = labels[row];
  const bool valid = t >= 0 && t < V;
  for (int i = threadIdx.x; i < V; i += XE_THREADS) {
    float p = __expf(to_f32<T>(l[i]) - r_lse);
    if (i == t) p -= 1.f;
    d[i] = from_f32<T>(valid ? p * g : 0.f);
  }
}

KB_API int kb200_xent_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long rows, int V, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1)
    xent_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, labels, loss, lse, V);
  else
    xent_fwd_kernel<float><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const float*)logits, labels, loss, lse, V);
  KB_CHECK_LAUNCH("xent_fwd");
  return 0;
}

KB_API int kb200_xent_bwd(const void* logits, const long long* labels, const float* lse, const float* dloss, void* dlogits, long long rows, int V,
                          int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1)
    xent_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, labels, lse, dloss, (__nv_bfloat16*)dlogits, V);
  else
    xent_bwd_kernel<float><<<(unsigned)rows, XE_THREADS, 0, stream>>>((const float*)logits, labels, lse, dloss, (float*)dlogits, V);
  KB_CHECK_LAUNCH("xent_bwd");
  return 0;
}
