// LayerNorm / RMSNorm forward and backward over the last axis: rows x D, bf16 or fp32 I/O, fp32 math.
// Replaces F.layer_norm / F.rms_norm plus the two cast kernels around them
// (keras/src/ops/nn.py:3035-3069,3151-3210).  One block per row in forward; backward uses a
// persistent grid that accumulates dgamma/dbeta partials in registers and reduces them in a second
// kernel.
#include "common.cuh"

constexpr int NORM_THREADS = 256;

// rms != 0: RMSNorm (no mean subtraction, no beta)
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS) norm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int D,
                                                                float eps, int rms) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * D;
  T* yr = y + row * D;
  float s = 0.f, ss = 0.f;
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) {
    const float v = to_f32<T>(xr[i]);
    s += v;
    ss += v * v;
  }
  s = block_sum(s, red);
  ss = block_sum(ss, red);
  const float mean = rms ? 0.f : s / D;
  const float var = rms ? ss / D : fmaxf(ss / D - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) {
    float v = (to_f32<T>(xr[i]) - mean) * rstd;
    if (gamma) v *= gamma[i];
    if (beta) v += beta[i];
    yr[i] = from_f32<T>(v);
  }
}

// Each block walks rows blockIdx.x, +gridDim.x, ...; thread t owns columns t, t+256, ... (<= MAXC per thread)
template <typename T, int MAXC>
__global__ void __launch_bounds__(NORM_THREADS) norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                                                                const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                                                                float* __restrict__ partial_dgamma, float* __restrict__ partial_dbeta,
                                                                long long rows, int D, int rms) {
  __shared__ float red[32];
  float dg[MAXC], db[MAXC];
#pragma unroll
  for (int k = 0; k < MAXC; ++k) { dg[k] = 0.f; db[k] = 0.f; }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    const float mu = rms ? 0.f : mean[row];
    const float rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < D) {
        const float xhat = (to_f32<T>(xr[i]) - mu) * rs;
        const float d = to_f32<T>(dyr[i]);
        const float g = gamma ? gamma[i] * d : d;
        s1 += g;
        s2 += g * xhat;
        dg[k] += d * xhat;
        db[k] += d;
      }
    }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    const float m1 = rms ? 0.f : s1 / D, m2 = s2 / D;
    T* dxr = dx + row * D;
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < D) {
        const float xhat = (to_f32<T>(xr[i]) - mu) * rs;
        const float d = to_f32<T>(dyr[i]);
        const float g = gamma ? gamma[i] * d : d;
        dxr[i] = from_f32<T>(rs * (g - m1 - xhat * m2));
      }
    }
  }
#pragma unroll
  for (int k = 0; k < MAXC; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    if (i < D) {
      partial_dgamma[(long long)blockIdx.x * D + i] = dg[k];
      if (partial_dbeta) partial_dbeta[(long long)blockIdx.x * D + i] = db[k];
    }
  }
}

__global__ void norm_partial_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int D) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(long long)b * D + i];
  out[i] = s;
}

KB_API int kb200_norm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, long long rows, int D, float eps,
                          int rms, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 1)
    norm_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, NORM_THREADS, 0, stream>>>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, D, eps, rms);
  else
    norm_fwd_kernel<float><<<(unsigned)rows, NORM_THREADS, 0, stream>>>((const float*)x, gamma, beta, (float*)y, mean, rstd, D, eps, rms);
  KB_CHECK_LAUNCH("norm_fwd");
  return 0;
}

KB_API int kb200_norm_bwd_blocks(long long rows) {
  long long b = 148 * 4;
  return (int)(rows < b ? rows : b);
}

// partial_dgamma / partial_dbeta: scratch [kb200_norm_bwd_blocks(rows), D] fp32
KB_API int kb200_norm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx, float* partial_dgamma,
                          float* partial_dbeta, float* dgamma, float* dbeta, long long rows, int D, int rms, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D > NORM_THREADS * 32) { kb200_set_error("norm_bwd: D too large (max 8192)"); return -2; }
  const int blocks = kb200_norm_bwd_blocks(rows);
  const int per = (D + NORM_THREADS - 1) / NORM_THREADS;
#define LAUNCH(T, MAXC)                                                                                                            \
  norm_bwd_kernel<T, MAXC><<<blocks, NORM_THREADS, 0, stream>>>((const T*)dy, (const T*)x, gamma, mean, rstd, (T*)dx, partial_dgamma, \
                                                                 partial_dbeta, rows, D, rms)
  if (dtype == 1) {
    if (per <= 4) LAUNCH(__nv_bfloat16, 4);
    else if (per <= 8) LAUNCH(__nv_bfloat16, 8);
    else if (per <= 16) LAUNCH(__nv_bfloat16, 16);
    else LAUNCH(__nv_bfloat16, 32);
  } else {
    if (per <= 4) LAUNCH(float, 4);
    else if (per <= 8) LAUNCH(float, 8);
    else if (per <= 16) LAUNCH(float, 16);
    else LAUNCH(float, 32);
  }
#undef LAUNCH
  KB_CHECK_LAUNCH("norm_bwd");
  if (dgamma) norm_partial_reduce_kernel<<<(D + 127) / 128, 128, 0, stream>>>(partial_dgamma, dgamma, blocks, D);
  if (dbeta && partial_dbeta) norm_partial_reduce_kernel<<<(D + 127) / 128, 128, 0, stream>>>(partial_dbeta, dbeta, blocks, D);
  KB_CHECK_LAUNCH("norm_partial_reduce");
  return 0;
}
