// BatchNorm (training) for channels-last activations x[M, C], fused with ReLU and a residual add.
//
// Replaces the reference's chain of ~8 elementwise/reduction kernels in fp32
// (keras/src/backend/torch/nn.py:1020-1092, keras/src/layers/normalization/batch_normalization.py:345-399)
// by: one statistics pass (per-channel sum / sum of squares, fp32 accumulation, E[x^2]-E[x]^2
// variance as the reference), a C-sized finalize (scale/shift, moving statistics update) and one
// apply pass y = relu(x*scale + shift + residual) with bf16 or fp32 I/O.  Backward is one
// reduction pass plus one apply pass.
#include "common.cuh"

template <typename T>
struct Vec;
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  using Raw = bf16x8;
  __device__ static void load(const __nv_bfloat16* p, float* f) { unpack8(*reinterpret_cast<const bf16x8*>(p), f); }
  __device__ static void store(__nv_bfloat16* p, const float* f) { *reinterpret_cast<bf16x8*>(p) = pack8(f); }
};
template <>
struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* f) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  __device__ static void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};

constexpr int BN_CX = 32;  // channel vectors per block (one warp wide)
constexpr int BN_RY = 8;   // row lanes per block

// sums[0:C] += sum_rows a(row, c);  sums[C:2C] += sum_rows b(row, c)
// MODE 0 (forward stats): a = x, b = x*x
// MODE 1 (backward):      a = dy', b = dy' * xhat, dy' = dy * (y > 0 if relu)
template <typename T, int MODE>
__global__ void __launch_bounds__(BN_CX* BN_RY) bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                                                                const float* __restrict__ mean, const float* __restrict__ invstd,
                                                                long long M, int C, float* __restrict__ sums) {
  constexpr int V = Vec<T>::N;
  const int cv = blockIdx.y * BN_CX + threadIdx.x;  // channel-vector index
  const int cvecs = C / V;
  const bool active = cv < cvecs;
  const int c0 = cv * V;
  float sa[V], sb[V], mu[V], is[V];
#pragma unroll
  for (int k = 0; k < V; ++k) { sa[k] = 0.f; sb[k] = 0.f; mu[k] = 0.f; is[k] = 1.f; }
  if (MODE == 1 && active) {
#pragma unroll
    for (int k = 0; k < V; ++k) { mu[k] = mean[c0 + k]; is[k] = invstd[c0 + k]; }
  }
  if (active) {
    for (long long r = (long long)blockIdx.x * BN_RY + threadIdx.y; r < M; r += (long long)gridDim.x * BN_RY) {
      float xv[V];
      Vec<T>::load(x + r * C + c0, xv);
      if (MODE == 0) {
#pragma unroll
        for (int k = 0; k < V; ++k) { sa[k] += xv[k]; sb[k] += xv[k] * xv[k]; }
      } else {
        float dv[V];
        Vec<T>::load(dy + r * C + c0, dv);
        if (y != nullptr) {
          float yv[V];
          Vec<T>::load(y + r * C + c0, yv);
#pragma unroll
          for (int k = 0; k < V; ++k) dv[k] = yv[k] > 0.f ? dv[k] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < V; ++k) { sa[k] += dv[k]; sb[k] += dv[k] * (xv[k] - mu[k]) * is[k]; }
      }
    }
  }
  __shared__ float red[2][BN_RY][BN_CX][Vec<T>::N + 1];
#pragma unroll
  for (int k = 0; k < V; ++k) { red[0][threadIdx.y][threadIdx.x][k] = sa[k]; red[1][threadIdx.y][threadIdx.x][k] = sb[k]; }
  __syncthreads();
  if (threadIdx.y == 0 && active) {
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int j = 0; j < BN_RY; ++j) { a += red[0][j][threadIdx.x][k]; b += red[1][j][threadIdx.x][k]; }
      atomicAdd(&sums[c0 + k], a);
      atomicAdd(&sums[C + c0 + k], b);
    }
  }
}

__global__ void bn_finalize_kernel(const float* __restrict__ sums, const float* __restrict__ gamma, const float* __restrict__ beta,
                                   float* __restrict__ moving_mean, float* __restrict__ moving_var, float momentum, float eps, float inv_m,
                                   int C, float* __restrict__ mean_out, float* __restrict__ invstd_out, float* __restrict__ scale_out,
                                   float* __restrict__ shift_out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float mean = sums[c] * inv_m;
  const float var = fmaxf(sums[C + c] * inv_m - mean * mean, 0.f);
  const float invstd = rsqrtf(var + eps);
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  mean_out[c] = mean;
  invstd_out[c] = invstd;
  scale_out[c] = g * invstd;
  shift_out[c] = b - mean * g * invstd;
  if (moving_mean) moving_mean[c] = moving_mean[c] * momentum + mean * (1.f - momentum);
  if (moving_var) moving_var[c] = moving_var[c] * momentum + var * (1.f - momentum);
}

template <typename T>
__global__ void __launch_bounds__(256) bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ res, T* __restrict__ y,
                                                       const float* __restrict__ scale, const float* __restrict__ shift, long long nvec, int C,
                                                       int relu) {
  constexpr int V = Vec<T>::N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * V;
    const int c0 = (int)(e % C);
    float xv[V];
    Vec<T>::load(x + e, xv);
#pragma unroll
    for (int k = 0; k < V; ++k) xv[k] = xv[k] * scale[c0 + k] + shift[c0 + k];
    if (res != nullptr) {
      float rv[V];
      Vec<T>::load(res + e, rv);
#pragma unroll
      for (int k = 0; k < V; ++k) xv[k] += rv[k];
    }
    if (relu) {
#pragma unroll
      for (int k = 0; k < V; ++k) xv[k] = fmaxf(xv[k], 0.f);
    }
    Vec<T>::store(y + e, xv);
  }
}

// dx = scale * (dy' - sum_dy/M - xhat * sum_dy_xhat/M);  dres = dy'
template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y,
                                                           const float* __restrict__ mean, const float* __restrict__ invstd,
                                                           const float* __restrict__ gamma, const float* __restrict__ sums, T* __restrict__ dx,
                                                           T* __restrict__ dres, long long nvec, int C, float inv_m) {
  constexpr int V = Vec<T>::N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * V;
    const int c0 = (int)(e % C);
    float dv[V], xv[V], out[V];
    Vec<T>::load(dy + e, dv);
    Vec<T>::load(x + e, xv);
    if (y != nullptr) {
      float yv[V];
      Vec<T>::load(y + e, yv);
#pragma unroll
      for (int k = 0; k < V; ++k) dv[k] = yv[k] > 0.f ? dv[k] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int c = c0 + k;
      const float is = invstd[c];
      const float xhat = (xv[k] - mean[c]) * is;
      const float g = gamma ? gamma[c] : 1.f;
      out[k] = g * is * (dv[k] - sums[c] * inv_m - xhat * sums[C + c] * inv_m);
    }
    Vec<T>::store(dx + e, out);
    if (dres != nullptr) Vec<T>::store(dres + e, dv);
  }
}

static inline int bn_grid_rows(long long M, int col_tiles) {
  long long want = (148ll * 8 + col_tiles - 1) / col_tiles;
  long long maxb = (M + BN_RY - 1) / BN_RY;
  long long g = want < maxb ? want : maxb;
  return (int)(g < 1 ? 1 : g);
}

template <typename T>
static int bn_reduce_launch(int mode, const void* x, const void* dy, const void* y, const float* mean, const float* invstd, long long M, int C,
                            float* sums, cudaStream_t stream) {
  constexpr int V = Vec<T>::N;
  if (C % V != 0) { kb200_set_error("bn: C must be a multiple of the vector width"); return -2; }
  cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, stream);
  const int col_tiles = (C / V + BN_CX - 1) / BN_CX;
  dim3 grid(bn_grid_rows(M, col_tiles), col_tiles), block(BN_CX, BN_RY);
  if (mode == 0)
    bn_reduce_kernel<T, 0><<<grid, block, 0, stream>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, M, C, sums);
  else
    bn_reduce_kernel<T, 1><<<grid, block, 0, stream>>>((const T*)x, (const T*)dy, (const T*)y, mean, invstd, M, C, sums);
  KB_CHECK_LAUNCH("bn_reduce");
  return 0;
}

// dtype: 0 = float32, 1 = bfloat16
KB_API int kb200_bn_stats(const void* x, long long M, int C, int dtype, float* sums, cudaStream_t stream) {
  return dtype == 1 ? bn_reduce_launch<__nv_bfloat16>(0, x, nullptr, nullptr, nullptr, nullptr, M, C, sums, stream)
                    : bn_reduce_launch<float>(0, x, nullptr, nullptr, nullptr, nullptr, M, C, sums, stream);
}

KB_API int kb200_bn_finalize(const float* sums, const float* gamma, const float* beta, float* moving_mean, float* moving_var, float momentum,
                             float eps, long long M, int C, float* mean_out, float* invstd_out, float* scale_out, float* shift_out,
                             cudaStream_t stream) {
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, stream>>>(sums, gamma, beta, moving_mean, moving_var, momentum, eps, 1.f / (float)M, C, mean_out,
                                                          invstd_out, scale_out, shift_out);
  KB_CHECK_LAUNCH("bn_finalize");
  return 0;
}

KB_API int kb200_bn_apply(const void* x, const void* res, void* y, const float* scale, const float* shift, long long M, int C, int relu, int dtype,
                          cudaStream_t stream) {
  const int V = dtype == 1 ? 8 : 4;
  if (C % V != 0) { kb200_set_error("bn: C must be a multiple of the vector width"); return -2; }
  const long long nvec = M * C / V;
  int blocks = (int)((nvec + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == 1)
    bn_apply_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (__nv_bfloat16*)y, scale, shift, nvec, C, relu);
  else
    bn_apply_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, (const float*)res, (float*)y, scale, shift, nvec, C, relu);
  KB_CHECK_LAUNCH("bn_apply");
  return 0;
}

KB_API int kb200_bn_bwd_reduce(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, long long M, int C, int dtype,
                               float* sums, cudaStream_t stream) {
  return dtype == 1 ? bn_reduce_launch<__nv_bfloat16>(1, x, dy, y, mean, invstd, M, C, sums, stream)
                    : bn_reduce_launch<float>(1, x, dy, y, mean, invstd, M, C, sums, stream);
}

KB_API int kb200_bn_bwd_apply(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, const float* gamma,
                              const float* sums, void* dx, void* dres, long long M, int C, int dtype, cudaStream_t stream) {
  const int V = dtype == 1 ? 8 : 4;
  if (C % V != 0) { kb200_set_error("bn: C must be a multiple of the vector width"); return -2; }
  const long long nvec = M * C / V;
  int blocks = (int)((nvec + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  const float inv_m = 1.f / (float)M;
  if (dtype == 1)
    bn_bwd_apply_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, mean, invstd, gamma, sums,
                                                                  (__nv_bfloat16*)dx, (__nv_bfloat16*)dres, nvec, C, inv_m);
  else
    bn_bwd_apply_kernel<float><<<blocks, 256, 0, stream>>>((const float*)dy, (const float*)x, (const float*)y, mean, invstd, gamma, sums, (float*)dx, (float*)dres, nvec,
                                                          C, inv_m);
  KB_CHECK_LAUNCH("bn_bwd_apply");
  return 0;
}
