// BatchNorm (training) for channels-last activations x[M, C], fused with ReLU and a residual add.
//
// Replaces the reference's chain of ~8 elementwise/reduction kernels in fp32
// (keras/src/backend/torch/nn.py:1020-1092, keras/src/layers/normalization/batch_normalization.py:345-399)
// by: one statistics pass (per-channel sum / sum of squares, fp32 accumulation, E[x^2]-E[x]^2
// variance as the reference), a C-sized finalize (scale/shift, moving statistics update) and one
// apply pass y = relu(x*scale + shift + residual) with bf16 or fp32 I/O.  Backward is one
// reduction pass, a C-sized coefficient kernel and one apply pass dx = A*dy' + B*x + C.
//
// All passes are HBM-bound.  Work split: a thread owns one 16-byte channel vector for the whole
// kernel (its per-channel coefficients live in registers, no index arithmetic per element) and
// walks rows with four independent 16-byte loads in flight per tensor.
#include "common.cuh"

template <typename T>
struct Vec;
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  using Raw = uint4;
  __device__ static Raw load_raw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  __device__ static void unpack(const Raw& r, float* f) { unpack8(reinterpret_cast<const bf16x8&>(r), f); }
  __device__ static void store(__nv_bfloat16* p, const float* f) { *reinterpret_cast<bf16x8*>(p) = pack8(f); }
};
template <>
struct Vec<float> {
  static constexpr int N = 4;
  using Raw = float4;
  __device__ static Raw load_raw(const float* p) { return *reinterpret_cast<const float4*>(p); }
  __device__ static void unpack(const Raw& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  __device__ static void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};

// bn_stream.cu: the two-input passes on a shared-memory ring fed by bulk copies (bf16); returns 1 when it does not apply
int kb200_bn_stream_launch(int mode, const void* in0, const void* in1, const unsigned char* bits_in, void* out0, void* out1, unsigned char* bits_out,
                           const float* p0, const float* p1, const float* p2, float* sums, long long M, int C, int relu, cudaStream_t stream);

template <typename T>
struct IsBf16 { static constexpr bool value = false; };
template <>
struct IsBf16<__nv_bfloat16> { static constexpr bool value = true; };

constexpr int BN_THREADS = 256;
constexpr int BN_U = 4;  // rows in flight per thread (apply and backward-reduce kernels)

struct BnGeom {
  int cx;       // channel vectors per block (power of two <= 32)
  int ry;       // row lanes per block = 256 / cx
  int gy;       // blocks along channels
  int gx;       // blocks along rows
};

static int bn_sm_count() { return kb_sm_count(); }

// Grid = one resident wave: `resident` blocks per SM (from the occupancy calculator), capped by the rows available.
static BnGeom bn_geom(long long M, int cvecs, int resident, int rows_per_iter) {
  BnGeom g;
  g.cx = 1;
  while (g.cx < 32 && g.cx < cvecs) g.cx <<= 1;
  g.ry = BN_THREADS / g.cx;
  g.gy = (cvecs + g.cx - 1) / g.cx;
  long long want = ((long long)bn_sm_count() * resident) / g.gy;
  if (want < 1) want = 1;
  long long maxb = (M + (long long)g.ry * rows_per_iter - 1) / ((long long)g.ry * rows_per_iter);
  long long gx = want < maxb ? want : maxb;
  g.gx = (int)(gx < 1 ? 1 : gx);
  return g;
}

template <typename K>
static int bn_resident_blocks(K kernel) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, BN_THREADS, 0) != cudaSuccess || n < 1) n = 2;
  return n;
}

// ReLU mask of a row vector: from the saved bit mask (one byte per thread vector), else from y > 0, else all ones.
template <typename T>
__device__ __forceinline__ unsigned bn_mask_bits(const typename Vec<T>::Raw& ry, bool have_y, const unsigned char* bits, long long vec_index) {
  constexpr int V = Vec<T>::N;
  if (bits != nullptr) return bits[vec_index];
  if (!have_y) return 0xffu;
  float yv[V];
  Vec<T>::unpack(ry, yv);
  unsigned m = 0;
#pragma unroll
  for (int k = 0; k < V; ++k) m |= (yv[k] > 0.f ? 1u : 0u) << k;
  return m;
}

// sums[0:C] += sum_rows a(row, c);  sums[C:2C] += sum_rows b(row, c)
// MODE 0 (forward stats): a = x, b = x*x
// MODE 1 (backward):      a = dy', b = dy' * xhat, dy' = dy * relu_mask
template <typename T, int MODE, int U>
__global__ void __launch_bounds__(BN_THREADS, 2) bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                                                              const unsigned char* __restrict__ bits, const float* __restrict__ mean,
                                                              const float* __restrict__ invstd, long long M, int C, int cx_log2,
                                                              float* __restrict__ sums) {
  constexpr int V = Vec<T>::N;
  const int cx = 1 << cx_log2, ry = BN_THREADS >> cx_log2;
  const int tx = threadIdx.x & (cx - 1), ty = threadIdx.x >> cx_log2;
  const int cvecs = C / V;
  const int cv = blockIdx.y * cx + tx;
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
    const long long step = (long long)gridDim.x * ry * U;
    for (long long r0 = (long long)blockIdx.x * ry * U + ty; r0 < M; r0 += step) {
      typename Vec<T>::Raw rx[U], rd[U], rm[U];
      unsigned mb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long r = r0 + (long long)u * ry;
        if (r < M) {
          rx[u] = Vec<T>::load_raw(x + r * C + c0);
          if (MODE == 1) {
            rd[u] = Vec<T>::load_raw(dy + r * C + c0);
            if (bits != nullptr) mb[u] = bits[r * cvecs + cv];
            else if (y != nullptr) rm[u] = Vec<T>::load_raw(y + r * C + c0);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (r0 + (long long)u * ry >= M) continue;
        float xv[V];
        Vec<T>::unpack(rx[u], xv);
        if (MODE == 0) {
#pragma unroll
          for (int k = 0; k < V; ++k) { sa[k] += xv[k]; sb[k] += xv[k] * xv[k]; }
        } else {
          float dv[V];
          Vec<T>::unpack(rd[u], dv);
          const unsigned m = bits != nullptr ? mb[u] : bn_mask_bits<T>(rm[u], y != nullptr, nullptr, 0);
#pragma unroll
          for (int k = 0; k < V; ++k) {
            const float d = ((m >> k) & 1u) ? dv[k] : 0.f;
            sa[k] += d;
            sb[k] += d * (xv[k] - mu[k]) * is[k];
          }
        }
      }
    }
  }
  // lanes of a warp that own the same channel vector differ by multiples of cx
#pragma unroll
  for (int k = 0; k < V; ++k) {
    for (int o = 16; o >= cx; o >>= 1) {
      sa[k] += __shfl_xor_sync(0xffffffffu, sa[k], o);
      sb[k] += __shfl_xor_sync(0xffffffffu, sb[k], o);
    }
  }
  __shared__ float red[BN_THREADS / 32][2][32 * V];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane < cx) {
#pragma unroll
    for (int k = 0; k < V; ++k) { red[warp][0][lane * V + k] = sa[k]; red[warp][1][lane * V + k] = sb[k]; }
  }
  __syncthreads();
  // warps whose lanes all map to tx = lane & (cx-1); every warp holds a partial for each of the cx vectors
  for (int i = threadIdx.x; i < 2 * cx * V; i += BN_THREADS) {
    const int which = i / (cx * V), j = i % (cx * V);
    const int c = (blockIdx.y * cx) * V + j;
    if (c < C) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < BN_THREADS / 32; ++w) a += red[w][which][j];
      atomicAdd(&sums[which * C + c], a);
    }
  }
}

// pre_bias: bias of the producing convolution that was folded away (the normalised output does not
// depend on it; only the moving mean does).
__global__ void bn_finalize_kernel(const float* __restrict__ sums, const float* __restrict__ gamma, const float* __restrict__ beta,
                                   const float* __restrict__ pre_bias, float* __restrict__ moving_mean, float* __restrict__ moving_var,
                                   float momentum, float eps, float inv_m, int C, float* __restrict__ mean_out, float* __restrict__ invstd_out,
                                   float* __restrict__ scale_out, float* __restrict__ shift_out) {
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
  const float full_mean = mean + (pre_bias ? pre_bias[c] : 0.f);
  if (moving_mean) moving_mean[c] = moving_mean[c] * momentum + full_mean * (1.f - momentum);
  if (moving_var) moving_var[c] = moving_var[c] * momentum + var * (1.f - momentum);
}

// As bn_finalize_kernel, with the per-channel sums gathered from the per-warp partials that the convolution epilogue
// (conv_sm100.cu) leaves behind: partials[cta][2][ld]; CTA `cta` covers channels [(cta % n_tiles) * bn, + bn).
// One warp per channel; the order of the additions is fixed, so the result is reproducible bit for bit.
__global__ void bn_finalize_partials_kernel(const float* __restrict__ partials, int grid, int n_tiles, int bn, int ld,
                                            const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ pre_bias,
                                            float* __restrict__ moving_mean, float* __restrict__ moving_var, float momentum, float eps, float inv_m,
                                            int C, float* __restrict__ mean_out, float* __restrict__ invstd_out, float* __restrict__ scale_out,
                                            float* __restrict__ shift_out) {
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= C) return;
  const int ntile = c / bn;
  const int count = ntile < grid ? (grid - 1 - ntile) / n_tiles + 1 : 0;
  float s = 0.f, q = 0.f;
  for (int i = lane; i < count; i += 32) {
    const int b = ntile + i * n_tiles;
    const float* src = partials + (size_t)b * 2 * ld + c;
    s += src[0];
    q += src[ld];
  }
  s = warp_sum(s);
  q = warp_sum(q);
  if (lane != 0) return;
  const float mean = s * inv_m;
  const float var = fmaxf(q * inv_m - mean * mean, 0.f);
  const float invstd = rsqrtf(var + eps);
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  mean_out[c] = mean;
  invstd_out[c] = invstd;
  scale_out[c] = g * invstd;
  shift_out[c] = b - mean * g * invstd;
  const float full_mean = mean + (pre_bias ? pre_bias[c] : 0.f);
  if (moving_mean) moving_mean[c] = moving_mean[c] * momentum + full_mean * (1.f - momentum);
  if (moving_var) moving_var[c] = moving_var[c] * momentum + var * (1.f - momentum);
}

// Backward coefficients: dx = A*dy' + B*x + Cc
// dgamma_acc / dbeta_acc (optional): persistent gradient storage of gamma and beta; the sums are added there as well
__global__ void bn_bwd_coeff_kernel(const float* __restrict__ sums, const float* __restrict__ gamma, const float* __restrict__ mean,
                                    const float* __restrict__ invstd, float inv_m, int C, float* __restrict__ coef, float* __restrict__ dgamma_acc,
                                    float* __restrict__ dbeta_acc) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (dgamma_acc != nullptr) dgamma_acc[c] += sums[C + c];
  if (dbeta_acc != nullptr) dbeta_acc[c] += sums[c];
  const float g = gamma ? gamma[c] : 1.f, is = invstd[c], mu = mean[c];
  const float s1 = sums[c] * inv_m, s2 = sums[C + c] * inv_m;
  const float a = g * is;
  coef[c] = a;
  coef[C + c] = -a * is * s2;
  coef[2 * C + c] = a * (mu * is * s2 - s1);
}

// MODE 0: y  = relu?(x*p0 + p1 (+ res)), bits = (y > 0)      (p0 = scale, p1 = shift)
// MODE 1: dx = p0*dy' + p1*x + p2, dres = dy'                 (in0 = dy, in1 = x, mask from bits or y)
// U rows in flight per thread: 4, or 8 for the forward pass without a residual input (one stream of loads only)
template <typename T, int MODE, int U = BN_U>
__global__ void __launch_bounds__(BN_THREADS, 2) bn_apply_kernel(const T* __restrict__ in0, const T* __restrict__ in1, const T* __restrict__ ymask,
                                                             unsigned char* __restrict__ bits, T* __restrict__ out0, T* __restrict__ out1,
                                                             const float* __restrict__ p0, const float* __restrict__ p1,
                                                             const float* __restrict__ p2, long long M, int C, int cx_log2, int relu) {
  constexpr int V = Vec<T>::N;
  // the 8-row instance is the forward pass without a second input: known at compile time so that no registers are held for it
  const bool has1 = (U == 8) ? false : in1 != nullptr;
  const int cvecs = C / V;
  const int cx = 1 << cx_log2, ry = BN_THREADS >> cx_log2;
  const int tx = threadIdx.x & (cx - 1), ty = threadIdx.x >> cx_log2;
  const int cv = blockIdx.y * cx + tx;
  if (cv >= C / V) return;
  const int c0 = cv * V;
  float a[V], b[V], cc[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    a[k] = p0[c0 + k];
    b[k] = p1[c0 + k];
    cc[k] = (MODE == 1) ? p2[c0 + k] : 0.f;
  }
  const long long step = (long long)gridDim.x * ry * U;
  for (long long r0 = (long long)blockIdx.x * ry * U + ty; r0 < M; r0 += step) {
    typename Vec<T>::Raw q0[U], q1[U], qm[U];
    unsigned mb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long r = r0 + (long long)u * ry;
      if (r < M) {
        const long long e = r * C + c0;
        q0[u] = Vec<T>::load_raw(in0 + e);
        if (has1) q1[u] = Vec<T>::load_raw(in1 + e);
        if (MODE == 1) {
          if (bits != nullptr) mb[u] = bits[r * cvecs + cv];
          else if (ymask != nullptr) qm[u] = Vec<T>::load_raw(ymask + e);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long r = r0 + (long long)u * ry;
      if (r >= M) continue;
      const long long e = r * C + c0;
      float o[V], v0[V], v1[V];
      Vec<T>::unpack(q0[u], v0);
      if (has1) Vec<T>::unpack(q1[u], v1);
      if (MODE == 0) {
        unsigned m = 0;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          float t = v0[k] * a[k] + b[k];
          if (has1) t += v1[k];
          m |= (t > 0.f ? 1u : 0u) << k;
          o[k] = relu ? fmaxf(t, 0.f) : t;
        }
        Vec<T>::store(out0 + e, o);
        if (bits != nullptr) bits[r * cvecs + cv] = (unsigned char)m;
      } else {
        const unsigned m = bits != nullptr ? mb[u] : bn_mask_bits<T>(qm[u], ymask != nullptr, nullptr, 0);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const float d = ((m >> k) & 1u) ? v0[k] : 0.f;
          v0[k] = d;
          o[k] = a[k] * d + b[k] * v1[k] + cc[k];
        }
        Vec<T>::store(out0 + e, o);
        if (out1 != nullptr) Vec<T>::store(out1 + e, v0);
      }
    }
  }
}

static inline int ilog2(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}

template <typename T>
static int bn_reduce_launch(int mode, const void* x, const void* dy, const void* y, const unsigned char* bits, const float* mean,
                            const float* invstd, long long M, int C, float* sums, cudaStream_t stream) {
  constexpr int V = Vec<T>::N;
  constexpr int U0 = 8;
  if (C % V != 0) { kb200_set_error("bn: C must be a multiple of the vector width"); return -2; }
  cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, stream);
  if (mode == 0) {
    static const int resident = bn_resident_blocks(bn_reduce_kernel<T, 0, U0>);
    const BnGeom g = bn_geom(M, C / V, resident, U0);
    bn_reduce_kernel<T, 0, U0><<<dim3(g.gx, g.gy), BN_THREADS, 0, stream>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, nullptr, M, C,
                                                                           ilog2(g.cx), sums);
  } else {
    if (IsBf16<T>::value && y == nullptr) {
      const int rc = kb200_bn_stream_launch(1, dy, x, bits, nullptr, nullptr, nullptr, mean, invstd, nullptr, sums, M, C, 0, stream);
      if (rc <= 0) return rc;
    }
    static const int resident = bn_resident_blocks(bn_reduce_kernel<T, 1, BN_U>);
    const BnGeom g = bn_geom(M, C / V, resident, BN_U);
    bn_reduce_kernel<T, 1, BN_U><<<dim3(g.gx, g.gy), BN_THREADS, 0, stream>>>((const T*)x, (const T*)dy, (const T*)y, bits, mean, invstd, M, C,
                                                                             ilog2(g.cx), sums);
  }
  KB_CHECK_LAUNCH("bn_reduce");
  return 0;
}

// dtype: 0 = float32, 1 = bfloat16
KB_API int kb200_bn_stats(const void* x, long long M, int C, int dtype, float* sums, cudaStream_t stream) {
  return dtype == 1 ? bn_reduce_launch<__nv_bfloat16>(0, x, nullptr, nullptr, nullptr, nullptr, nullptr, M, C, sums, stream)
                    : bn_reduce_launch<float>(0, x, nullptr, nullptr, nullptr, nullptr, nullptr, M, C, sums, stream);
}

KB_API int kb200_bn_finalize(const float* sums, const float* gamma, const float* beta, const float* pre_bias, float* moving_mean,
                             float* moving_var, float momentum, float eps, long long M, int C, float* mean_out, float* invstd_out,
                             float* scale_out, float* shift_out, cudaStream_t stream) {
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, stream>>>(sums, gamma, beta, pre_bias, moving_mean, moving_var, momentum, eps, 1.f / (float)M, C,
                                                          mean_out, invstd_out, scale_out, shift_out);
  KB_CHECK_LAUNCH("bn_finalize");
  return 0;
}

// Finalize from the convolution epilogue's partial sums (see bn_finalize_partials_kernel); `grid`, `n_tiles`, `bn` are
// the plan values that kb200_conv_igemm reported, `ld` the row pitch of `partials`.
KB_API int kb200_bn_finalize_partials(const float* partials, int grid, int n_tiles, int bn, int ld, const float* gamma, const float* beta,
                                      const float* pre_bias, float* moving_mean, float* moving_var, float momentum, float eps, long long M, int C,
                                      float* mean_out, float* invstd_out, float* scale_out, float* shift_out, cudaStream_t stream) {
  if (grid <= 0 || n_tiles <= 0 || bn <= 0 || C > n_tiles * bn || ld < n_tiles * bn) {
    kb200_set_error("bn_finalize_partials: inconsistent plan");
    return -2;
  }
  bn_finalize_partials_kernel<<<(C + 3) / 4, 128, 0, stream>>>(partials, grid, n_tiles, bn, ld, gamma, beta, pre_bias, moving_mean, moving_var, momentum,
                                                                eps, 1.f / (float)M, C, mean_out, invstd_out, scale_out, shift_out);
  KB_CHECK_LAUNCH("bn_finalize_partials");
  return 0;
}

template <typename T>
static int bn_apply_launch(const void* x, const void* res, void* y, unsigned char* bits, const float* scale, const float* shift, long long M,
                           int C, int relu, cudaStream_t stream) {
  constexpr int V = Vec<T>::N;
  if (C % V != 0) { kb200_set_error("bn: C must be a multiple of the vector width"); return -2; }
  if (res == nullptr) {
    static const int resident8 = bn_resident_blocks(bn_apply_kernel<T, 0, 8>);
    const BnGeom g8 = bn_geom(M, C / V, resident8, 8);
    bn_apply_kernel<T, 0, 8><<<dim3(g8.gx, g8.gy), BN_THREADS, 0, stream>>>((const T*)x, nullptr, nullptr, bits, (T*)y, nullptr, scale, shift, nullptr,
                                                                           M, C, ilog2(g8.cx), relu);
    KB_CHECK_LAUNCH("bn_apply");
    return 0;
  }
  if (IsBf16<T>::value) {
    const int rc = kb200_bn_stream_launch(0, x, res, nullptr, y, nullptr, bits, scale, shift, nullptr, nullptr, M, C, relu, stream);
    if (rc <= 0) return rc;
  }
  static const int resident = bn_resident_blocks(bn_apply_kernel<T, 0>);
  const BnGeom g = bn_geom(M, C / V, resident, BN_U);
  bn_apply_kernel<T, 0><<<dim3(g.gx, g.gy), BN_THREADS, 0, stream>>>((const T*)x, (const T*)res, nullptr, bits, (T*)y, nullptr, scale, shift,
                                                                    nullptr, M, C, ilog2(g.cx), relu);
  KB_CHECK_LAUNCH("bn_apply");
  return 0;
}

KB_API int kb200_bn_apply(const void* x, const void* res, void* y, const float* scale, const float* shift, long long M, int C, int relu, int dtype,
                          cudaStream_t stream) {
  return dtype == 1 ? bn_apply_launch<__nv_bfloat16>(x, res, y, nullptr, scale, shift, M, C, relu, stream)
                    : bn_apply_launch<float>(x, res, y, nullptr, scale, shift, M, C, relu, stream);
}

// As kb200_bn_apply, and also writes the ReLU mask: one byte per 16-byte vector of y (bit k = element k > 0),
// M * C / V bytes with V = 8 (bf16) or 4 (fp32).  The backward entry points read it instead of y.
KB_API int kb200_bn_apply_mask(const void* x, const void* res, void* y, unsigned char* bits, const float* scale, const float* shift, long long M,
                               int C, int relu, int dtype, cudaStream_t stream) {
  return dtype == 1 ? bn_apply_launch<__nv_bfloat16>(x, res, y, bits, scale, shift, M, C, relu, stream)
                    : bn_apply_launch<float>(x, res, y, bits, scale, shift, M, C, relu, stream);
}

KB_API int kb200_bn_bwd_reduce(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, long long M, int C, int dtype,
                               float* sums, cudaStream_t stream) {
  return dtype == 1 ? bn_reduce_launch<__nv_bfloat16>(1, x, dy, y, nullptr, mean, invstd, M, C, sums, stream)
                    : bn_reduce_launch<float>(1, x, dy, y, nullptr, mean, invstd, M, C, sums, stream);
}

template <typename T>
static int bn_bwd_apply_launch(const void* dy, const void* x, const void* y, const unsigned char* bits, const float* coef, void* dx, void* dres,
                               long long M, int C, cudaStream_t stream) {
  constexpr int V = Vec<T>::N;
  if (IsBf16<T>::value && y == nullptr) {
    const int rc = kb200_bn_stream_launch(2, dy, x, bits, dx, dres, nullptr, coef, coef + C, coef + 2 * C, nullptr, M, C, 0, stream);
    if (rc <= 0) return rc;
  }
  static const int resident = bn_resident_blocks(bn_apply_kernel<T, 1>);
  const BnGeom g = bn_geom(M, C / V, resident, BN_U);
  bn_apply_kernel<T, 1><<<dim3(g.gx, g.gy), BN_THREADS, 0, stream>>>((const T*)dy, (const T*)x, (const T*)y, const_cast<unsigned char*>(bits),
                                                                    (T*)dx, (T*)dres, coef, coef + C, coef + 2 * C, M, C, ilog2(g.cx), 0);
  KB_CHECK_LAUNCH("bn_bwd_apply");
  return 0;
}

static int bn_bwd_apply_any(const void* dy, const void* x, const void* y, const unsigned char* bits, const float* mean, const float* invstd,
                            const float* gamma, const float* sums, float* coef, void* dx, void* dres, long long M, int C, int dtype,
                            cudaStream_t stream, float* dgamma_acc = nullptr, float* dbeta_acc = nullptr) {
  const int V = dtype == 1 ? 8 : 4;
  if (C % V != 0) { kb200_set_error("bn: C must be a multiple of the vector width"); return -2; }
  bn_bwd_coeff_kernel<<<(C + 127) / 128, 128, 0, stream>>>(sums, gamma, mean, invstd, 1.f / (float)M, C, coef, dgamma_acc, dbeta_acc);
  KB_CHECK_LAUNCH("bn_bwd_coeff");
  return dtype == 1 ? bn_bwd_apply_launch<__nv_bfloat16>(dy, x, y, bits, coef, dx, dres, M, C, stream)
                    : bn_bwd_apply_launch<float>(dy, x, y, bits, coef, dx, dres, M, C, stream);
}

// coef: scratch of 3*C floats (written here)
KB_API int kb200_bn_bwd_apply(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, const float* gamma,
                              const float* sums, float* coef, void* dx, void* dres, long long M, int C, int dtype, cudaStream_t stream) {
  return bn_bwd_apply_any(dy, x, y, nullptr, mean, invstd, gamma, sums, coef, dx, dres, M, C, dtype, stream);
}

// Backward with the ReLU mask taken from the bit mask of kb200_bn_apply_mask (bits may be null: no ReLU).
KB_API int kb200_bn_bwd_reduce_mask(const void* dy, const void* x, const unsigned char* bits, const float* mean, const float* invstd, long long M,
                                    int C, int dtype, float* sums, cudaStream_t stream) {
  return dtype == 1 ? bn_reduce_launch<__nv_bfloat16>(1, x, dy, nullptr, bits, mean, invstd, M, C, sums, stream)
                    : bn_reduce_launch<float>(1, x, dy, nullptr, bits, mean, invstd, M, C, sums, stream);
}

KB_API int kb200_bn_bwd_apply_mask(const void* dy, const void* x, const unsigned char* bits, const float* mean, const float* invstd,
                                   const float* gamma, const float* sums, float* coef, void* dx, void* dres, long long M, int C, int dtype,
                                   cudaStream_t stream) {
  return bn_bwd_apply_any(dy, x, nullptr, bits, mean, invstd, gamma, sums, coef, dx, dres, M, C, dtype, stream);
}

// As kb200_bn_bwd_apply_mask; in addition the gradients of gamma and beta are ADDED into dgamma_acc / dbeta_acc (fp32 [C],
// either may be null): persistent gradient storage, so that no separate accumulation kernel runs.
KB_API int kb200_bn_bwd_apply_mask_acc(const void* dy, const void* x, const unsigned char* bits, const float* mean, const float* invstd,
                                       const float* gamma, const float* sums, float* coef, void* dx, void* dres, float* dgamma_acc,
                                       float* dbeta_acc, long long M, int C, int dtype, cudaStream_t stream) {
  return bn_bwd_apply_any(dy, x, nullptr, bits, mean, invstd, gamma, sums, coef, dx, dres, M, C, dtype, stream, dgamma_acc, dbeta_acc);
}
