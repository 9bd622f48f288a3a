// Memory-bound row and window kernels: softmax / log-softmax over the last axis with an optional additive mask (forward and
// backward), embedding gather and its scatter-add gradient, channels-last average and global-average pooling (forward and
// backward), and bilinear / nearest image resizing.  Each replaces a chain of library kernels with up-casts in between:
//   softmax      keras/src/backend/torch/nn.py:159-196, keras/src/layers/activations/softmax.py (mask added as a large negative)
//   embedding    keras/src/layers/core/embedding.py:193-197 (take + cast; gradient = dense zeros + index_add)
//   pooling      keras/src/backend/torch/nn.py:361-533 (transposes to channels-first and back around the library call)
//   resize       keras/src/backend/torch/image.py (interpolate on a permuted view)
// All arithmetic is fp32; tensors are bf16 or fp32 (uint8 also for resize).
#include "common.cuh"

namespace {

constexpr int RO_THREADS = 256;

template <typename T>
struct RoVec {
  static constexpr int N = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void ro_load(const T* p, float* v) {
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
__device__ __forceinline__ void ro_store(T* p, const float* v) {
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

// A row is handled by one warp (BLOCK = false, several rows per CTA) or by one CTA (BLOCK = true).
template <bool BLOCK>
struct RowGroup {
  __device__ static int tid() { return BLOCK ? (int)threadIdx.x : (int)(threadIdx.x & 31); }
  __device__ static int size() { return BLOCK ? (int)blockDim.x : 32; }
  __device__ static long long row() {
    return BLOCK ? (long long)blockIdx.x : (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  }
  __device__ static float max(float v, float* red) { return BLOCK ? block_max(v, red) : warp_max(v); }
  __device__ static float sum(float v, float* red) { return BLOCK ? block_sum(v, red) : warp_sum(v); }
};

__device__ __forceinline__ void online(float v, float& m, float& s) {
  if (v > m) {
    s = s * __expf(m - v) + 1.f;
    m = v;
  } else {
    s += __expf(v - m);
  }
}

// ------------------------------------------------------------------------------------------------ softmax
// y = softmax(x + (mask ? 0 : masked_add)) over rows of C elements; LOG: log-softmax.  Two passes over the row: the second
// one finds it in L1/L2, so the memory system sees one read and one write.
template <typename T, bool BLOCK, bool LOG>
__global__ void __launch_bounds__(RO_THREADS) softmax_fwd_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask, T* __restrict__ y, long long rows,
                                                                 int C, float masked_add, int vec) {
  __shared__ float red[32];
  using G = RowGroup<BLOCK>;
  const long long row = G::row();
  if (!BLOCK && row >= rows) return;
  constexpr int VN = RoVec<T>::N;
  const T* xr = x + row * C;
  const uint8_t* mr = mask != nullptr ? mask + row * C : nullptr;
  T* yr = y + row * C;
  const int tid = G::tid(), step = G::size();
  const int body = vec ? (C / VN) * VN : 0;
  float m = -INFINITY, s = 0.f;
  for (int i = tid * VN; i < body; i += step * VN) {
    float v[VN];
    ro_load<T>(xr + i, v);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      if (mr != nullptr && !mr[i + j]) v[j] += masked_add;
      online(v[j], m, s);
    }
  }
  for (int i = body + tid; i < C; i += step) {
    float v = to_f32<T>(xr[i]);
    if (mr != nullptr && !mr[i]) v += masked_add;
    online(v, m, s);
  }
  const float gm = G::max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = G::sum(s, red);
  const float inv = 1.f / s, lse = gm + logf(s);
  for (int i = tid * VN; i < body; i += step * VN) {
    float v[VN];
    ro_load<T>(xr + i, v);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      if (mr != nullptr && !mr[i + j]) v[j] += masked_add;
      v[j] = LOG ? v[j] - lse : __expf(v[j] - gm) * inv;
    }
    ro_store<T>(yr + i, v);
  }
  for (int i = body + tid; i < C; i += step) {
    float v = to_f32<T>(xr[i]);
    if (mr != nullptr && !mr[i]) v += masked_add;
    yr[i] = from_f32<T>(LOG ? v - lse : __expf(v - gm) * inv);
  }
}

// softmax: dx = y * (dy - sum(dy * y));  log-softmax: dx = dy - exp(y) * sum(dy)
template <typename T, bool BLOCK, bool LOG>
__global__ void __launch_bounds__(RO_THREADS) softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, long long rows, int C,
                                                                 int vec) {
  __shared__ float red[32];
  using G = RowGroup<BLOCK>;
  const long long row = G::row();
  if (!BLOCK && row >= rows) return;
  constexpr int VN = RoVec<T>::N;
  const T* yr = y + row * C;
  const T* gr = dy + row * C;
  T* dr = dx + row * C;
  const int tid = G::tid(), step = G::size();
  const int body = vec ? (C / VN) * VN : 0;
  float acc = 0.f;
  for (int i = tid * VN; i < body; i += step * VN) {
    float a[VN], g[VN];
    ro_load<T>(yr + i, a);
    ro_load<T>(gr + i, g);
#pragma unroll
    for (int j = 0; j < VN; ++j) acc += LOG ? g[j] : g[j] * a[j];
  }
  for (int i = body + tid; i < C; i += step) {
    const float g = to_f32<T>(gr[i]);
    acc += LOG ? g : g * to_f32<T>(yr[i]);
  }
  const float total = G::sum(acc, red);
  for (int i = tid * VN; i < body; i += step * VN) {
    float a[VN], g[VN];
    ro_load<T>(yr + i, a);
    ro_load<T>(gr + i, g);
#pragma unroll
    for (int j = 0; j < VN; ++j) g[j] = LOG ? g[j] - __expf(a[j]) * total : a[j] * (g[j] - total);
    ro_store<T>(dr + i, g);
  }
  for (int i = body + tid; i < C; i += step) {
    const float a = to_f32<T>(yr[i]), g = to_f32<T>(gr[i]);
    dr[i] = from_f32<T>(LOG ? g - __expf(a) * total : a * (g - total));
  }
}

template <typename T>
int launch_softmax_fwd(const void* x, const uint8_t* mask, void* y, long long rows, int C, float masked_add, int log_mode, cudaStream_t stream) {
  const int vec = ((((uintptr_t)x | (uintptr_t)y) & 15) == 0 && ((long long)C * sizeof(T)) % 16 == 0) ? 1 : 0;
  const T* xi = (const T*)x;
  T* yo = (T*)y;
  if (C <= 2048) {
    const unsigned grid = (unsigned)((rows + RO_THREADS / 32 - 1) / (RO_THREADS / 32));
    if (log_mode) softmax_fwd_kernel<T, false, true><<<grid, RO_THREADS, 0, stream>>>(xi, mask, yo, rows, C, masked_add, vec);
    else softmax_fwd_kernel<T, false, false><<<grid, RO_THREADS, 0, stream>>>(xi, mask, yo, rows, C, masked_add, vec);
  } else {
    if (log_mode) softmax_fwd_kernel<T, true, true><<<(unsigned)rows, RO_THREADS, 0, stream>>>(xi, mask, yo, rows, C, masked_add, vec);
    else softmax_fwd_kernel<T, true, false><<<(unsigned)rows, RO_THREADS, 0, stream>>>(xi, mask, yo, rows, C, masked_add, vec);
  }
  return 0;
}

template <typename T>
int launch_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int C, int log_mode, cudaStream_t stream) {
  const int vec = ((((uintptr_t)y | (uintptr_t)dy | (uintptr_t)dx) & 15) == 0 && ((long long)C * sizeof(T)) % 16 == 0) ? 1 : 0;
  const T* yi = (const T*)y;
  const T* gi = (const T*)dy;
  T* dxo = (T*)dx;
  if (C <= 2048) {
    const unsigned grid = (unsigned)((rows + RO_THREADS / 32 - 1) / (RO_THREADS / 32));
    if (log_mode) softmax_bwd_kernel<T, false, true><<<grid, RO_THREADS, 0, stream>>>(yi, gi, dxo, rows, C, vec);
    else softmax_bwd_kernel<T, false, false><<<grid, RO_THREADS, 0, stream>>>(yi, gi, dxo, rows, C, vec);
  } else {
    if (log_mode) softmax_bwd_kernel<T, true, true><<<(unsigned)rows, RO_THREADS, 0, stream>>>(yi, gi, dxo, rows, C, vec);
    else softmax_bwd_kernel<T, true, false><<<(unsigned)rows, RO_THREADS, 0, stream>>>(yi, gi, dxo, rows, C, vec);
  }
  return 0;
}

}  // namespace

// dtype: 0 = fp32, 1 = bf16.  `mask` (or null): one byte per element, 0 = masked; masked elements get `masked_add` added.
KB_API int kb200_softmax_fwd(const void* x, const uint8_t* mask, void* y, long long rows, int C, float masked_add, int log_mode, int dtype,
                             cudaStream_t stream) {
  if (rows <= 0 || C <= 0) return 0;
  if (rows > 0x7fffffffLL) {
    kb200_set_error("softmax: too many rows");
    return -2;
  }
  if (dtype == 1) launch_softmax_fwd<__nv_bfloat16>(x, mask, y, rows, C, masked_add, log_mode, stream);
  else launch_softmax_fwd<float>(x, mask, y, rows, C, masked_add, log_mode, stream);
  KB_CHECK_LAUNCH("softmax_fwd");
  return 0;
}

KB_API int kb200_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int C, int log_mode, int dtype, cudaStream_t stream) {
  if (rows <= 0 || C <= 0) return 0;
  if (rows > 0x7fffffffLL) {
    kb200_set_error("softmax: too many rows");
    return -2;
  }
  if (dtype == 1) launch_softmax_bwd<__nv_bfloat16>(y, dy, dx, rows, C, log_mode, stream);
  else launch_softmax_bwd<float>(y, dy, dx, rows, C, log_mode, stream);
  KB_CHECK_LAUNCH("softmax_bwd");
  return 0;
}

// ------------------------------------------------------------------------------------------------ embedding
namespace {

// out[r, :] = table[ids[r], :] converted to the output type; one thread per 8 output elements.  Ids outside [0, V) give zeros.
template <typename TT, typename TO>
__global__ void __launch_bounds__(RO_THREADS) embedding_fwd_kernel(const TT* __restrict__ table, const long long* __restrict__ ids, TO* __restrict__ out,
                                                                   long long n, int D, long long V) {
  const int vpr = D >> 3;  // vectors of 8 elements per row
  const long long total = n * vpr;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / vpr;
    const int c = (int)(idx - r * vpr) << 3;
    const long long id = ids[r];
    float v[8];
    if (id >= 0 && id < V) {
      const TT* src = table + id * D + c;
      if constexpr (sizeof(TT) == 2) {
        ro_load<TT>(src, v);
      } else {
        ro_load<TT>(src, v);
        ro_load<TT>(src + 4, v + 4);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    TO* dst = out + r * D + c;
    if constexpr (sizeof(TO) == 2) {
      ro_store<TO>(dst, v);
    } else {
      ro_store<TO>(dst, v);
      ro_store<TO>(dst + 4, v + 4);
    }
  }
}

// dtable[ids[r], :] += dout[r, :] in fp32 (vector atomics: four floats per instruction).
template <typename TG>
__global__ void __launch_bounds__(RO_THREADS) embedding_bwd_kernel(const TG* __restrict__ dout, const long long* __restrict__ ids, float* __restrict__ dtable,
                                                                   long long n, int D, long long V) {
  const int vpr = D >> 3;
  const long long total = n * vpr;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / vpr;
    const int c = (int)(idx - r * vpr) << 3;
    const long long id = ids[r];
    if (id < 0 || id >= V) continue;
    float v[8];
    const TG* src = dout + r * D + c;
    if constexpr (sizeof(TG) == 2) {
      ro_load<TG>(src, v);
    } else {
      ro_load<TG>(src, v);
      ro_load<TG>(src + 4, v + 4);
    }
    float4* dst = reinterpret_cast<float4*>(dtable + id * D + c);
    atomicAdd(dst, make_float4(v[0], v[1], v[2], v[3]));
    atomicAdd(dst + 1, make_float4(v[4], v[5], v[6], v[7]));
  }
}

inline unsigned flat_grid(long long work_items) {
  long long blocks = (work_items + RO_THREADS - 1) / RO_THREADS;
  const long long cap = (long long)kb_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

}  // namespace

// table: [V, D] fp32 (table_dtype 0) or bf16 (1); out: [n, D] fp32 or bf16; D a multiple of 8, pointers 16-byte aligned.
KB_API int kb200_embedding_fwd(const void* table, const long long* ids, void* out, long long n, int D, long long V, int table_dtype, int out_dtype,
                               cudaStream_t stream) {
  if (n <= 0 || D <= 0) return 0;
  if ((D & 7) || (((uintptr_t)table | (uintptr_t)out) & 15)) {
    kb200_set_error("embedding_fwd: width must be a multiple of 8 and pointers 16-byte aligned");
    return -2;
  }
  const unsigned grid = flat_grid(n * (D >> 3));
  if (table_dtype == 1 && out_dtype == 1)
    embedding_fwd_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, n, D, V);
  else if (table_dtype == 0 && out_dtype == 1)
    embedding_fwd_kernel<float, __nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const float*)table, ids, (__nv_bfloat16*)out, n, D, V);
  else if (table_dtype == 0 && out_dtype == 0)
    embedding_fwd_kernel<float, float><<<grid, RO_THREADS, 0, stream>>>((const float*)table, ids, (float*)out, n, D, V);
  else
    embedding_fwd_kernel<__nv_bfloat16, float><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)table, ids, (float*)out, n, D, V);
  KB_CHECK_LAUNCH("embedding_fwd");
  return 0;
}

// dtable: fp32 [V, D], ADDED to (zero it for a plain gradient); dout: [n, D] fp32 (0) or bf16 (1).
KB_API int kb200_embedding_bwd(const void* dout, const long long* ids, float* dtable, long long n, int D, long long V, int grad_dtype, cudaStream_t stream) {
  if (n <= 0 || D <= 0) return 0;
  if ((D & 7) || (((uintptr_t)dout | (uintptr_t)dtable) & 15)) {
    kb200_set_error("embedding_bwd: width must be a multiple of 8 and pointers 16-byte aligned");
    return -2;
  }
  const unsigned grid = flat_grid(n * (D >> 3));
  if (grad_dtype == 1) embedding_bwd_kernel<__nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)dout, ids, dtable, n, D, V);
  else embedding_bwd_kernel<float><<<grid, RO_THREADS, 0, stream>>>((const float*)dout, ids, dtable, n, D, V);
  KB_CHECK_LAUNCH("embedding_bwd");
  return 0;
}

// ------------------------------------------------------------------------------------------------ average pooling (NHWC)
namespace {

// Window average over the elements inside the image (padding does not count): one thread per output pixel and 16-byte
// channel vector.
template <typename T>
__global__ void __launch_bounds__(RO_THREADS) avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int H, int W, int C, int OH, int OW, int KH,
                                                                 int KW, int SH, int SW, int PT, int PL) {
  constexpr int VN = RoVec<T>::N;
  const int cv = C / VN;
  const long long total = (long long)N * OH * OW * cv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % cv) * VN;
    long long t = idx / cv;
    const int ow = (int)(t % OW);
    t /= OW;
    const int oh = (int)(t % OH);
    const int n = (int)(t / OH);
    const int h0 = max(oh * SH - PT, 0), h1 = min(oh * SH - PT + KH, H);
    const int w0 = max(ow * SW - PL, 0), w1 = min(ow * SW - PL + KW, W);
    float acc[VN];
#pragma unroll
    for (int j = 0; j < VN; ++j) acc[j] = 0.f;
    for (int h = h0; h < h1; ++h)
      for (int w = w0; w < w1; ++w) {
        float v[VN];
        ro_load<T>(x + (((long long)n * H + h) * W + w) * C + c, v);
#pragma unroll
        for (int j = 0; j < VN; ++j) acc[j] += v[j];
      }
    const int cnt = (h1 - h0) * (w1 - w0);
    const float inv = cnt > 0 ? 1.f / (float)cnt : 0.f;
#pragma unroll
    for (int j = 0; j < VN; ++j) acc[j] *= inv;
    ro_store<T>(y + (((long long)n * OH + oh) * OW + ow) * C + c, acc);
  }
}

// dx[n, h, w, :] = sum over the windows that contain (h, w) of dy / (elements of that window inside the image).
template <typename T>
__global__ void __launch_bounds__(RO_THREADS) avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, int N, int H, int W, int C, int OH, int OW, int KH,
                                                                 int KW, int SH, int SW, int PT, int PL) {
  constexpr int VN = RoVec<T>::N;
  const int cv = C / VN;
  const long long total = (long long)N * H * W * cv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % cv) * VN;
    long long t = idx / cv;
    const int w = (int)(t % W);
    t /= W;
    const int h = (int)(t % H);
    const int n = (int)(t / H);
    // windows oh with oh*SH - PT <= h < oh*SH - PT + KH
    const int oh_lo = max((h + PT - KH + SH) / SH, 0), oh_hi = min((h + PT) / SH, OH - 1);
    const int ow_lo = max((w + PL - KW + SW) / SW, 0), ow_hi = min((w + PL) / SW, OW - 1);
    float acc[VN];
#pragma unroll
    for (int j = 0; j < VN; ++j) acc[j] = 0.f;
    for (int oh = oh_lo; oh <= oh_hi; ++oh) {
      const int hc = min(oh * SH - PT + KH, H) - max(oh * SH - PT, 0);
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const int wc = min(ow * SW - PL + KW, W) - max(ow * SW - PL, 0);
        const float inv = 1.f / (float)(hc * wc);
        float v[VN];
        ro_load<T>(dy + (((long long)n * OH + oh) * OW + ow) * C + c, v);
#pragma unroll
        for (int j = 0; j < VN; ++j) acc[j] += v[j] * inv;
      }
    }
    ro_store<T>(dx + idx * VN, acc);
  }
}

// y[n, :] = mean over the P pixels of x[n, :, :]: one thread per image and channel vector, consecutive threads on consecutive
// channel vectors.
template <typename T>
__global__ void __launch_bounds__(RO_THREADS) global_avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int P, int C) {
  constexpr int VN = RoVec<T>::N;
  const int cv = C / VN;
  const long long total = (long long)N * cv;
  const float inv = 1.f / (float)P;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % cv) * VN;
    const long long n = idx / cv;
    const T* src = x + n * (long long)P * C + c;
    float acc[VN];
#pragma unroll
    for (int j = 0; j < VN; ++j) acc[j] = 0.f;
#pragma unroll 4
    for (int p = 0; p < P; ++p) {
      float v[VN];
      ro_load<T>(src + (long long)p * C, v);
#pragma unroll
      for (int j = 0; j < VN; ++j) acc[j] += v[j];
    }
#pragma unroll
    for (int j = 0; j < VN; ++j) acc[j] *= inv;
    ro_store<T>(y + n * C + c, acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(RO_THREADS) global_avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, int N, int P, int C) {
  constexpr int VN = RoVec<T>::N;
  const int cv = C / VN;
  const long long total = (long long)N * P * cv;
  const float inv = 1.f / (float)P;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % cv) * VN;
    const long long n = idx / ((long long)P * cv);
    float v[VN];
    ro_load<T>(dy + n * C + c, v);
#pragma unroll
    for (int j = 0; j < VN; ++j) v[j] *= inv;
    ro_store<T>(dx + idx * VN, v);
  }
}

template <typename T>
bool pool_ok(const void* a, const void* b, int C) {
  return C % RoVec<T>::N == 0 && ((((uintptr_t)a | (uintptr_t)b) & 15) == 0);
}

}  // namespace

KB_API int kb200_avgpool2d_fwd(const void* x, void* y, int N, int H, int W, int C, int OH, int OW, int KH, int KW, int SH, int SW, int PT, int PL, int dtype,
                               cudaStream_t stream) {
  if (N <= 0 || OH <= 0 || OW <= 0 || C <= 0) return 0;
  if (!(dtype == 1 ? pool_ok<__nv_bfloat16>(x, y, C) : pool_ok<float>(x, y, C))) {
    kb200_set_error("avgpool2d: channels must fill 16-byte vectors and pointers be 16-byte aligned");
    return -2;
  }
  const int vn = dtype == 1 ? 8 : 4;
  const unsigned grid = flat_grid((long long)N * OH * OW * (C / vn));
  if (dtype == 1)
    avgpool_fwd_kernel<__nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, H, W, C, OH, OW, KH, KW, SH, SW, PT, PL);
  else
    avgpool_fwd_kernel<float><<<grid, RO_THREADS, 0, stream>>>((const float*)x, (float*)y, N, H, W, C, OH, OW, KH, KW, SH, SW, PT, PL);
  KB_CHECK_LAUNCH("avgpool2d_fwd");
  return 0;
}

KB_API int kb200_avgpool2d_bwd(const void* dy, void* dx, int N, int H, int W, int C, int OH, int OW, int KH, int KW, int SH, int SW, int PT, int PL, int dtype,
                               cudaStream_t stream) {
  if (N <= 0 || H <= 0 || W <= 0 || C <= 0) return 0;
  if (!(dtype == 1 ? pool_ok<__nv_bfloat16>(dy, dx, C) : pool_ok<float>(dy, dx, C))) {
    kb200_set_error("avgpool2d: channels must fill 16-byte vectors and pointers be 16-byte aligned");
    return -2;
  }
  const int vn = dtype == 1 ? 8 : 4;
  const unsigned grid = flat_grid((long long)N * H * W * (C / vn));
  if (dtype == 1)
    avgpool_bwd_kernel<__nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, N, H, W, C, OH, OW, KH, KW, SH, SW, PT, PL);
  else
    avgpool_bwd_kernel<float><<<grid, RO_THREADS, 0, stream>>>((const float*)dy, (float*)dx, N, H, W, C, OH, OW, KH, KW, SH, SW, PT, PL);
  KB_CHECK_LAUNCH("avgpool2d_bwd");
  return 0;
}

// x: [N, P, C] -> y: [N, C] (mean over P);  backward: dx[n, p, :] = dy[n, :] / P.
KB_API int kb200_global_avgpool_fwd(const void* x, void* y, int N, int P, int C, int dtype, cudaStream_t stream) {
  if (N <= 0 || P <= 0 || C <= 0) return 0;
  if (!(dtype == 1 ? pool_ok<__nv_bfloat16>(x, y, C) : pool_ok<float>(x, y, C))) {
    kb200_set_error("global_avgpool: channels must fill 16-byte vectors and pointers be 16-byte aligned");
    return -2;
  }
  const int vn = dtype == 1 ? 8 : 4;
  const unsigned grid = flat_grid((long long)N * (C / vn));
  if (dtype == 1) global_avgpool_fwd_kernel<__nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, P, C);
  else global_avgpool_fwd_kernel<float><<<grid, RO_THREADS, 0, stream>>>((const float*)x, (float*)y, N, P, C);
  KB_CHECK_LAUNCH("global_avgpool_fwd");
  return 0;
}

KB_API int kb200_global_avgpool_bwd(const void* dy, void* dx, int N, int P, int C, int dtype, cudaStream_t stream) {
  if (N <= 0 || P <= 0 || C <= 0) return 0;
  if (!(dtype == 1 ? pool_ok<__nv_bfloat16>(dy, dx, C) : pool_ok<float>(dy, dx, C))) {
    kb200_set_error("global_avgpool: channels must fill 16-byte vectors and pointers be 16-byte aligned");
    return -2;
  }
  const int vn = dtype == 1 ? 8 : 4;
  const unsigned grid = flat_grid((long long)N * P * (C / vn));
  if (dtype == 1) global_avgpool_bwd_kernel<__nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, N, P, C);
  else global_avgpool_bwd_kernel<float><<<grid, RO_THREADS, 0, stream>>>((const float*)dy, (float*)dx, N, P, C);
  KB_CHECK_LAUNCH("global_avgpool_bwd");
  return 0;
}

// ------------------------------------------------------------------------------------------------ image resize (NHWC)
namespace {

template <typename T>
__device__ __forceinline__ float px_load(const T* p) { return to_f32<T>(*p); }
template <>
__device__ __forceinline__ float px_load<uint8_t>(const uint8_t* p) { return (float)*p; }

template <typename T>
__device__ __forceinline__ T px_store(float v) { return from_f32<T>(v); }
template <>
__device__ __forceinline__ uint8_t px_store<uint8_t>(float v) { return (uint8_t)fminf(fmaxf(rintf(v), 0.f), 255.f); }

// mode 0: bilinear with half-pixel centres (source = (dst + 0.5) * in / out - 0.5, clamped at 0, neighbours clamped at the
// border); mode 1: nearest with half-pixel centres (source = floor((dst + 0.5) * in / out)).  One thread per output element.
template <typename TI, typename TO>
__global__ void __launch_bounds__(RO_THREADS) resize_kernel(const TI* __restrict__ x, TO* __restrict__ y, int N, int H, int W, int C, int OH, int OW,
                                                            float scale_h, float scale_w, int mode) {
  const long long total = (long long)N * OH * OW * C;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % C);
    long long t = idx / C;
    const int ow = (int)(t % OW);
    t /= OW;
    const int oh = (int)(t % OH);
    const long long n = t / OH;
    const TI* img = x + n * (long long)H * W * C + c;
    float out;
    if (mode == 1) {
      const int sh = min((int)floorf(((float)oh + 0.5f) * scale_h), H - 1);
      const int sw = min((int)floorf(((float)ow + 0.5f) * scale_w), W - 1);
      out = px_load<TI>(img + ((long long)sh * W + sw) * C);
    } else {
      const float fh = fmaxf(((float)oh + 0.5f) * scale_h - 0.5f, 0.f), fw = fmaxf(((float)ow + 0.5f) * scale_w - 0.5f, 0.f);
      const int h0 = min((int)fh, H - 1), w0 = min((int)fw, W - 1);
      const int h1 = min(h0 + 1, H - 1), w1 = min(w0 + 1, W - 1);
      const float lh = fh - (float)h0, lw = fw - (float)w0;
      const float v00 = px_load<TI>(img + ((long long)h0 * W + w0) * C), v01 = px_load<TI>(img + ((long long)h0 * W + w1) * C);
      const float v10 = px_load<TI>(img + ((long long)h1 * W + w0) * C), v11 = px_load<TI>(img + ((long long)h1 * W + w1) * C);
      out = (1.f - lh) * ((1.f - lw) * v00 + lw * v01) + lh * ((1.f - lw) * v10 + lw * v11);
    }
    y[idx] = px_store<TO>(out);
  }
}

}  // namespace

// dtype codes: 0 = fp32, 1 = bf16, 2 = uint8.  Supported pairs: same type in and out, and uint8 in with fp32 out.
KB_API int kb200_resize_nhwc(const void* x, void* y, int N, int H, int W, int C, int OH, int OW, int mode, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (N <= 0 || OH <= 0 || OW <= 0 || C <= 0 || H <= 0 || W <= 0) return 0;
  const float sh = (float)H / (float)OH, sw = (float)W / (float)OW;
  const unsigned grid = flat_grid((long long)N * OH * OW * C);
  if (in_dtype == 0 && out_dtype == 0)
    resize_kernel<float, float><<<grid, RO_THREADS, 0, stream>>>((const float*)x, (float*)y, N, H, W, C, OH, OW, sh, sw, mode);
  else if (in_dtype == 1 && out_dtype == 1)
    resize_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, RO_THREADS, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, H, W, C, OH, OW, sh, sw, mode);
  else if (in_dtype == 2 && out_dtype == 2)
    resize_kernel<uint8_t, uint8_t><<<grid, RO_THREADS, 0, stream>>>((const uint8_t*)x, (uint8_t*)y, N, H, W, C, OH, OW, sh, sw, mode);
  else if (in_dtype == 2 && out_dtype == 0)
    resize_kernel<uint8_t, float><<<grid, RO_THREADS, 0, stream>>>((const uint8_t*)x, (float*)y, N, H, W, C, OH, OW, sh, sw, mode);
  else {
    kb200_set_error("resize: unsupported type pair");
    return -2;
  }
  KB_CHECK_LAUNCH("resize_nhwc");
  return 0;
}

// ------------------------------------------------------------------------------------------------ int8 row quantisation
namespace {

template <typename T>
__device__ __forceinline__ float round_like(float v);
template <>
__device__ __forceinline__ float round_like<float>(float v) { return v; }
template <>
__device__ __forceinline__ float round_like<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Dynamic per-row quantisation of activations (keras/src/quantizers/quantizers.py:60-117, abs_max_quantize over the last
// axis): scale = qmax / (max|x| + eps), q = clip(round(x * scale), -qmax, qmax).  Every intermediate is rounded to the
// tensor's own type as the chain of library ops would round it, so the codes are the ones that chain produces.
// Outputs: q int8 [rows, K]; scale [rows] in the tensor's type; inv_scale [rows] fp32 (= 1 / scale, what the GEMM epilogue
// multiplies by).
template <typename T, bool BLOCK>
__global__ void __launch_bounds__(RO_THREADS) int8_quantize_rows_kernel(const T* __restrict__ x, int8_t* __restrict__ q, T* __restrict__ scale_out,
                                                                        float* __restrict__ inv_out, long long rows, int K, float eps, float qmax, int vec) {
  __shared__ float red[32];
  using G = RowGroup<BLOCK>;
  const long long row = G::row();
  if (!BLOCK && row >= rows) return;
  constexpr int VN = RoVec<T>::N;
  const T* xr = x + row * K;
  int8_t* qr = q + row * K;
  const int tid = G::tid(), step = G::size();
  const int body = vec ? (K / VN) * VN : 0;
  float m = 0.f;
  for (int i = tid * VN; i < body; i += step * VN) {
    float v[VN];
    ro_load<T>(xr + i, v);
#pragma unroll
    for (int j = 0; j < VN; ++j) m = fmaxf(m, fabsf(v[j]));
  }
  for (int i = body + tid; i < K; i += step) m = fmaxf(m, fabsf(to_f32<T>(xr[i])));
  m = G::max(m, red);
  // qmax / d is evaluated as (1 / d) * qmax, each step rounded to the tensor's type: that is how the library forms it
  const float scale = round_like<T>(round_like<T>(__frcp_rn(round_like<T>(m + eps))) * qmax);
  if (tid == 0) {
    scale_out[row] = from_f32<T>(scale);
    inv_out[row] = __fdiv_rn(1.f, scale);
  }
  for (int i = tid * VN; i < body; i += step * VN) {
    float v[VN];
    ro_load<T>(xr + i, v);
    if constexpr (VN == 8) {
      int8_t o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (int8_t)fminf(fmaxf(rintf(round_like<T>(v[j] * scale)), -qmax), qmax);
      *reinterpret_cast<uint2*>(qr + i) = *reinterpret_cast<const uint2*>(o);
    } else {
      int8_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = (int8_t)fminf(fmaxf(rintf(round_like<T>(v[j] * scale)), -qmax), qmax);
      *reinterpret_cast<uint32_t*>(qr + i) = *reinterpret_cast<const uint32_t*>(o);
    }
  }
  for (int i = body + tid; i < K; i += step) qr[i] = (int8_t)fminf(fmaxf(rintf(round_like<T>(to_f32<T>(xr[i]) * scale)), -qmax), qmax);
}

template <typename T>
void launch_int8_rows(const void* x, int8_t* q, void* scale, float* inv, long long rows, int K, float eps, float qmax, cudaStream_t stream) {
  // vector path: 16-byte loads and 8- or 4-byte stores, so K must keep every row of x and q aligned
  const int vec = ((((uintptr_t)x) & 15) == 0 && (((uintptr_t)q) & 7) == 0 && ((long long)K * sizeof(T)) % 16 == 0 && K % 8 == 0) ? 1 : 0;
  if (K <= 4096) {
    const unsigned grid = (unsigned)((rows + RO_THREADS / 32 - 1) / (RO_THREADS / 32));
    int8_quantize_rows_kernel<T, false><<<grid, RO_THREADS, 0, stream>>>((const T*)x, q, (T*)scale, inv, rows, K, eps, qmax, vec);
  } else {
    int8_quantize_rows_kernel<T, true><<<(unsigned)rows, RO_THREADS, 0, stream>>>((const T*)x, q, (T*)scale, inv, rows, K, eps, qmax, vec);
  }
}

}  // namespace

KB_API int kb200_int8_quantize_rows(const void* x, void* q, void* scale, float* inv_scale, long long rows, int K, float eps, float qmax, int dtype,
                                    cudaStream_t stream) {
  if (rows <= 0 || K <= 0) return 0;
  if (rows > 0x7fffffffLL) {
    kb200_set_error("int8_quantize_rows: too many rows");
    return -2;
  }
  if (dtype == 1) launch_int8_rows<__nv_bfloat16>(x, (int8_t*)q, scale, inv_scale, rows, K, eps, qmax, stream);
  else launch_int8_rows<float>(x, (int8_t*)q, scale, inv_scale, rows, K, eps, qmax, stream);
  KB_CHECK_LAUNCH("int8_quantize_rows");
  return 0;
}
