// 2-D max pooling for channels-last activations x[N, H, W, C] with the zero (or -inf) padding folded in.
//
// The reference runs ZeroPadding2D as a fill plus a strided copy and then the backend's pooling
// (keras/src/layers/reshaping/zero_padding2d.py, keras/src/backend/torch/nn.py max_pool), i.e. the
// 3x3/2 stem pooling of ResNet reads and writes the 112x112x64 tensor three times forward and
// three times backward.  Here the padded tensor never exists: out-of-range window positions
// contribute the pad value directly, the forward pass stores the arg-max position inside the
// window (one byte per output element) and the backward pass is a gather over the <= ceil(k/s)^2
// windows that cover an input pixel, so dx is written exactly once and no atomics are needed.
#include "common.cuh"

namespace {

template <typename T>
struct PVec;
template <>
struct PVec<__nv_bfloat16> {
  static constexpr int N = 8;
  using Raw = uint4;
  using Idx = uint2;
  __device__ static void unpack(const Raw& r, float* f) { unpack8(reinterpret_cast<const bf16x8&>(r), f); }
  __device__ static Raw pack(const float* f) {
    bf16x8 p = pack8(f);
    return reinterpret_cast<const uint4&>(p);
  }
};
template <>
struct PVec<float> {
  static constexpr int N = 4;
  using Raw = float4;
  using Idx = unsigned int;
  __device__ static void unpack(const Raw& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  __device__ static Raw pack(const float* f) { return make_float4(f[0], f[1], f[2], f[3]); }
};

struct PoolGeom {
  int N, H, W, C, OH, OW, kh, kw, sh, sw, pt, pl;
};

// pad_mode 0: positions outside the input are ignored (-inf); 1: they hold 0 (a folded ZeroPadding2D)
template <typename T>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, unsigned char* __restrict__ idx, PoolGeom g,
                                                          int pad_mode, long long total) {
  constexpr int V = PVec<T>::N;
  const int cvecs = g.C / V;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(t % cvecs);
    long long p = t / cvecs;
    const int ow = (int)(p % g.OW); p /= g.OW;
    const int oh = (int)(p % g.OH);
    const int n = (int)(p / g.OH);
    float best[V];
    unsigned char arg[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { best[k] = -INFINITY; arg[k] = 0; }
    for (int ki = 0; ki < g.kh; ++ki) {
      const int ih = oh * g.sh - g.pt + ki;
      for (int kj = 0; kj < g.kw; ++kj) {
        const int iw = ow * g.sw - g.pl + kj;
        const bool inside = ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
        if (!inside && pad_mode == 0) continue;
        float v[V];
        if (inside) {
          const typename PVec<T>::Raw raw =
              *reinterpret_cast<const typename PVec<T>::Raw*>(x + (((long long)n * g.H + ih) * g.W + iw) * g.C + (long long)cv * V);
          PVec<T>::unpack(raw, v);
        } else {
#pragma unroll
          for (int k = 0; k < V; ++k) v[k] = 0.f;
        }
        const unsigned char code = (unsigned char)(ki * g.kw + kj);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          if (v[k] > best[k] || v[k] != v[k]) { best[k] = v[k]; arg[k] = code; }
        }
      }
    }
    const long long o = t * V;
    *reinterpret_cast<typename PVec<T>::Raw*>(y + o) = PVec<T>::pack(best);
    typename PVec<T>::Idx packed;
    unsigned char* pb = reinterpret_cast<unsigned char*>(&packed);
#pragma unroll
    for (int k = 0; k < V; ++k) pb[k] = arg[k];
    *reinterpret_cast<typename PVec<T>::Idx*>(idx + o) = packed;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const T* __restrict__ dy, const unsigned char* __restrict__ idx, T* __restrict__ dx,
                                                          PoolGeom g, long long total) {
  constexpr int V = PVec<T>::N;
  const int cvecs = g.C / V;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(t % cvecs);
    long long p = t / cvecs;
    const int iw = (int)(p % g.W); p /= g.W;
    const int ih = (int)(p % g.H);
    const int n = (int)(p / g.H);
    const int ph = ih + g.pt, pw = iw + g.pl;
    int oh0 = ph - g.kh + 1;
    oh0 = oh0 <= 0 ? 0 : (oh0 + g.sh - 1) / g.sh;
    int ow0 = pw - g.kw + 1;
    ow0 = ow0 <= 0 ? 0 : (ow0 + g.sw - 1) / g.sw;
    const int oh1 = min(ph / g.sh, g.OH - 1), ow1 = min(pw / g.sw, g.OW - 1);
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
    for (int oh = oh0; oh <= oh1; ++oh) {
      for (int ow = ow0; ow <= ow1; ++ow) {
        const unsigned char code = (unsigned char)((ph - oh * g.sh) * g.kw + (pw - ow * g.sw));
        const long long o = ((((long long)n * g.OH + oh) * g.OW + ow) * cvecs + cv) * V;
        const typename PVec<T>::Idx packed = *reinterpret_cast<const typename PVec<T>::Idx*>(idx + o);
        const unsigned char* pb = reinterpret_cast<const unsigned char*>(&packed);
        bool any = false;
#pragma unroll
        for (int k = 0; k < V; ++k) any |= pb[k] == code;
        if (!any) continue;
        float d[V];
        PVec<T>::unpack(*reinterpret_cast<const typename PVec<T>::Raw*>(dy + o), d);
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] += pb[k] == code ? d[k] : 0.f;
      }
    }
    *reinterpret_cast<typename PVec<T>::Raw*>(dx + t * V) = PVec<T>::pack(acc);
  }
}

// Window known at compile time (3x3 stride 2, 2x2 stride 2): every load of a window is issued before the first compare,
// so a thread has KH*KW independent 16-byte loads in flight instead of one at a time.
template <typename T, int KH, int KW, int SH, int SW>
__global__ void __launch_bounds__(256) maxpool_fwd_fixed_kernel(const T* __restrict__ x, T* __restrict__ y, unsigned char* __restrict__ idx, PoolGeom g,
                                                                int pad_mode, long long total) {
  constexpr int V = PVec<T>::N;
  const int cvecs = g.C / V;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(t % cvecs);
    long long p = t / cvecs;
    const int ow = (int)(p % g.OW); p /= g.OW;
    const int oh = (int)(p % g.OH);
    const int n = (int)(p / g.OH);
    typename PVec<T>::Raw raw[KH * KW];
    bool inside[KH * KW];
#pragma unroll
    for (int ki = 0; ki < KH; ++ki) {
#pragma unroll
      for (int kj = 0; kj < KW; ++kj) {
        const int ih = oh * SH - g.pt + ki, iw = ow * SW - g.pl + kj;
        const bool in = ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
        inside[ki * KW + kj] = in;
        if (in) raw[ki * KW + kj] = *reinterpret_cast<const typename PVec<T>::Raw*>(x + (((long long)n * g.H + ih) * g.W + iw) * g.C + (long long)cv * V);
      }
    }
    float best[V];
    unsigned char arg[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { best[k] = -INFINITY; arg[k] = 0; }
#pragma unroll
    for (int w = 0; w < KH * KW; ++w) {
      if (!inside[w] && pad_mode == 0) continue;
      float v[V];
      if (inside[w]) {
        PVec<T>::unpack(raw[w], v);
      } else {
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] = 0.f;
      }
#pragma unroll
      for (int k = 0; k < V; ++k) {
        if (v[k] > best[k] || v[k] != v[k]) { best[k] = v[k]; arg[k] = (unsigned char)w; }
      }
    }
    const long long o = t * V;
    *reinterpret_cast<typename PVec<T>::Raw*>(y + o) = PVec<T>::pack(best);
    typename PVec<T>::Idx packed;
    unsigned char* pb = reinterpret_cast<unsigned char*>(&packed);
#pragma unroll
    for (int k = 0; k < V; ++k) pb[k] = arg[k];
    *reinterpret_cast<typename PVec<T>::Idx*>(idx + o) = packed;
  }
}

// At most NH x NW windows cover an input pixel (NH = ceil(KH / SH)): their arg-max codes and gradients are all loaded first.
template <typename T, int KH, int KW, int SH, int SW>
__global__ void __launch_bounds__(256) maxpool_bwd_fixed_kernel(const T* __restrict__ dy, const unsigned char* __restrict__ idx, T* __restrict__ dx,
                                                                PoolGeom g, long long total) {
  constexpr int V = PVec<T>::N;
  constexpr int NH = (KH + SH - 1) / SH, NW = (KW + SW - 1) / SW;
  const int cvecs = g.C / V;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(t % cvecs);
    long long p = t / cvecs;
    const int iw = (int)(p % g.W); p /= g.W;
    const int ih = (int)(p % g.H);
    const int n = (int)(p / g.H);
    const int ph = ih + g.pt, pw = iw + g.pl;
    const int oh1 = ph / SH, ow1 = pw / SW;  // the last window that can cover this pixel; earlier ones are oh1 - a, ow1 - b
    typename PVec<T>::Idx codes[NH * NW];
    typename PVec<T>::Raw grads[NH * NW];
    int want[NH * NW];
#pragma unroll
    for (int a = 0; a < NH; ++a) {
#pragma unroll
      for (int b = 0; b < NW; ++b) {
        const int oh = oh1 - a, ow = ow1 - b;
        const int ki = ph - oh * SH, kj = pw - ow * SW;
        const bool ok = oh >= 0 && oh < g.OH && ow >= 0 && ow < g.OW && ki < KH && kj < KW;
        want[a * NW + b] = ok ? ki * KW + kj : -1;
        if (ok) {
          const long long o = ((((long long)n * g.OH + oh) * g.OW + ow) * cvecs + cv) * V;
          codes[a * NW + b] = *reinterpret_cast<const typename PVec<T>::Idx*>(idx + o);
          grads[a * NW + b] = *reinterpret_cast<const typename PVec<T>::Raw*>(dy + o);
        }
      }
    }
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
#pragma unroll
    for (int w = 0; w < NH * NW; ++w) {
      if (want[w] < 0) continue;
      const unsigned char* pb = reinterpret_cast<const unsigned char*>(&codes[w]);
      float d[V];
      PVec<T>::unpack(grads[w], d);
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] += pb[k] == (unsigned char)want[w] ? d[k] : 0.f;
    }
    *reinterpret_cast<typename PVec<T>::Raw*>(dx + t * V) = PVec<T>::pack(acc);
  }
}

int pool_check(const PoolGeom& g, int dtype) {
  const int V = dtype == 1 ? 8 : 4;
  if (g.C % V != 0) { kb200_set_error("maxpool: C must be a multiple of the vector width"); return -2; }
  if (g.kh * g.kw > 255 || g.kh < 1 || g.kw < 1 || g.sh < 1 || g.sw < 1) { kb200_set_error("maxpool: unsupported window"); return -2; }
  return 0;
}

int pool_grid(long long total) {
  long long b = (total + 255) / 256;
  const long long cap = 148ll * 32;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

}  // namespace

// x[N,H,W,C] -> y[N,OH,OW,C], idx[N,OH,OW,C] (uint8: row-major position of the maximum inside the window).
// dtype: 0 = float32, 1 = bfloat16.
KB_API int kb200_maxpool2d_fwd(const void* x, void* y, unsigned char* idx, int N, int H, int W, int C, int OH, int OW, int kh, int kw, int sh,
                               int sw, int pad_top, int pad_left, int pad_mode, int dtype, cudaStream_t stream) {
  PoolGeom g{N, H, W, C, OH, OW, kh, kw, sh, sw, pad_top, pad_left};
  if (int rc = pool_check(g, dtype)) return rc;
  const long long total = (long long)N * OH * OW * (C / (dtype == 1 ? 8 : 4));
  if (total == 0) return 0;
  if (dtype == 1 && kh == 3 && kw == 3 && sh == 2 && sw == 2)
    maxpool_fwd_fixed_kernel<__nv_bfloat16, 3, 3, 2, 2><<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, idx, g, pad_mode,
                                                                                             total);
  else if (dtype == 1 && kh == 2 && kw == 2 && sh == 2 && sw == 2)
    maxpool_fwd_fixed_kernel<__nv_bfloat16, 2, 2, 2, 2><<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, idx, g, pad_mode,
                                                                                             total);
  else if (dtype == 1)
    maxpool_fwd_kernel<__nv_bfloat16><<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, idx, g, pad_mode, total);
  else
    maxpool_fwd_kernel<float><<<pool_grid(total), 256, 0, stream>>>((const float*)x, (float*)y, idx, g, pad_mode, total);
  KB_CHECK_LAUNCH("maxpool_fwd");
  return 0;
}

KB_API int kb200_maxpool2d_bwd(const void* dy, const unsigned char* idx, void* dx, int N, int H, int W, int C, int OH, int OW, int kh, int kw,
                               int sh, int sw, int pad_top, int pad_left, int dtype, cudaStream_t stream) {
  PoolGeom g{N, H, W, C, OH, OW, kh, kw, sh, sw, pad_top, pad_left};
  if (int rc = pool_check(g, dtype)) return rc;
  const long long total = (long long)N * H * W * (C / (dtype == 1 ? 8 : 4));
  if (total == 0) return 0;
  if (dtype == 1 && kh == 3 && kw == 3 && sh == 2 && sw == 2)
    maxpool_bwd_fixed_kernel<__nv_bfloat16, 3, 3, 2, 2><<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, g, total);
  else if (dtype == 1 && kh == 2 && kw == 2 && sh == 2 && sw == 2)
    maxpool_bwd_fixed_kernel<__nv_bfloat16, 2, 2, 2, 2><<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, g, total);
  else if (dtype == 1)
    maxpool_bwd_kernel<__nv_bfloat16><<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, g, total);
  else
    maxpool_bwd_kernel<float><<<pool_grid(total), 256, 0, stream>>>((const float*)dy, idx, (float*)dx, g, total);
  KB_CHECK_LAUNCH("maxpool_bwd");
  return 0;
}
