// Quantisation of a bf16 / fp32 matrix to one-byte floating point (e4m3 or e5m2) for the fp8 tensor-core GEMM:
//   q[r, c] = fp8(saturate(x[r, c] / scale))
// written row-major (pitch ldq bytes) and, optionally, transposed (qt[c, r], pitch ldqt bytes) from the same read of x, and
// the absolute maximum of x accumulated into *amax (non-negative floats order like their bit patterns, so an integer
// atomic max does it).  Replaces the divide / clip / cast / cast-back / multiply chain of the reference's
// quantize_and_dequantize (keras/src/quantizers/quantizers.py:611-627) and the separate amax reduction (:598-608).
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr int QT = 64;  // tile edge

template <typename T>
__global__ void __launch_bounds__(256) fp8_quantize_kernel(const T* __restrict__ x, long long ldx, int rows, int cols, const float* __restrict__ scale,
                                                           int e5m2, uint8_t* __restrict__ q, long long ldq, uint8_t* __restrict__ qt, long long ldqt,
                                                           unsigned* __restrict__ amax) {
  __shared__ uint8_t tile[QT][QT + 4];
  __shared__ float red[32];
  const int r0 = blockIdx.y * QT, c0 = blockIdx.x * QT;
  const float inv = 1.f / __ldg(scale);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, each 4 columns x 4 rows
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty * 4 + i;
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + tx * 4 + j;
      float v = 0.f;
      if (r < rows && c < cols) v = to_f32<T>(x[(long long)r * ldx + c]);
      m = fmaxf(m, fabsf(v));
      const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3);
      packed |= (uint32_t)b << (8 * j);
      tile[ty * 4 + i][tx * 4 + j] = b;
    }
    if (q != nullptr && r < rows) {
      const int c = c0 + tx * 4;
      if (c + 3 < cols) {
        *reinterpret_cast<uint32_t*>(q + (long long)r * ldq + c) = packed;
      } else {
        for (int j = 0; j < 4; ++j)
          if (c + j < cols) q[(long long)r * ldq + c + j] = (uint8_t)(packed >> (8 * j));
      }
    }
  }
  if (qt != nullptr) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = c0 + ty * 4 + i;  // row of the transposed output
      if (c < cols) {
        const int r = r0 + tx * 4;
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) packed |= (uint32_t)tile[tx * 4 + j][ty * 4 + i] << (8 * j);
        if (r + 3 < rows) {
          *reinterpret_cast<uint32_t*>(qt + (long long)c * ldqt + r) = packed;
        } else {
          for (int j = 0; j < 4; ++j)
            if (r + j < rows) qt[(long long)c * ldqt + r + j] = (uint8_t)(packed >> (8 * j));
        }
      }
    }
  }
  if (amax != nullptr) {
    m = warp_max(m);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = m;
    __syncthreads();
    if (threadIdx.x < 8) {
      m = red[threadIdx.x];
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffu, m, o));
      if (threadIdx.x == 0) atomicMax(amax, __float_as_uint(m));
    }
  }
}


// Vector variant for 16-byte aligned rows (ldx a multiple of 8 elements, aligned base, output pitches multiples of 16):
// every thread converts 8 consecutive elements of a row per pass (one or two 16-byte loads, one 8-byte store) and the
// transposed tile leaves shared memory as 16-byte stores.
template <typename T>
__global__ void __launch_bounds__(256) fp8_quantize_vec_kernel(const T* __restrict__ x, long long ldx, int rows, int cols, const float* __restrict__ scale,
                                                               int e5m2, uint8_t* __restrict__ q, long long ldq, uint8_t* __restrict__ qt, long long ldqt,
                                                               unsigned* __restrict__ amax) {
  __shared__ __align__(16) uint8_t tile[QT][QT + 16];
  __shared__ float red[8];
  const int r0 = blockIdx.y * QT, c0 = blockIdx.x * QT;
  const float inv = 1.f / __ldg(scale);
  const int seg = threadIdx.x & 7, rl = threadIdx.x >> 3;  // 8 column segments of 8 elements, 32 rows per pass
  float m = 0.f;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int r = r0 + pass * 32 + rl, c = c0 + seg * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (r < rows && c < cols) {  // cols is a multiple of 8 here: a segment is inside or outside as a whole
      const T* src = x + (long long)r * ldx + c;
      if constexpr (sizeof(T) == 2) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          v[2 * j] = f.x;
          v[2 * j + 1] = f.y;
        }
      } else {
        const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      }
    }
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      m = fmaxf(m, fabsf(v[j]));
      const uint32_t b = __nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3);
      if (j < 4) lo |= b << (8 * j); else hi |= b << (8 * (j - 4));
    }
    *reinterpret_cast<uint2*>(&tile[pass * 32 + rl][seg * 8]) = make_uint2(lo, hi);
    if (q != nullptr && r < rows && c < cols) *reinterpret_cast<uint2*>(q + (long long)r * ldq + c) = make_uint2(lo, hi);
  }
  if (qt != nullptr) {
    __syncthreads();
    const int tc = threadIdx.x >> 2, ts = threadIdx.x & 3;  // transposed row (source column) and 16-row segment
    const int c = c0 + tc, r = r0 + ts * 16;
    if (c < cols && r < rows) {
      uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i >> 2] |= (uint32_t)tile[ts * 16 + i][tc] << (8 * (i & 3));
      if (r + 15 < rows) {
        *reinterpret_cast<uint4*>(qt + (long long)c * ldqt + r) = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
        for (int i = 0; i < 16; ++i)
          if (r + i < rows) qt[(long long)c * ldqt + r + i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
      }
    }
  }
  if (amax != nullptr) {
    m = warp_max(m);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = red[0];
#pragma unroll
      for (int k = 1; k < 8; ++k) t = fmaxf(t, red[k]);
      atomicMax(amax, __float_as_uint(t));
    }
  }
}

// Delayed-scaling bookkeeping of one tensor in one launch (the reference spends about nine elementwise kernels on it):
//   new_scale   = 1 / (dtype_max / max(history))      kept at `scale` when that maximum is 0 or not finite
//   new_history = history rolled by one towards the front, with the new max |x| in slot 0
// (keras/src/quantizers/quantizers.py:585-606).  `amax` holds float bits (as written by the quantise kernel).
__global__ void __launch_bounds__(256) fp8_delayed_scaling_kernel(const float* __restrict__ history, int length, const float* __restrict__ scale,
                                                                  const unsigned* __restrict__ amax, float dtype_max,
                                                                  float* __restrict__ new_scale, float* __restrict__ new_history) {
  __shared__ float red[8];
  float m = -INFINITY;
  bool nan = false;
  for (int i = threadIdx.x; i < length; i += 256) {
    const float h = history[i];
    nan |= h != h;
    m = fmaxf(m, h);
    new_history[i] = i == 0 ? __uint_as_float(*amax) : history[(i + 1 == length) ? 0 : i + 1];
  }
  // slot 0 of the rolled history is the old slot 1, then overwritten by the new amax: handled above; the last slot takes old slot 0
  m = nan ? NAN : m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, m, o);
    m = (m != m || other != other) ? NAN : fmaxf(m, other);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int k = 1; k < 8; ++k) t = (t != t || red[k] != red[k]) ? NAN : fmaxf(t, red[k]);
    const float old_sf = 1.f / *scale;
    float sf = dtype_max / t;
    if (!(t > 0.f)) sf = old_sf;     // zero (or NaN) maximum: keep the old scale factor
    if (!isfinite(t)) sf = old_sf;
    *new_scale = 1.f / sf;
  }
}

}  // namespace

// history: [length] fp32; scale: device scalar; amax: device word with float bits; outputs: new_scale [1], new_history [length].
KB_API int kb200_fp8_delayed_scaling(const float* history, int length, const float* scale, const unsigned* amax, float dtype_max, float* new_scale,
                                     float* new_history, cudaStream_t stream) {
  if (length <= 0) return 0;
  fp8_delayed_scaling_kernel<<<1, 256, 0, stream>>>(history, length, scale, amax, dtype_max, new_scale, new_history);
  KB_CHECK_LAUNCH("fp8_delayed_scaling");
  return 0;
}

// x: [rows, cols] bf16 (dtype 1) or fp32 (0) with row pitch ldx elements.  q: [rows, ldq] bytes or null; qt: [cols, ldqt] bytes or
// null (pitches multiples of 4).  scale: device scalar.  amax: device word, zeroed by the caller, receives max |x| as float bits.
KB_API int kb200_fp8_quantize(const void* x, long long ldx, int rows, int cols, const float* scale, int e5m2, void* q, long long ldq, void* qt,
                              long long ldqt, unsigned* amax, int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((q != nullptr && (ldq % 4 || ((uintptr_t)q & 3))) || (qt != nullptr && (ldqt % 4 || ((uintptr_t)qt & 3)))) {
    kb200_set_error("fp8_quantize: output pitches and pointers must be multiples of 4 bytes");
    return -2;
  }
  dim3 grid((cols + QT - 1) / QT, (rows + QT - 1) / QT);
  const bool vec = cols % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && (q == nullptr || (ldq % 16 == 0 && ((uintptr_t)q & 15) == 0)) &&
                   (qt == nullptr || (ldqt % 16 == 0 && ((uintptr_t)qt & 15) == 0));
  if (vec) {
    if (dtype == 1)
      fp8_quantize_vec_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, rows, cols, scale, e5m2, (uint8_t*)q, ldq,
                                                                       (uint8_t*)qt, ldqt, amax);
    else
      fp8_quantize_vec_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, ldx, rows, cols, scale, e5m2, (uint8_t*)q, ldq, (uint8_t*)qt, ldqt, amax);
    KB_CHECK_LAUNCH("fp8_quantize");
    return 0;
  }
  if (dtype == 1)
    fp8_quantize_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, rows, cols, scale, e5m2, (uint8_t*)q, ldq, (uint8_t*)qt,
                                                                 ldqt, amax);
  else
    fp8_quantize_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, ldx, rows, cols, scale, e5m2, (uint8_t*)q, ldq, (uint8_t*)qt, ldqt, amax);
  KB_CHECK_LAUNCH("fp8_quantize");
  return 0;
}
