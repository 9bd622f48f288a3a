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

}  // namespace

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
  if (dtype == 1)
    fp8_quantize_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, rows, cols, scale, e5m2, (uint8_t*)q, ldq, (uint8_t*)qt,
                                                                 ldqt, amax);
  else
    fp8_quantize_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, ldx, rows, cols, scale, e5m2, (uint8_t*)q, ldq, (uint8_t*)qt, ldqt, amax);
  KB_CHECK_LAUNCH("fp8_quantize");
  return 0;
}
