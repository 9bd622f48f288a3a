// LayerNorm / RMSNorm forward and backward over the last axis: rows x D, bf16 or fp32 I/O, fp32 math.
// Replaces F.layer_norm / F.rms_norm plus the two cast kernels around them
// (keras/src/ops/nn.py:3035-3069,3151-3210).
//
// Fast path (rows 16-byte aligned, D a multiple of the 16-byte vector, at most 8 vectors per lane): one warp per row,
// the row lives in registers as raw 16-byte vectors, statistics by warp shuffles only (mean first, then the centred
// second moment), one read and one write of every element.  Backward walks rows with a persistent grid, accumulates
// dgamma/dbeta per lane in registers, reduces them across the block's warps in shared memory and writes one partial
// row per block; a second kernel sums the partial rows (fixed order: deterministic).
// General path: one block per row with scalar accesses.
#include "common.cuh"

constexpr int NORM_THREADS = 256;
constexpr int NW_THREADS = 128;  // fast path: 4 warps = 4 rows per block

template <typename T>
struct NVec {
  static constexpr int N = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void nv_unpack(const uint4& raw, float* v) {
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
__device__ __forceinline__ uint4 nv_pack(const float* v) {
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
  return raw;
}

// VN consecutive fp32 parameters starting at a 16-byte aligned offset
template <int VN>
__device__ __forceinline__ void load_params(const float* __restrict__ p, int idx, float* out) {
#pragma unroll
  for (int q = 0; q < VN / 4; ++q) {
    const float4 f = __ldg(reinterpret_cast<const float4*>(p + idx) + q);
    out[4 * q] = f.x;
    out[4 * q + 1] = f.y;
    out[4 * q + 2] = f.z;
    out[4 * q + 3] = f.w;
  }
}

// A row is shared by WPR warps of an NT-thread block (WPR = 1: one warp per row, no block barrier at all); thread t of
// the row group owns vectors t, t + 32*WPR, ... (VPL of them, `nvec` valid in the row).
template <int NT, int WPR>
__device__ __forceinline__ float row_sum(float v, float* red, int row_in_block, int warp_in_row, int lane, int phase) {
  v = warp_sum(v);
  if constexpr (WPR == 1) {
    return v;
  } else {
    // `red`: [2 phases][rows per block][WPR]; alternating phases make one barrier per reduction enough
    float* slot = red + (phase * (NT / 32 / WPR) + row_in_block) * WPR;
    if (lane == 0) slot[warp_in_row] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w) r += slot[w];
    return r;
  }
}

template <typename T, int VPL, int NT, int WPR>
__global__ void __launch_bounds__(NT) norm_fwd_warp_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                           T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                           long long rows, int D, float eps, int rms) {
  constexpr int VN = NVec<T>::N;
  constexpr int RPB = NT / 32 / WPR;  // rows per block
  __shared__ float red[2 * RPB * WPR];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row_in_block = warp / WPR, warp_in_row = warp % WPR;
  const int t = warp_in_row * 32 + lane;
  long long row = (long long)blockIdx.x * RPB + row_in_block;
  const bool live = row < rows;
  if (WPR == 1 && !live) return;
  if (!live) row = rows - 1;  // keep the barriers uniform; results of the duplicate are not written
  const int nvec = D / VN;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  uint4 raw[VPL];
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = t + k * 32 * WPR;
    raw[k] = i < nvec ? __ldg(xr + i) : make_uint4(0, 0, 0, 0);
  }
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    float v[VN];
    nv_unpack<T>(raw[k], v);
#pragma unroll
    for (int j = 0; j < VN; ++j) s += v[j];
  }
  const float mean = rms ? 0.f : row_sum<NT, WPR>(s, red, row_in_block, warp_in_row, lane, 0) / D;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    if (t + k * 32 * WPR < nvec) {
      float v[VN];
      nv_unpack<T>(raw[k], v);
#pragma unroll
      for (int j = 0; j < VN; ++j) ss += (v[j] - mean) * (v[j] - mean);
    }
  }
  const float rstd = rsqrtf(row_sum<NT, WPR>(ss, red, row_in_block, warp_in_row, lane, 1) / D + eps);
  if (!live) return;
  if (t == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = t + k * 32 * WPR;
    if (i < nvec) {
      float v[VN], gv[VN], bv[VN];
      nv_unpack<T>(raw[k], v);
      if (gamma) load_params<VN>(gamma, i * VN, gv);
      if (beta) load_params<VN>(beta, i * VN, bv);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        float o = (v[j] - mean) * rstd;
        if (gamma) o *= gv[j];
        if (beta) o += bv[j];
        v[j] = o;
      }
      yr[i] = nv_pack<T>(v);
    }
  }
}

template <typename T, int VPL, int NT, int WPR>
__global__ void __launch_bounds__(NT) norm_bwd_warp_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                                                           const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                                                           float* __restrict__ partial_dgamma, float* __restrict__ partial_dbeta,
                                                           long long rows, int D, int rms) {
  constexpr int VN = NVec<T>::N;
  constexpr int RPB = NT / 32 / WPR;
  extern __shared__ float nsm[];  // [RPB][D] staging for the cross-row-group reduction of dgamma, then dbeta
  __shared__ float red[2 * RPB * WPR];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row_in_block = warp / WPR, warp_in_row = warp % WPR;
  const int t = warp_in_row * 32 + lane;
  const int nvec = D / VN;
  float dg[VPL * VN], db[VPL * VN];
#pragma unroll
  for (int k = 0; k < VPL; ++k)
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      dg[k * VN + j] = 0.f;
      db[k * VN + j] = 0.f;
    }
  const float inv_d = 1.f / D;
  // with WPR > 1 every warp of the block runs the same number of iterations (barriers inside row_sum)
  const long long stride = (long long)gridDim.x * RPB;
  const long long first = (long long)blockIdx.x * RPB;
  for (long long base = first; base < rows; base += stride) {
    long long row = base + row_in_block;
    const bool live = row < rows;
    if (WPR == 1 && !live) break;
    if (!live) row = rows - 1;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * D);
    uint4 xraw[VPL], draw[VPL];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int i = t + k * 32 * WPR;
      xraw[k] = i < nvec ? __ldg(xr + i) : make_uint4(0, 0, 0, 0);
      draw[k] = i < nvec ? __ldg(dyr + i) : make_uint4(0, 0, 0, 0);
    }
    const float mu = rms ? 0.f : mean[row];
    const float rs = rstd[row];
    const float keep = live ? 1.f : 0.f;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      if (t + k * 32 * WPR < nvec) {
        float xv[VN], dv[VN], gv[VN];
        nv_unpack<T>(xraw[k], xv);
        nv_unpack<T>(draw[k], dv);
        if (gamma) load_params<VN>(gamma, (t + k * 32 * WPR) * VN, gv);
#pragma unroll
        for (int j = 0; j < VN; ++j) {
          const float xhat = (xv[j] - mu) * rs;
          const float g = gamma ? gv[j] * dv[j] : dv[j];
          s1 += g;
          s2 += g * xhat;
          dg[k * VN + j] += keep * dv[j] * xhat;
          db[k * VN + j] += keep * dv[j];
        }
      }
    }
    const float m2 = row_sum<NT, WPR>(s2, red, row_in_block, warp_in_row, lane, 0) * inv_d;
    const float m1 = rms ? 0.f : row_sum<NT, WPR>(s1, red, row_in_block, warp_in_row, lane, 1) * inv_d;
    if (WPR > 1 && rms) __syncthreads();  // keep the two-phase alternation of `red` when the second reduction is skipped
    if (live) {
      uint4* dxr = reinterpret_cast<uint4*>(dx + row * D);
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int i = t + k * 32 * WPR;
        if (i < nvec) {
          float xv[VN], dv[VN], gv[VN];
          nv_unpack<T>(xraw[k], xv);
          nv_unpack<T>(draw[k], dv);
          if (gamma) load_params<VN>(gamma, i * VN, gv);
#pragma unroll
          for (int j = 0; j < VN; ++j) {
            const float xhat = (xv[j] - mu) * rs;
            const float g = gamma ? gv[j] * dv[j] : dv[j];
            dv[j] = rs * (g - m1 - xhat * m2);
          }
          dxr[i] = nv_pack<T>(dv);
        }
      }
    }
  }
  // reduction over the block's row groups, one quantity at a time through shared memory
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    float* out = pass == 0 ? partial_dgamma : partial_dbeta;
    if (out == nullptr) continue;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < VPL; ++k)
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        const int c = (t + k * 32 * WPR) * VN + j;
        if (c < D) nsm[row_in_block * D + c] = pass == 0 ? dg[k * VN + j] : db[k * VN + j];
      }
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += NT) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < RPB; ++w) s += nsm[w * D + c];
      out[(long long)blockIdx.x * D + c] = s;
    }
  }
}

// Sums `nblocks` partial rows of D columns: 32 columns x 32 row groups per block, four loads in flight per thread.
__global__ void __launch_bounds__(1024) norm_partial_reduce2_kernel(const float* __restrict__ pa, float* __restrict__ oa, const float* __restrict__ pb,
                                                                    float* __restrict__ ob, int nblocks, int D, int accumulate) {
  __shared__ float tile[32][33];
  const float* partial = blockIdx.y == 0 ? pa : pb;
  float* out = blockIdx.y == 0 ? oa : ob;
  if (partial == nullptr || out == nullptr) return;
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < D) {
    int b = ry;
    for (; b + 96 < nblocks; b += 128) {
      s0 += partial[(long long)b * D + c];
      s1 += partial[(long long)(b + 32) * D + c];
      s2 += partial[(long long)(b + 64) * D + c];
      s3 += partial[(long long)(b + 96) * D + c];
    }
    for (; b < nblocks; b += 32) s0 += partial[(long long)b * D + c];
  }
  tile[ry][cx] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (ry == 0 && c < D) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) s += tile[r][cx];
    out[c] = accumulate ? out[c] + s : s;
  }
}

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

__global__ void norm_partial_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int D, int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(long long)b * D + i];
  out[i] = accumulate ? out[i] + s : s;
}

KB_API int kb200_norm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, long long rows, int D, float eps,
                          int rms, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  {
    const int vn = dtype == 1 ? 8 : 4;
    const bool aligned = ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)beta) & 15) == 0) && D % vn == 0;
    const int nvec = aligned ? D / vn : 0;
    // shapes: (threads, warps per row); up to 8 vectors per thread
#define LAUNCH_FW(T, VPL, NT, WPR)                                                                                                                \
  do {                                                                                                                                            \
    constexpr int rpb = NT / 32 / WPR;                                                                                                            \
    norm_fwd_warp_kernel<T, VPL, NT, WPR><<<(unsigned)((rows + rpb - 1) / rpb), NT, 0, stream>>>((const T*)x, gamma, beta, (T*)y, mean, rstd,     \
                                                                                                  rows, D, eps, rms);                             \
  } while (0)
#define PICK_FW(T)                                                   \
  do {                                                               \
    if (nvec <= 32) LAUNCH_FW(T, 1, 128, 1);                         \
    else if (nvec <= 64) LAUNCH_FW(T, 2, 128, 1);                    \
    else if (nvec <= 128) LAUNCH_FW(T, 4, 128, 1);                   \
    else if (nvec <= 256) LAUNCH_FW(T, 2, 128, 4);                   \
    else if (nvec <= 512) LAUNCH_FW(T, 4, 128, 4);                   \
    else if (nvec <= 1024) LAUNCH_FW(T, 4, 256, 8);                  \
    else LAUNCH_FW(T, 8, 256, 8);                                    \
  } while (0)
    if (nvec >= 1 && nvec <= 2048) {
      if (dtype == 1) PICK_FW(__nv_bfloat16);
      else PICK_FW(float);
      KB_CHECK_LAUNCH("norm_fwd");
      return 0;
    }
#undef PICK_FW
#undef LAUNCH_FW
  }
  if (dtype == 1)
    norm_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, NORM_THREADS, 0, stream>>>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, D, eps, rms);
  else
    norm_fwd_kernel<float><<<(unsigned)rows, NORM_THREADS, 0, stream>>>((const float*)x, gamma, beta, (float*)y, mean, rstd, D, eps, rms);
  KB_CHECK_LAUNCH("norm_fwd");
  return 0;
}

KB_API int kb200_norm_bwd_blocks(long long rows) {
  long long b = 148 * 6;
  return (int)(rows < b ? rows : b);
}

// partial_dgamma / partial_dbeta: scratch [kb200_norm_bwd_blocks(rows), D] fp32; accumulate != 0: dgamma and dbeta are added to
KB_API int kb200_norm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx, float* partial_dgamma,
                          float* partial_dbeta, float* dgamma, float* dbeta, long long rows, int D, int rms, int dtype, int accumulate,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D > NORM_THREADS * 32) { kb200_set_error("norm_bwd: D too large (max 8192)"); return -2; }
  const int blocks = kb200_norm_bwd_blocks(rows);
  {
    const int vn = dtype == 1 ? 8 : 4;
    const bool aligned = ((((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx | (uintptr_t)gamma) & 15) == 0) && D % vn == 0;
    const int nvec = aligned ? D / vn : 0;
#define LAUNCH_BW(T, VPL, NT, WPR)                                                                                                                 \
  do {                                                                                                                                             \
    const size_t smem = (size_t)(NT / 32 / WPR) * D * sizeof(float);                                                                               \
    norm_bwd_warp_kernel<T, VPL, NT, WPR><<<blocks, NT, smem, stream>>>((const T*)dy, (const T*)x, gamma, mean, rstd, (T*)dx, partial_dgamma,      \
                                                                         partial_dbeta, rows, D, rms);                                             \
  } while (0)
    // per-thread accumulators: 2 x VPL x (8 or 4) floats, so at most 4 vectors per thread for bf16 and 8 for fp32
    bool done = true;
    if (dtype == 1) {
      if (nvec < 1) done = false;
      else if (nvec <= 32) LAUNCH_BW(__nv_bfloat16, 1, 128, 1);
      else if (nvec <= 64) LAUNCH_BW(__nv_bfloat16, 2, 128, 1);
      else if (nvec <= 128) LAUNCH_BW(__nv_bfloat16, 4, 128, 1);
      else if (nvec <= 256) LAUNCH_BW(__nv_bfloat16, 2, 128, 4);
      else if (nvec <= 512) LAUNCH_BW(__nv_bfloat16, 4, 128, 4);
      else if (nvec <= 1024) LAUNCH_BW(__nv_bfloat16, 4, 256, 8);
      else done = false;
    } else {
      if (nvec < 1) done = false;
      else if (nvec <= 32) LAUNCH_BW(float, 1, 128, 1);
      else if (nvec <= 64) LAUNCH_BW(float, 2, 128, 1);
      else if (nvec <= 128) LAUNCH_BW(float, 4, 128, 1);
      else if (nvec <= 256) LAUNCH_BW(float, 8, 128, 1);
      else if (nvec <= 512) LAUNCH_BW(float, 4, 128, 4);
      else if (nvec <= 1024) LAUNCH_BW(float, 8, 128, 4);
      else if (nvec <= 2048) LAUNCH_BW(float, 8, 256, 8);
      else done = false;
    }
#undef LAUNCH_BW
    if (done) {
      KB_CHECK_LAUNCH("norm_bwd");
      if (dgamma || (dbeta && partial_dbeta)) {
        dim3 grid((D + 31) / 32, 2);
        norm_partial_reduce2_kernel<<<grid, 1024, 0, stream>>>(dgamma ? partial_dgamma : nullptr, dgamma, partial_dbeta, dbeta, blocks, D, accumulate);
        KB_CHECK_LAUNCH("norm_partial_reduce");
      }
      return 0;
    }
  }
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
  if (dgamma) norm_partial_reduce_kernel<<<(D + 127) / 128, 128, 0, stream>>>(partial_dgamma, dgamma, blocks, D, accumulate);
  if (dbeta && partial_dbeta) norm_partial_reduce_kernel<<<(D + 127) / 128, 128, 0, stream>>>(partial_dbeta, dbeta, blocks, D, accumulate);
  KB_CHECK_LAUNCH("norm_partial_reduce");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Column sums of a [rows, cols] bf16/fp32 matrix into fp32 (bias gradients): blocks of 32 column vectors x 8 row lanes
// accumulate a slab of rows in registers, combine the row lanes through shared memory and write one partial row per
// slab; norm_partial_reduce2_kernel sums the slabs in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const T* __restrict__ x, long long ld, long long rows, int cols, float* __restrict__ partial) {
  constexpr int VN = NVec<T>::N;
  __shared__ float sm[8][32 * VN + 1];
  const int cv = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + cv) * VN;
  const long long per = (rows + gridDim.y - 1) / gridDim.y;
  const long long r0 = (long long)blockIdx.y * per, r1 = min(rows, r0 + per);
  float acc[VN];
#pragma unroll
  for (int j = 0; j < VN; ++j) acc[j] = 0.f;
  if (c0 < cols) {
    for (long long r = r0 + rl; r < r1; r += 8) {
      float v[VN];
      nv_unpack<T>(__ldg(reinterpret_cast<const uint4*>(x + r * ld + c0)), v);
#pragma unroll
      for (int j = 0; j < VN; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < VN; ++j) sm[rl][cv * VN + j] = acc[j];
  __syncthreads();
  for (int c = threadIdx.x; c < 32 * VN; c += 256) {
    const int col = blockIdx.x * 32 * VN + c;
    if (col < cols) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) s += sm[k][c];
      partial[(long long)blockIdx.y * cols + col] = s;
    }
  }
}

KB_API int kb200_colsum_slabs(long long rows, int cols, int dtype) {
  const int vn = dtype == 1 ? 8 : 4;
  const int col_blocks = (cols + 32 * vn - 1) / (32 * vn);
  long long slabs = (148 * 6 + col_blocks - 1) / col_blocks;
  if (slabs > (rows + 63) / 64) slabs = (rows + 63) / 64;
  if (slabs < 1) slabs = 1;
  if (slabs > 512) slabs = 512;
  return (int)slabs;
}

// x: [rows, cols] with row pitch ld (elements), cols a multiple of the 16-byte vector and rows 16-byte aligned;
// partial: scratch [kb200_colsum_slabs(rows, cols, dtype), cols] fp32; out: [cols] fp32.
// accumulate != 0: out += the sums (a bias gradient added into persistent storage).
KB_API int kb200_colsum(const void* x, long long ld, long long rows, int cols, float* partial, float* out, int dtype, int accumulate,
                        cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if (cols % vn || ld % vn || ((uintptr_t)x & 15)) {
    kb200_set_error("colsum: columns and pitch must be multiples of the 16-byte vector and the base pointer aligned");
    return -2;
  }
  const int slabs = kb200_colsum_slabs(rows, cols, dtype);
  dim3 grid((cols + 32 * vn - 1) / (32 * vn), slabs);
  if (dtype == 1)
    colsum_partial_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ld, rows, cols, partial);
  else
    colsum_partial_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, ld, rows, cols, partial);
  KB_CHECK_LAUNCH("colsum");
  dim3 grid2((cols + 31) / 32, 1);
  norm_partial_reduce2_kernel<<<grid2, 1024, 0, stream>>>(partial, out, nullptr, nullptr, slabs, cols, accumulate);
  KB_CHECK_LAUNCH("colsum_reduce");
  return 0;
}
