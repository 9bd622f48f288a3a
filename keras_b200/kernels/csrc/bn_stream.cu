// Streaming BatchNorm passes for bf16 activations x[M, C] that read TWO tensors per element: the forward apply with a
// residual input, the backward reduction (dy, x) and the backward apply (dy, x).
//
// With loads issued from registers these passes alternate between a load phase and an arithmetic phase and leave the
// memory system idle during the second; they reached about 4.2 TB/s where the one-input passes reach 6 TB/s.  Here a
// producer warp keeps a ring of shared-memory stages filled with bulk copies (cp.async.bulk, completion on an
// mbarrier): a tile is `tile_rows` whole rows, which is one contiguous range of a dense [M, C] tensor, so no tensor
// map is needed.  Sixteen consumer warps read the stages with conflict-free 16-byte shared loads; a thread owns one
// 16-byte channel vector for the whole kernel, as in the register kernels of bn.cu.  Several stages of 2 x 16 KB are
// in flight per SM all the time, independent of the register budget.
//
// Every mbarrier wait is bounded; a wait that runs out raises a device flag (kb200_bn_stream_status) and the block
// leaves its loops.  Formulas as bn.cu (keras/src/backend/torch/nn.py:1020-1092 for the forward definition).
#include "common.cuh"

namespace {

constexpr int BS_CONSUMERS = 512;
constexpr int BS_THREADS = BS_CONSUMERS + 32;
constexpr int BS_STAGES = 5;
constexpr int BS_TILE_BYTES = 16384;          // per input tensor and stage
constexpr uint32_t BS_SPIN_LIMIT = 1u << 20;  // try_wait calls (each suspends for a while) before a wait gives up

__device__ int g_bn_stream_status;  // 0 = fine; else 1 + index of the wait that ran out

struct BsParams {
  const __nv_bfloat16* in0;
  const __nv_bfloat16* in1;
  const unsigned char* bits_in;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  unsigned char* bits_out;
  const float* p0;
  const float* p1;
  const float* p2;
  float* sums;
  long long M;
  long long tiles;
  int C, cvecs, cv_log2;
  int rows_per_pass;  // BS_CONSUMERS / cvecs
  int tile_rows;      // multiple of rows_per_pass, tile_rows * C * 2 <= BS_TILE_BYTES
  int relu;
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  for (uint32_t it = 0; it < BS_SPIN_LIMIT; ++it) {
    if (bar_try(bar, parity)) return true;
    if ((it & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_bn_stream_status, 0, code);
  return false;
}
// contiguous global -> shared copy; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void bs_unpack8(const uint4& q, float* f) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 bs_pack8(const float* f) {
  uint4 q;
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(f[4], f[5]), d = __floats2bfloat162_rn(f[6], f[7]);
  q.x = *reinterpret_cast<uint32_t*>(&a);
  q.y = *reinterpret_cast<uint32_t*>(&b);
  q.z = *reinterpret_cast<uint32_t*>(&c);
  q.w = *reinterpret_cast<uint32_t*>(&d);
  return q;
}

// MODE 0: y = relu?(in0*p0 + p1 + in1), bits_out = (y > 0)                          in0 = x, in1 = residual
// MODE 1: sums[c] += sum d, sums[C + c] += p1[c] * sum d*(in1 - p0[c]),  d = mask ? in0 : 0   in0 = dy, in1 = x, p0 = mean, p1 = invstd
// MODE 2: out0 = p0*d + p1*in1 + p2, out1 = d (optional)                             in0 = dy, in1 = x
template <int MODE>
__global__ void __launch_bounds__(BS_THREADS, 1) bn_stream_kernel(const BsParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[BS_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[BS_STAGES];
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool stage_bits = MODE != 0 && p.bits_in != nullptr;
  const uint32_t bits_stage_bytes = (uint32_t)p.tile_rows * p.cvecs;  // a multiple of BS_CONSUMERS, hence of 16
  const uint32_t stage_bytes = 2u * BS_TILE_BYTES + (stage_bits ? bits_stage_bytes : 0u);
  if (tid == 0) {
    for (int s = 0; s < BS_STAGES; ++s) {
      bar_init(s_u32(&full_bar[s]), 1);
      bar_init(s_u32(&empty_bar[s]), BS_CONSUMERS / 32);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == BS_CONSUMERS / 32) {
    // ---- producer: one thread issues the copies of every tile this block owns
    if (lane == 0) {
      int it = 0;
      for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it) {
        const int s = it % BS_STAGES;
        if (it >= BS_STAGES && !bar_wait(s_u32(&empty_bar[s]), ((it / BS_STAGES) & 1) ^ 1, &abort_flag, 1)) break;
        const long long row0 = t * p.tile_rows;
        const long long rows = min((long long)p.tile_rows, p.M - row0);
        const uint32_t bytes = (uint32_t)(rows * p.C * 2);
        // the mask of a short last tile may not be a multiple of 16 bytes: its consumers read it from global memory
        const bool bits_here = stage_bits && rows == p.tile_rows;
        const uint32_t bar = s_u32(&full_bar[s]);
        const uint32_t base = s_u32(smem + (size_t)s * stage_bytes);
        bar_expect(bar, 2u * bytes + (bits_here ? bits_stage_bytes : 0u));
        bulk_load(base, p.in0 + row0 * p.C, bytes, bar);
        bulk_load(base + BS_TILE_BYTES, p.in1 + row0 * p.C, bytes, bar);
        if (bits_here) bulk_load(base + 2u * BS_TILE_BYTES, p.bits_in + row0 * p.cvecs, bits_stage_bytes, bar);
      }
    }
    return;
  }

  // ---- consumers
  const int cv = tid & (p.cvecs - 1), rl = tid >> p.cv_log2;
  const int c0 = cv * 8;
  float a[8], b[8], cc[8], sa[8], sb[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    a[k] = p.p0[c0 + k];
    b[k] = (MODE == 1) ? 0.f : p.p1[c0 + k];
    cc[k] = (MODE == 2) ? p.p2[c0 + k] : 0.f;
    sa[k] = 0.f;
    sb[k] = 0.f;
  }
  int it = 0;
  for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it) {
    const int s = it % BS_STAGES;
    if (!bar_wait(s_u32(&full_bar[s]), (it / BS_STAGES) & 1, &abort_flag, 2)) break;
    const unsigned char* st = smem + (size_t)s * stage_bytes;
    const long long row0 = t * p.tile_rows;
    const int rows = (int)min((long long)p.tile_rows, p.M - row0);
    const bool bits_here = stage_bits && rows == p.tile_rows;
    for (int r = rl; r < rows; r += p.rows_per_pass) {
      const int v = r * p.cvecs + cv;
      const uint4 q0 = *reinterpret_cast<const uint4*>(st + (size_t)v * 16);
      const uint4 q1 = *reinterpret_cast<const uint4*>(st + BS_TILE_BYTES + (size_t)v * 16);
      const long long gv = row0 * p.cvecs + v;  // index of this vector in the whole tensor
      float v0[8], v1[8];
      bs_unpack8(q0, v0);
      bs_unpack8(q1, v1);
      if (MODE == 0) {
        unsigned m = 0;
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float y = v0[k] * a[k] + b[k] + v1[k];
          m |= (y > 0.f ? 1u : 0u) << k;
          o[k] = p.relu ? fmaxf(y, 0.f) : y;
        }
        *reinterpret_cast<uint4*>(p.out0 + gv * 8) = bs_pack8(o);
        if (p.bits_out != nullptr) p.bits_out[gv] = (unsigned char)m;
      } else {
        unsigned m = 0xffu;
        if (bits_here) m = st[2u * BS_TILE_BYTES + v];
        else if (p.bits_in != nullptr) m = p.bits_in[gv];
        if (MODE == 1) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float d = ((m >> k) & 1u) ? v0[k] : 0.f;
            sa[k] += d;
            sb[k] = fmaf(d, v1[k] - a[k], sb[k]);
          }
        } else {
          float o[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float d = ((m >> k) & 1u) ? v0[k] : 0.f;
            v0[k] = d;
            o[k] = a[k] * d + b[k] * v1[k] + cc[k];
          }
          *reinterpret_cast<uint4*>(p.out0 + gv * 8) = bs_pack8(o);
          if (p.out1 != nullptr) {
            // the masked gradient keeps its bf16 bits: re-pack by truncation of values that are exact bf16 already
            uint4 qd = q0;
            qd.x &= ((m & 1u) ? 0x0000ffffu : 0u) | ((m & 2u) ? 0xffff0000u : 0u);
            qd.y &= ((m & 4u) ? 0x0000ffffu : 0u) | ((m & 8u) ? 0xffff0000u : 0u);
            qd.z &= ((m & 16u) ? 0x0000ffffu : 0u) | ((m & 32u) ? 0xffff0000u : 0u);
            qd.w &= ((m & 64u) ? 0x0000ffffu : 0u) | ((m & 128u) ? 0xffff0000u : 0u);
            *reinterpret_cast<uint4*>(p.out1 + gv * 8) = qd;
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) bar_arrive(s_u32(&empty_bar[s]));
  }
  if (MODE == 1) {
    // combine the row lanes of this block (threads with equal cv) through shared memory, then one atomic per channel
    asm volatile("bar.sync 1, %0;" ::"n"(BS_CONSUMERS) : "memory");  // every consumer is done with the stages
    float* red = reinterpret_cast<float*>(smem);                    // [16][BS_CONSUMERS]
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      red[k * BS_CONSUMERS + tid] = sa[k];
      red[(8 + k) * BS_CONSUMERS + tid] = sb[k];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(BS_CONSUMERS) : "memory");
    // 16 * cvecs sums, each over rows_per_pass threads: thread j handles (quantity q, vector v) pairs
    for (int j = tid; j < 16 * p.cvecs; j += BS_CONSUMERS) {
      const int q = j >> p.cv_log2, v = j & (p.cvecs - 1);
      float acc = 0.f;
      for (int r = 0; r < p.rows_per_pass; ++r) acc += red[q * BS_CONSUMERS + r * p.cvecs + v];
      const int c = v * 8 + (q & 7);
      if (q < 8) atomicAdd(p.sums + c, acc);
      else atomicAdd(p.sums + p.C + c, acc * p.p1[c]);
    }
  }
}

bool bs_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("KERAS_B200_BN_STREAM");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

int bs_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    sms[dev] = v;
  }
  return sms[dev];
}

template <int MODE>
int bs_set_attr(size_t smem) {
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -1;
  if (!done[dev]) {
    if (cudaFuncSetAttribute(bn_stream_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    done[dev] = true;
  }
  return 0;
}

}  // namespace

// Returns 1 when the streaming kernel does not apply (the caller then uses the register kernels), 0 when it was
// launched, a negative code on a launch error.  mode as bn_stream_kernel.  bf16 only.
int kb200_bn_stream_launch(int mode, const void* in0, const void* in1, const unsigned char* bits_in, void* out0, void* out1, unsigned char* bits_out,
                           const float* p0, const float* p1, const float* p2, float* sums, long long M, int C, int relu, cudaStream_t stream) {
  if (!bs_enabled() || in0 == nullptr || in1 == nullptr || C % 8 != 0) return 1;
  const int cvecs = C / 8;
  if (cvecs < 1 || cvecs > BS_CONSUMERS || (cvecs & (cvecs - 1)) != 0) return 1;
  if (M * (long long)C < (1ll << 21)) return 1;  // small tensors: the register kernels have less set-up
  const uintptr_t align = (uintptr_t)in0 | (uintptr_t)in1 | (uintptr_t)out0 | (uintptr_t)out1 | (uintptr_t)bits_in;
  if (align & 15) return 1;
  BsParams p;
  p.in0 = (const __nv_bfloat16*)in0;
  p.in1 = (const __nv_bfloat16*)in1;
  p.bits_in = bits_in;
  p.out0 = (__nv_bfloat16*)out0;
  p.out1 = (__nv_bfloat16*)out1;
  p.bits_out = bits_out;
  p.p0 = p0;
  p.p1 = p1;
  p.p2 = p2;
  p.sums = sums;
  p.M = M;
  p.C = C;
  p.cvecs = cvecs;
  p.cv_log2 = 0;
  while ((1 << p.cv_log2) < cvecs) ++p.cv_log2;
  p.rows_per_pass = BS_CONSUMERS / cvecs;
  int passes = BS_TILE_BYTES / (C * 2) / p.rows_per_pass;
  if (passes < 1) return 1;
  p.tile_rows = passes * p.rows_per_pass;
  p.tiles = (M + p.tile_rows - 1) / p.tile_rows;
  p.relu = relu;
  const size_t bits_stage = (mode != 0 && bits_in != nullptr) ? (size_t)p.tile_rows * cvecs : 0;
  const size_t smem = (size_t)BS_STAGES * (2 * BS_TILE_BYTES + bits_stage);
  long long grid = bs_sm_count();
  if (grid > p.tiles) grid = p.tiles;
  if (mode == 1 && grid > p.tiles / 4) grid = p.tiles / 4 > 0 ? p.tiles / 4 : 1;  // fewer blocks, fewer atomics per channel
  int rc = 0;
  if (mode == 0) {
    rc = bs_set_attr<0>(smem);
    if (rc == 0) bn_stream_kernel<0><<<(int)grid, BS_THREADS, smem, stream>>>(p);
  } else if (mode == 1) {
    rc = bs_set_attr<1>(smem);
    if (rc == 0) bn_stream_kernel<1><<<(int)grid, BS_THREADS, smem, stream>>>(p);
  } else {
    rc = bs_set_attr<2>(smem);
    if (rc == 0) bn_stream_kernel<2><<<(int)grid, BS_THREADS, smem, stream>>>(p);
  }
  if (rc != 0) return 1;
  KB_CHECK_LAUNCH("bn_stream");
  return 0;
}

// 0 when no bounded wait of the streaming kernels ran out on the current device since the last call; else the code.
// Synchronises the device.
KB_API int kb200_bn_stream_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_bn_stream_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_bn_stream_status, &zero, sizeof(int));
  }
  return v;
}
