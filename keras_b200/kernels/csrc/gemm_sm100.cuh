// Device and host helpers shared by the tcgen05 GEMM kernels (plain, persistent, and fused with collectives):
// mbarrier / TMA / tcgen05 wrappers, shared-memory and instruction descriptors, the TMA-store epilogue,
// tile constants and the tensor-map encoder.  Everything is `static`/inline: each including .cu file gets its own copy.
#pragma once
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"

namespace kbgemm {


constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 3;
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_TILE_BYTES = BN * BK * 2;  // 16 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 192;  // warp0 TMA, warp1 MMA, warps 2-5 epilogue
constexpr uint32_t TMEM_COLS = 128;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_GELU_ERF = 4 };

struct GemmParams {
  void* c;
  const float* bias;
  int M, N, K;
  long long ldc;
  int a_mn_major, b_mn_major;
  int act, out_fp32;
  int* err;
  int split_k;        // >1: each work unit covers `kb_per_split` K blocks and adds its fp32 partial tile into C (zeroed by the caller)
  int kb_per_split;
  int fp8 = 0;        // 0: bf16 operands; else 1 + a_format + 2 * b_format with format 0 = e4m3, 1 = e5m2 (both operands K-major)
  const float* alpha = nullptr;  // device scalar multiplied into the accumulator before bias and activation (fp8 de-scaling)
  int int8 = 0;                      // 1: signed 8-bit operands (kind::i8), int32 accumulators
  const float* row_scale = nullptr;  // [M] and [N] factors applied to the accumulator (int8 de-quantisation)
  const float* col_scale = nullptr;
  int accumulate = 0;                // 1: add the fp32 tile into C (TMA reduce store) instead of overwriting it
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bounded wait. Returns false when the limit expires or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, %1;\n\t"
      "@px mov.s32 %0, 1;\n\t}"
      : "+r"(pred)
      : "r"(0xFFFFFFFFu));
  return pred != 0;
}

// Shared-memory matrix descriptor for tcgen05.mma (128-byte swizzle).
//   K-major : rows of 128 B (64 bf16 along K); 8-row groups 1024 B apart (SBO); LBO unused (=1)
//   MN-major: rows of 128 B (64 bf16 along M/N), one row per K index; 8-row K groups 1024 B apart
//             (SBO); the next 64 M/N elements live 8192 B further (LBO)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, bool mn_major) {
  const uint64_t lbo = mn_major ? (8192u >> 4) : 1u;
  const uint64_t sbo = 1024u >> 4;
  uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= lbo << 16;
  d |= sbo << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case ACT_RELU: return fmaxf(v, 0.f);
    case ACT_GELU_TANH: {
      const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      return 0.5f * v * (1.f + tanhf(u));
    }
    case ACT_SILU: return v / (1.f + __expf(-v));
    case ACT_GELU_ERF: return 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
    default: return v;
  }
}

// Epilogue of one 32-row slice of an accumulator tile (rows `row0`.., `ncols` columns from TMEM address `tmem_row`).
// The warp converts 128 bytes of each row at a time (64 bf16 or 32 fp32 columns), writes them into a swizzled
// 32 x 128 B staging buffer (`stage`: two such buffers, 1024-byte aligned) and lets the TMA engine store that box, so
// global memory sees full 128-byte lines and rows/columns beyond M/N are clipped by the tensor map.  `stores` counts
// the boxes this warp has issued (selects the staging buffer).  Lane 0 must run `cp.async.bulk.wait_group 0` before
// the CTA exits.
__device__ __forceinline__ void store_rows_tma(uint32_t tmem_row, int ncols, int n0, int row0, uint32_t stage, uint32_t& stores,
                                               const CUtensorMap* map_c, const GemmParams& p, int lane) {
  const int cols_per_chunk = p.out_fp32 ? 32 : 64;
  const int chunks = ncols / cols_per_chunk;
  const uint32_t sw = (uint32_t)(lane & 7);
  float alpha = p.alpha != nullptr ? __ldg(p.alpha) : 1.f;
  if (p.row_scale != nullptr) alpha *= __ldg(p.row_scale + min(row0 + lane, p.M - 1));
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    const int col0 = n0 + c * cols_per_chunk;
    if (col0 >= p.N) break;
    uint32_t r[64];
    tmem_ld32(tmem_row + (uint32_t)(c * cols_per_chunk), r);
    if (!p.out_fp32) tmem_ld32(tmem_row + (uint32_t)(c * cols_per_chunk + 32), r + 32);
    // the staging buffer used two stores ago must have been read out by the TMA engine
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    __syncwarp();
    const uint32_t buf = stage + (stores & 1u) * 4096u + (uint32_t)lane * 128u;
    if (p.out_fp32) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (p.int8 ? __int2float_rn((int)r[j]) : __uint_as_float(r[j])) * alpha;
      if (p.col_scale != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= __ldg(p.col_scale + min(col0 + j, p.N - 1));
      }
      if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += __ldg(p.bias + min(col0 + j, p.N - 1));
      }
      if (p.act != ACT_NONE) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(buf + (((uint32_t)u ^ sw) << 4)), "f"(v[u * 4]), "f"(v[u * 4 + 1]),
                     "f"(v[u * 4 + 2]), "f"(v[u * 4 + 3]) : "memory");
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (p.int8 ? __int2float_rn((int)r[h * 32 + j]) : __uint_as_float(r[h * 32 + j])) * alpha;
        if (p.col_scale != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= __ldg(p.col_scale + min(col0 + h * 32 + j, p.N - 1));
        }
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += __ldg(p.bias + min(col0 + h * 32 + j, p.N - 1));
        }
        if (p.act != ACT_NONE) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const bf16x8 pk = pack8(v + u * 8);
          const uint4 w = *reinterpret_cast<const uint4*>(&pk);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + (((uint32_t)(h * 4 + u) ^ sw) << 4)), "r"(w.x), "r"(w.y),
                       "r"(w.z), "r"(w.w) : "memory");
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0 && row0 < p.M) {
      if (p.split_k > 1 || p.accumulate) {
        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c),
                     "r"(stage + (stores & 1u) * 4096u), "r"(col0), "r"(row0) : "memory");
      } else {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c),
                     "r"(stage + (stores & 1u) * 4096u), "r"(col0), "r"(row0) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    // the staging buffers alternate per committed store group: `wait_group.read 1` above only protects the buffer of
    // the group before last, so a chunk that issued no store must not advance the buffer index
    if (row0 < p.M) ++stores;
  }
}


// that keeps the CTAs running at the same time on neighbouring tiles (8 row-tiles per group) for L2 reuse.
namespace v2 {
constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OUT_BYTES = 4 * 2 * 4096;  // per epilogue warp: two 32-row x 128-byte staging buffers for TMA stores
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES + 1024 + 256;
constexpr uint32_t TMEM_COLS = 512;
constexpr int GROUP_M = 8;
}  // namespace v2

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& m0, int& n0) {
  const int per_group = v2::GROUP_M * n_tiles;
  const int g = t / per_group;
  const int first_m = g * v2::GROUP_M;
  const int rows = min(v2::GROUP_M, m_tiles - first_m);
  const int r = t - g * per_group;
  m0 = (first_m + r % rows) * v2::BM;
  n0 = (r / rows) * v2::BN;
}



typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch `pitch_elems`.
static inline bool make_map(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long pitch_elems, int box_inner, int box_outer,
              bool fp32 = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * (fp32 ? 4 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}


// 2-D byte tensor map (fp8 operands): `inner` contiguous bytes per row, `outer` rows, row pitch `pitch_bytes`.
static inline bool make_map_u8(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long pitch_bytes, int box_inner, int box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace kbgemm
