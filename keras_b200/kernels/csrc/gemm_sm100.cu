// bf16 GEMM on 5th-generation tensor cores (tcgen05), Blackwell sm_100a.
//
//   C[M,N] = act(A x B + bias)        fp32 accumulation in tensor memory (TMEM)
//
// Operands are fed by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a 3-stage shared-memory
// ring; one elected thread issues tcgen05.mma (128x128x16 per instruction, cta_group::1) with the
// accumulator in TMEM; four epilogue warps read the accumulator back with tcgen05.ld and apply
// bias / activation / output cast on the way to global memory.  Both operands may be K-major or
// MN-major (set in the UMMA instruction and shared-memory descriptors), which covers the forward
// (X·W), input-gradient (dY·Wᵀ) and weight-gradient (Xᵀ·dY) products of a dense layer without any
// transposed copy.  Two CTAs fit per SM (96 KB of operand stages, 128 TMEM columns each) so one
// CTA's epilogue overlaps the other's main loop.
//
// Replaces torch.matmul / cuBLASLt + separate bias and activation kernels
// (keras/src/backend/torch/numpy.py:101-160, keras/src/layers/core/dense.py:238-244).
//
// Every wait on an mbarrier is bounded: on expiry the kernel records a code in `*err`, drains its
// outstanding copies (also bounded), releases TMEM and returns.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"

namespace {

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
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
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
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[h * 32 + j]);
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
      if (p.split_k > 1) {
        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c),
                     "r"(stage + (stores & 1u) * 4096u), "r"(col0), "r"(row0) : "memory");
      } else {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c),
                     "r"(stage + (stores & 1u) * 4096u), "r"(col0), "r"(row0) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    ++stores;
  }
}

__global__ void __launch_bounds__(THREADS, 2)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + STAGES * STAGE_BYTES);
  const uint32_t bar_base = base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t tmem_full_bar = bar_base + 8u * (2 * STAGES);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int m0 = (blockIdx.x / n_tiles) * BM;
  const int n0 = (blockIdx.x % n_tiles) * BN;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int issued = 0;
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t parity = ((kb / STAGES) & 1) ^ 1;
        ok = mbar_wait(empty_bar(s), parity, abort_flag);
        if (!ok) break;
        const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_TILE_BYTES;
        mbar_expect_tx(full_bar(s), STAGE_BYTES);
        const int k0 = kb * BK;
        if (p.a_mn_major) {
          tma_load_2d(sa, &map_a, full_bar(s), m0, k0);
          tma_load_2d(sa + 8192, &map_a, full_bar(s), m0 + 64, k0);
        } else {
          tma_load_2d(sa, &map_a, full_bar(s), k0, m0);
        }
        if (p.b_mn_major) {
          tma_load_2d(sb, &map_b, full_bar(s), n0, k0);
          tma_load_2d(sb + 8192, &map_b, full_bar(s), n0 + 64, k0);
        } else {
          tma_load_2d(sb, &map_b, full_bar(s), k0, n0);
        }
        issued = kb + 1;
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 1);
        *abort_flag = 1;
        // drain: give copies already issued a bounded time to land before the CTA exits
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int kb = first; kb < issued; ++kb) {
          const int s = kb % STAGES;
          for (uint32_t it = 0; it < (1u << 16); ++it)
            if (mbar_try_wait(full_bar(s), (kb / STAGES) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t a_step = p.a_mn_major ? (2048u >> 4) : (32u >> 4);
      const uint32_t b_step = p.b_mn_major ? (2048u >> 4) : (32u >> 4);
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(full_bar(s), (kb / STAGES) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_TILE_BYTES;
        const uint64_t adesc = make_smem_desc(sa, p.a_mn_major), bdesc = make_smem_desc(sb, p.b_mn_major);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          umma_bf16(tmem_base, adesc + (uint64_t)(a_step * k), bdesc + (uint64_t)(b_step * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));  // frees the stage when these MMAs have read it
      }
      if (ok) {
        umma_commit(tmem_full_bar);
      } else {
        if (p.err) atomicExch(p.err, 2);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const bool ok = mbar_wait(tmem_full_bar, 0, abort_flag);
    if (!ok) {
      if (lane == 0 && p.err) atomicExch(p.err, 3);
      *abort_flag = 1;
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int q = warp & 3;  // TMEM lane quarter this warp may access
      // every MMA of this CTA's only tile has completed, so the operand ring is free: stage 0 holds the staging buffers
      uint32_t stores = 0;
      store_rows_tma(tmem_base + ((uint32_t)(q * 32) << 16), BN, n0, m0 + q * 32, base + (uint32_t)(warp - 2) * 8192u, stores, &map_c, p, lane);
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}


// ---------------------------------------------------------------------------------------------
// Persistent variant for large problems: 128x256 output tiles, four 48 KB operand stages, the whole
// tensor memory (512 columns) split into two 256-column accumulators so that the epilogue of tile i
// overlaps the main loop of tile i+1.  One CTA per SM; tiles are handed out round-robin in an order
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

__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_tcgen05_persistent(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                             const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  constexpr int BM = v2::BM, BN = v2::BN, BK = v2::BK, STAGES = v2::STAGES, STAGE_BYTES = v2::STAGE_BYTES, A_BYTES = v2::A_BYTES;
  constexpr uint32_t TMEM_COLS = v2::TMEM_COLS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  // after the operand ring: 4 epilogue warps x 2 staging buffers of 4 KB (32 rows x 128 B, swizzled), then the barriers
  const uint32_t stage_out = base + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + STAGES * STAGE_BYTES + v2::OUT_BYTES);
  const uint32_t bar_base = stage_out + v2::OUT_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int split = p.split_k > 1 ? p.split_k : 1;
  const int total_tiles = m_tiles * n_tiles * split;  // work units: (output tile, K slice)
  const int k_blocks_all = (p.K + BK - 1) / BK;
  const int kb_per = split > 1 ? p.kb_per_split : k_blocks_all;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      uint32_t issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int m0, n0;
        tile_coords(t / split, m_tiles, n_tiles, m0, n0);
        const int kb0 = (t % split) * kb_per, kb1 = min(kb0 + kb_per, k_blocks_all);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const int k0 = kb * BK;
          if (p.a_mn_major) {
            tma_load_2d(sa, &map_a, full_bar(s), m0, k0);
            tma_load_2d(sa + 8192, &map_a, full_bar(s), m0 + 64, k0);
          } else {
            tma_load_2d(sa, &map_a, full_bar(s), k0, m0);
          }
          if (p.b_mn_major) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &map_b, full_bar(s), n0 + j * 64, k0);
          } else {
            tma_load_2d(sb, &map_b, full_bar(s), k0, n0);
          }
          issued = it + 1;
        }
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 11);
        *abort_flag = 1;
        const uint32_t first = issued > STAGES ? issued - STAGES : 0;
        for (uint32_t i = first; i < issued; ++i) {
          for (uint32_t spin = 0; spin < (1u << 16); ++spin)
            if (mbar_try_wait(full_bar(i % STAGES), (i / STAGES) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t a_step = p.a_mn_major ? (2048u >> 4) : (32u >> 4);
      const uint32_t b_step = p.b_mn_major ? (2048u >> 4) : (32u >> 4);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
        const uint32_t acc = local & 1;
        ok = mbar_wait(acc_empty_bar(acc), ((local >> 1) & 1) ^ 1, abort_flag);  // epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * (uint32_t)BN;
        const int kb0 = (t % split) * kb_per, kb1 = min(kb0 + kb_per, k_blocks_all);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full_bar(s), (it / STAGES) & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t adesc = make_smem_desc(sa, p.a_mn_major), bdesc = make_smem_desc(sb, p.b_mn_major);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_d, adesc + (uint64_t)(a_step * k), bdesc + (uint64_t)(b_step * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(empty_bar(s));
        }
        if (ok) umma_commit(acc_full_bar(acc));
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 12);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const uint32_t my_stage = stage_out + (uint32_t)(warp - 2) * 8192u;
    uint32_t local = 0, stores = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
      int m0, n0;
      tile_coords(t / split, m_tiles, n_tiles, m0, n0);
      const uint32_t acc = local & 1;
      ok = mbar_wait(acc_full_bar(acc), (local >> 1) & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_row = tmem_base + acc * (uint32_t)BN + ((uint32_t)(q * 32) << 16);
      store_rows_tma(tmem_row, BN, n0, m0 + q * 32, my_stage, stores, &map_c, p, lane);
      // this warp has finished reading the accumulator: hand it back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (!ok) {
      if (lane == 0 && p.err) atomicExch(p.err, 13);
      *abort_flag = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(v2::TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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
bool make_map(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long pitch_elems, int box_inner, int box_outer,
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

}  // namespace

// C[M,N] = act(op(A) op(B) + bias).
//   a_mn_major = 0: A stored [M, K] row-major (pitch lda);  1: A stored [K, M] row-major (pitch lda)
//   b_mn_major = 0: B stored [N, K] row-major (pitch ldb);  1: B stored [K, N] row-major (pitch ldb)
// Requirements: bf16 operands, 16-byte aligned base pointers, pitches multiples of 8 elements;
// C bf16 (out_fp32 = 0) or fp32, ldc multiple of 8 (bf16) / 4 (fp32).  `err` is an int in device
// memory that receives a non-zero code if a bounded wait expires (0 otherwise untouched).
//
// split_k > 1 (persistent kernel only): the K range is cut into `split_k` slices that run as separate work units and
// add their fp32 partial tiles into C with TMA reduce stores; C must be fp32 and zero on entry, bias/act must be off.
KB_API int kb200_gemm_bf16_splitk(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn_major, int b_mn_major, int act, int out_fp32, int split_k, int* err,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (split_k > 1 && (!out_fp32 || bias != nullptr || act != ACT_NONE)) {
    kb200_set_error("gemm_bf16: split-K needs an fp32 output without bias or activation");
    return -4;
  }
  if ((lda % 8) || (ldb % 8) || (((uintptr_t)a | (uintptr_t)b) & 15) || (((uintptr_t)c) & 15) || (ldc % (out_fp32 ? 4 : 8))) {
    kb200_set_error("gemm_bf16: operands must be 16-byte aligned with pitches that are multiples of 8 elements");
    return -2;
  }
  CUtensorMap map_a, map_b, map_c;
  static int force_v1 = -1, sm_count = 0;
  if (force_v1 < 0) {
    const char* e = getenv("KB200_GEMM_V1");
    force_v1 = (e != nullptr && e[0] == '1') ? 1 : 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
  }
  const long long tiles_v2 = (long long)((M + v2::BM - 1) / v2::BM) * ((N + v2::BN - 1) / v2::BN);
  int kb_per_split = 0;
  if (split_k > 1) {
    const int k_blocks = (K + v2::BK - 1) / v2::BK;
    if (split_k > k_blocks) split_k = k_blocks;
    kb_per_split = (k_blocks + split_k - 1) / split_k;
    split_k = (k_blocks + kb_per_split - 1) / kb_per_split;  // every slice holds at least one K block
  }
  if (split_k < 1) split_k = 1;
  const bool use_v2 = split_k > 1 || (!force_v1 && N > 128 && tiles_v2 >= sm_count / 2);
  const int bn = use_v2 ? v2::BN : BN;
  bool ok = a_mn_major ? make_map(&map_a, a, M, K, lda, 64, BK) : make_map(&map_a, a, K, M, lda, BK, BM);
  ok = ok && (b_mn_major ? make_map(&map_b, b, N, K, ldb, 64, BK) : make_map(&map_b, b, K, N, ldb, BK, bn));
  ok = ok && make_map(&map_c, c, N, M, ldc, out_fp32 ? 32 : 64, 32, out_fp32 != 0);
  if (!ok) {
    kb200_set_error("gemm_bf16: cuTensorMapEncodeTiled failed");
    return -3;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_tcgen05_persistent, cudaFuncAttributeMaxDynamicSharedMemorySize, v2::SMEM_BYTES);
    attr_set = true;
  }
  GemmParams p{c, bias, M, N, K, ldc, a_mn_major, b_mn_major, act, out_fp32, err, split_k, kb_per_split};
  if (use_v2) {
    const long long units = tiles_v2 * split_k;
    const unsigned grid = (unsigned)(units < sm_count ? units : sm_count);
    gemm_bf16_tcgen05_persistent<<<grid, THREADS, v2::SMEM_BYTES, stream>>>(map_a, map_b, map_c, p);
  } else {
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    gemm_bf16_tcgen05_kernel<<<(unsigned)tiles, THREADS, SMEM_BYTES, stream>>>(map_a, map_b, map_c, p);
  }
  KB_CHECK_LAUNCH("gemm_bf16");
  return 0;
}

KB_API int kb200_gemm_bf16(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, int a_mn_major, int b_mn_major, int act, int out_fp32, int* err, cudaStream_t stream) {
  return kb200_gemm_bf16_splitk(a, b, c, bias, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, act, out_fp32, 1, err, stream);
}
