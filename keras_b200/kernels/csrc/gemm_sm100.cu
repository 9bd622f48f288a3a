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
#include "gemm_sm100.cuh"

namespace {
using namespace kbgemm;

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
  const int bk = (p.fp8 || p.int8) ? 2 * BK : BK;  // elements per 128-byte K block
  const int k_blocks_all = (p.K + bk - 1) / bk;
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
          const int k0 = kb * bk;
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
      // instruction descriptor: fp32 accumulate; operand formats bf16 (kind::f16: 1) or e4m3 / e5m2 (kind::f8f6f4: 0 / 1)
      const uint32_t a_fmt = p.fp8 ? (uint32_t)((p.fp8 - 1) & 1) : 1u, b_fmt = p.fp8 ? (uint32_t)(((p.fp8 - 1) >> 1) & 1) : 1u;
      // kind::i8: accumulator format 2 (s32), operand format 1 (signed 8-bit)
      const uint32_t idesc = p.int8 ? ((2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24))
                                    : ((1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24));
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
          if (p.int8) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_i8(tmem_d, adesc + (uint64_t)(a_step * k), bdesc + (uint64_t)(b_step * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          } else if (p.fp8) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)  // 32 one-byte elements per instruction: the same 32-byte descriptor step
              umma_f8(tmem_d, adesc + (uint64_t)(a_step * k), bdesc + (uint64_t)(b_step * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_bf16(tmem_d, adesc + (uint64_t)(a_step * k), bdesc + (uint64_t)(b_step * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
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
// split_k < 0: |split_k| slices and the product is ADDED to what C holds (fp32 gradient accumulation in place).
KB_API int kb200_gemm_bf16_splitk(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn_major, int b_mn_major, int act, int out_fp32, int split_k, int* err,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int accumulate = split_k < 0 ? 1 : 0;
  if (split_k < 0) split_k = -split_k;
  if ((split_k > 1 || accumulate) && (!out_fp32 || bias != nullptr || act != ACT_NONE)) {
    kb200_set_error("gemm_bf16: split-K needs an fp32 output without bias or activation");
    return -4;
  }
  if ((lda % 8) || (ldb % 8) || (((uintptr_t)a | (uintptr_t)b) & 15) || (((uintptr_t)c) & 15) || (ldc % (out_fp32 ? 4 : 8))) {
    kb200_set_error("gemm_bf16: operands must be 16-byte aligned with pitches that are multiples of 8 elements");
    return -2;
  }
  CUtensorMap map_a, map_b, map_c;
  static int force_v1 = -1;
  if (force_v1 < 0) {
    const char* e = getenv("KB200_GEMM_V1");
    force_v1 = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  const int sm_count = kb_sm_count();
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
  static bool attr_v1[KB_MAX_DEVICES] = {false}, attr_v2[KB_MAX_DEVICES] = {false};
  if (!kb_allow_smem(gemm_bf16_tcgen05_kernel, SMEM_BYTES, attr_v1) || !kb_allow_smem(gemm_bf16_tcgen05_persistent, v2::SMEM_BYTES, attr_v2)) {
    kb200_set_error("gemm_bf16: cannot raise the shared-memory limit of the kernels on this device");
    return -3;
  }
  GemmParams p{c, bias, M, N, K, ldc, a_mn_major, b_mn_major, act, out_fp32, err, split_k, kb_per_split};
  p.accumulate = accumulate;
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

// C[M,N] = act(alpha * (A x B^T) + bias) with one-byte floating-point operands on kind::f8f6f4 tensor-core instructions.
//   A: [M, K] bytes, row pitch lda bytes;  B: [N, K] bytes, row pitch ldb bytes (both K-major)
//   a_format / b_format: 0 = e4m3, 1 = e5m2;  alpha: device scalar (product of the operands' scales) or null
// Pitches must be multiples of 16 bytes and base pointers 16-byte aligned.  Always runs the persistent kernel.
KB_API int kb200_gemm_fp8(const void* a, const void* b, void* c, const float* bias, const float* alpha, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, int a_format, int b_format, int act, int out_fp32, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16) || (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) || (ldc % (out_fp32 ? 4 : 8)) || (a_format & ~1) || (b_format & ~1)) {
    kb200_set_error("gemm_fp8: operands must be 16-byte aligned with pitches that are multiples of 16 bytes; formats 0 (e4m3) or 1 (e5m2)");
    return -2;
  }
  CUtensorMap map_a, map_b, map_c;
  bool ok = make_map_u8(&map_a, a, K, M, lda, 128, v2::BM) && make_map_u8(&map_b, b, K, N, ldb, 128, v2::BN);
  ok = ok && make_map(&map_c, c, N, M, ldc, out_fp32 ? 32 : 64, 32, out_fp32 != 0);
  if (!ok) {
    kb200_set_error("gemm_fp8: cuTensorMapEncodeTiled failed");
    return -3;
  }
  static bool attr_v2[KB_MAX_DEVICES] = {false};
  if (!kb_allow_smem(gemm_bf16_tcgen05_persistent, v2::SMEM_BYTES, attr_v2)) {
    kb200_set_error("gemm: cannot raise the shared-memory limit of the kernel on this device");
    return -3;
  }
  const int sm_count = kb_sm_count();
  GemmParams p{c, bias, M, N, K, ldc, 0, 0, act, out_fp32, err, 1, 0, 1 + a_format + 2 * b_format, alpha};
  const long long tiles = (long long)((M + v2::BM - 1) / v2::BM) * ((N + v2::BN - 1) / v2::BN);
  gemm_bf16_tcgen05_persistent<<<(unsigned)(tiles < sm_count ? tiles : sm_count), THREADS, v2::SMEM_BYTES, stream>>>(map_a, map_b, map_c, p);
  KB_CHECK_LAUNCH("gemm_fp8");
  return 0;
}

// C[M,N] = act((A x B^T) * row_scale[m] * col_scale[n] + bias) with signed 8-bit operands (kind::i8, int32 accumulation).
//   A: [M, K] int8, row pitch lda bytes;  B: [N, K] int8, row pitch ldb bytes (both K-major)
KB_API int kb200_gemm_i8(const void* a, const void* b, void* c, const float* bias, const float* row_scale, const float* col_scale, int M, int N, int K,
                         long long lda, long long ldb, long long ldc, int act, int out_fp32, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16) || (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) || (ldc % (out_fp32 ? 4 : 8))) {
    kb200_set_error("gemm_i8: operands must be 16-byte aligned with pitches that are multiples of 16 bytes");
    return -2;
  }
  CUtensorMap map_a, map_b, map_c;
  bool ok = make_map_u8(&map_a, a, K, M, lda, 128, v2::BM) && make_map_u8(&map_b, b, K, N, ldb, 128, v2::BN);
  ok = ok && make_map(&map_c, c, N, M, ldc, out_fp32 ? 32 : 64, 32, out_fp32 != 0);
  if (!ok) {
    kb200_set_error("gemm_i8: cuTensorMapEncodeTiled failed");
    return -3;
  }
  static bool attr_v2[KB_MAX_DEVICES] = {false};
  if (!kb_allow_smem(gemm_bf16_tcgen05_persistent, v2::SMEM_BYTES, attr_v2)) {
    kb200_set_error("gemm: cannot raise the shared-memory limit of the kernel on this device");
    return -3;
  }
  const int sm_count = kb_sm_count();
  GemmParams p{c, bias, M, N, K, ldc, 0, 0, act, out_fp32, err, 1, 0, 0, nullptr, 1, row_scale, col_scale};
  const long long tiles = (long long)((M + v2::BM - 1) / v2::BM) * ((N + v2::BN - 1) / v2::BN);
  gemm_bf16_tcgen05_persistent<<<(unsigned)(tiles < sm_count ? tiles : sm_count), THREADS, v2::SMEM_BYTES, stream>>>(map_a, map_b, map_c, p);
  KB_CHECK_LAUNCH("gemm_i8");
  return 0;
}
