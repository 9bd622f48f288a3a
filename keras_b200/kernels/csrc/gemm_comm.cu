// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (one process per GPU, CUDA-IPC mapped
// symmetric buffers).  Both kernels are the persistent tcgen05 GEMM of gemm_sm100.cu (128x256x64 tiles, TMA-fed
// operand ring, two TMEM accumulators, TMA-store epilogue) with the transfer done tile by tile inside the kernel:
//
//   all-gather -> GEMM   C[world*Ms, N] = gather(A_r[Ms, K]) x B.  Every rank keeps a gathered-A buffer
//     [world*Ms, K] in symmetric memory and has written its own slice.  A few CTAs do no math: one thread of each
//     streams the peers' slices through shared memory with bulk async copies (peer -> smem -> local, several 32 KB
//     pieces in flight) and publishes a flag per 128-row block.  The GEMM CTAs start on the local slice and wait for
//     a block's flag only when their TMA producer reaches it, so the transfer hides behind the math.
//
//   GEMM -> reduce-scatter   out_r[Ms, N] = sum_s (A_s x B_s)[rows of r].  Every rank computes the full
//     [world*Ms, N] partial product, cycling through the owners block by block.  The epilogue stores each bf16 tile with a TMA store
//     straight into the owner's staging slot for this rank; when its own tiles are done a CTA adds what it delivered
//     to each owner's arrival counter, then waits for the counters of its rank and sums the `world` staged partials into `out`.
//
// The reference has no counterpart: its torch backend runs sharded layers as unsharded ones and its JAX backend
// leaves the collectives to XLA (keras/src/backend/jax/distribution_lib.py:32-106).
//
// Synchronisation.  `epoch` increases by one per call; buffers and counters are double-buffered by its parity.  A
// rank announces the start of call e to every peer (release store of e) and nobody reads a peer's slice before that
// peer has announced e, i.e. after the peer's earlier stream work, which wrote the slice, is complete.  Reuse of a
// parity buffer two calls later is safe because finishing call e+1 requires every peer to have started it.  Every
// wait (flags, counters, mbarriers) is bounded by an iteration count and wall-clock time; when one runs out the
// kernel raises `*status`, releases TMEM and returns.  Every load from peer memory is a plain (single-CTA) bulk copy.
#include "gemm_sm100.cuh"

namespace {
using namespace kbgemm;

constexpr int MAX_RANKS = 8;
// signal pad (unsigned words)
constexpr int SIG_STARTED = 0;     // [8]  epoch announced by each rank
constexpr int SIG_COUNT = 16;      // [2][8] arrival counters per parity and source rank (reduce-scatter)
constexpr int SIG_TICKET = 40;     // CTAs of this rank that finished the reduction
constexpr int SIG_CHUNK = 64;      // [..] epoch at which a 128-row block of the gathered operand became complete
constexpr int SIG_WORDS = 64 + 8192;

constexpr int PIECE = 32768;       // bytes per bulk copy of the all-gather stream
constexpr int PIECES = 6;          // ring slots of a copy CTA (the 192 KB operand ring of a GEMM CTA)
constexpr int LOADS_AHEAD = 4;     // peer loads in flight; the other slots are being stored to local memory

struct CommParams {
  int mode;  // 1: all-gather -> GEMM, 2: GEMM -> reduce-scatter
  int rank, world;
  unsigned epoch;
  unsigned long long timeout_ns;
  unsigned* status;
  unsigned* sig[MAX_RANKS];
  const uint8_t* gather[MAX_RANKS];  // mode 1: this call's gathered-A buffer of every rank
  int copy_ctas;
  const __nv_bfloat16* stage;  // mode 2: local staging [world][Ms][N]
  __nv_bfloat16* out;          // mode 2: local result [Ms, N]
  int rows_per_rank;           // Ms (multiple of 128)
};

struct CMaps {
  CUtensorMap m[MAX_RANKS];
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// mbarrier wait whose own limit lies far beyond the peer time-out: it ends through the CTA's abort flag
__device__ __forceinline__ bool mbar_wait_long(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (unsigned long long it = 0; it < (1ull << 34); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023ull) == 1023ull && *abort_flag) return false;
  }
  return false;
}

// One thread waits until *flag has reached `target` (wrap-safe).  False when the wait ran out or another waiter gave up.
template <bool SYS>
__device__ bool wait_reach(const unsigned* flag, unsigned target, const CommParams& c, unsigned code) {
  const unsigned long long t0 = global_ns();
  for (unsigned it = 0;; ++it) {
    const unsigned v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if ((int)(v - target) >= 0) return true;
    if ((it & 63u) == 63u) {
      if (*(volatile unsigned*)c.status != 0u) return false;
      if (it > (1u << 26) || global_ns() - t0 > c.timeout_ns) {
        atomicCAS(c.status, 0u, code);
        return false;
      }
    }
    __nanosleep(100);
  }
}

// Physical 128-row block of logical block `lm`.  Mode 1 starts on the local slice and then walks the peers' slices in
// ring order (the order in which the copy CTAs bring them in).  Mode 2 cycles through the owners block by block
// (rank+1, rank+2, ..., rank), which spreads the remote stores evenly over the whole run of the kernel.
__device__ __forceinline__ int rotate_block(int lm, int m_tiles, int tpr, const CommParams& c) {
  if (c.mode == 1) {
    int pm = lm + c.rank * tpr;
    if (pm >= m_tiles) pm -= m_tiles;
    return pm;
  }
  int owner = c.rank + 1 + lm % c.world;
  if (owner >= c.world) owner -= c.world;
  return owner * tpr + lm / c.world;
}

__device__ __forceinline__ void tile_coords_rot(int t, int m_tiles, int n_tiles, int tpr, const CommParams& c, int& m0, int& n0) {
  tile_coords(t, m_tiles, n_tiles, m0, n0);
  m0 = rotate_block(m0 / v2::BM, m_tiles, tpr, c) * v2::BM;
}

// ---------------------------------------------------------------------------------------------
// Copy CTA of the all-gather: one thread moves the peers' slices into the local gathered buffer.
__device__ void gather_stream(uint32_t ring, uint32_t bar_base, const CommParams& c, int m_tiles, int tpr, long long block_bytes) {
  if (threadIdx.x != 0) return;
  // peers must have announced this call before their slices are read
  for (int s = 0; s < c.world; ++s)
    if (s != c.rank && !wait_reach<true>(c.sig[c.rank] + SIG_STARTED + s, c.epoch, c, 0x100u + s)) return;
  for (int i = 0; i < PIECES; ++i) mbar_init(bar_base + 8u * i, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  uint32_t issued = 0, stored = 0;  // pieces loaded / stored so far (ring position = count % PIECES)
  const int remote_blocks = (c.world - 1) * tpr;
  bool ok = true;
  for (int j = blockIdx.x; j < remote_blocks && ok; j += c.copy_ctas) {
    const int pm = rotate_block(tpr + j, m_tiles, tpr, c);
    const int src = pm / tpr;
    const uint8_t* from = c.gather[src] + (long long)pm * block_bytes;
    uint8_t* to = const_cast<uint8_t*>(c.gather[c.rank]) + (long long)pm * block_bytes;
    const int n_pieces = (int)((block_bytes + PIECE - 1) / PIECE);
    int loaded = 0, done = 0;
    while (done < n_pieces && ok) {
      // keep the ring full
      while (loaded < n_pieces && issued - stored < (uint32_t)LOADS_AHEAD) {
        const uint32_t slot = issued % PIECES;
        // The store that last used this slot is store number issued-6; at least stored >= issued-4 stores exist, so it is
        // never the most recent one: letting only the most recent store still read is enough.
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        const long long off = (long long)loaded * PIECE;
        const uint32_t bytes = (uint32_t)min((long long)PIECE, block_bytes - off);
        mbar_expect_tx(bar_base + 8u * slot, bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ring + slot * PIECE),
                     "l"(from + off), "r"(bytes), "r"(bar_base + 8u * slot) : "memory");
        ++issued;
        ++loaded;
      }
      // oldest piece: wait for it, then store it to the local buffer
      const uint32_t slot = stored % PIECES;
      const unsigned long long t0 = global_ns();
      for (unsigned it = 0;; ++it) {
        if (mbar_try_wait(bar_base + 8u * slot, (stored / PIECES) & 1)) break;
        if ((it & 1023u) == 1023u && (global_ns() - t0 > c.timeout_ns || *(volatile unsigned*)c.status != 0u)) {
          atomicCAS(c.status, 0u, 0x200u + src);
          ok = false;
          break;
        }
      }
      if (!ok) break;
      const long long off = (long long)done * PIECE;
      const uint32_t bytes = (uint32_t)min((long long)PIECE, block_bytes - off);
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(to + off), "r"(ring + slot * PIECE), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      ++stored;
      ++done;
    }
    if (!ok) break;
    // the whole block is in local memory: publish it to the TMA producers of the GEMM CTAs
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence();
    st_release_gpu(c.sig[c.rank] + SIG_CHUNK + pm, c.epoch);
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (!ok) {
    // loads already issued into the ring get a bounded time to land before the CTA exits
    for (uint32_t i = stored; i < issued; ++i)
      for (uint32_t spin = 0; spin < (1u << 18); ++spin)
        if (mbar_try_wait(bar_base + 8u * (i % PIECES), (i / PIECES) & 1)) break;
  }
}

// out[i] = sum over ranks s < world of stage[s][i] for the vectors first, first + step, ...; U vectors of up to R ranks are
// requested before any is used.
template <int U, int R>
__device__ __forceinline__ void reduce_staged(const uint4* __restrict__ st, uint4* __restrict__ out, long long vecs, long long first, long long step,
                                              int world) {
  for (long long i0 = first; i0 < vecs; i0 += step * U) {
    uint4 raw[U][R];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * step;
#pragma unroll
      for (int s = 0; s < R; ++s)
        if (s < world && i < vecs) raw[u][s] = __ldcg(st + (long long)s * vecs + i);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * step;
      if (i >= vecs) break;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int s = 0; s < R; ++s) {
        if (s < world) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u][s]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
      }
      const bf16x8 pk = pack8(acc);
      out[i] = *reinterpret_cast<const uint4*>(&pk);
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_tcgen05_comm(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CMaps maps_c,
                       const GemmParams p, const CommParams c) {
  constexpr int BM = v2::BM, BN = v2::BN, BK = v2::BK, STAGES = v2::STAGES, STAGE_BYTES = v2::STAGE_BYTES, A_BYTES = v2::A_BYTES;
  constexpr uint32_t TMEM_COLS = v2::TMEM_COLS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t stage_out = base + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + STAGES * STAGE_BYTES + v2::OUT_BYTES);
  const uint32_t bar_base = stage_out + v2::OUT_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 5);
  volatile int* phase_ok = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int tpr = c.rows_per_rank / BM;  // 128-row blocks per rank
  const unsigned parity = c.epoch & 1u;

  // announce this call to every peer (the stream work that produced this rank's inputs is complete)
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int s = 0; s < c.world; ++s) st_release_sys(c.sig[s] + SIG_STARTED + c.rank, c.epoch);
  }

  const int copy_ctas = c.mode == 1 ? c.copy_ctas : 0;
  if ((int)blockIdx.x < copy_ctas) {
    gather_stream(base, bar_base, c, m_tiles, tpr, (long long)BM * p.K * 2);
    return;
  }
  const int cta = blockIdx.x - copy_ctas, ctas = gridDim.x - copy_ctas;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);
    }
    *abort_flag = 0;
    *phase_ok = 1;
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
      uint32_t it = 0, issued = 0;
      int ready_block = -1;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += ctas) {
        int m0, n0;
        tile_coords_rot(t, m_tiles, n_tiles, tpr, c, m0, n0);
        if (c.mode == 1) {
          const int pm = m0 / BM;
          if (pm / tpr != c.rank && pm != ready_block) {
            ok = wait_reach<false>(c.sig[c.rank] + SIG_CHUNK + pm, c.epoch, c, 0x300u + pm / tpr);
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");  // the block was written by other CTAs; TMA reads it next
            ready_block = pm;
          }
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait_long(empty_bar(s), ((it / STAGES) & 1) ^ 1, abort_flag);
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
        if (p.err) atomicExch(p.err, 21);
        *abort_flag = 1;
        const uint32_t first = issued > STAGES ? issued - STAGES : 0;
        for (uint32_t i = first; i < issued; ++i)
          for (uint32_t spin = 0; spin < (1u << 16); ++spin)
            if (mbar_try_wait(full_bar(i % STAGES), (i / STAGES) & 1)) break;
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
      for (int t = cta; t < total_tiles && ok; t += ctas, ++local) {
        const uint32_t acc = local & 1;
        ok = mbar_wait_long(acc_empty_bar(acc), ((local >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * (uint32_t)BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait_long(full_bar(s), (it / STAGES) & 1, abort_flag);  // may sit behind a wait for a remote block
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t adesc = make_smem_desc(sa, p.a_mn_major), bdesc = make_smem_desc(sb, p.b_mn_major);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_d, adesc + (uint64_t)(a_step * k), bdesc + (uint64_t)(b_step * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty_bar(s));
        }
        if (ok) umma_commit(acc_full_bar(acc));
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 22);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const uint32_t my_stage = stage_out + (uint32_t)(warp - 2) * 8192u;
    uint32_t local = 0, stores = 0;
    bool ok = true;
    for (int t = cta; t < total_tiles && ok; t += ctas, ++local) {
      int m0, n0;
      tile_coords_rot(t, m_tiles, n_tiles, tpr, c, m0, n0);
      const uint32_t acc = local & 1;
      ok = mbar_wait_long(acc_full_bar(acc), (local >> 1) & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_row = tmem_base + acc * (uint32_t)BN + ((uint32_t)(q * 32) << 16);
      if (c.mode == 2) {
        const int owner = m0 / c.rows_per_rank;
        store_rows_tma(tmem_row, BN, n0, m0 - owner * c.rows_per_rank + q * 32, my_stage, stores, &maps_c.m[owner], p, lane);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      } else {
        store_rows_tma(tmem_row, BN, n0, m0 + q * 32, my_stage, stores, &maps_c.m[0], p, lane);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      }
    }
    if (lane == 0) {
      // every tile this warp stored, local or in a peer's staging slot, is complete and visible system-wide
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async;" ::: "memory");
      if (c.mode == 2) __threadfence_system();
    }
    if (!ok) {
      if (lane == 0 && p.err) atomicExch(p.err, 23);
      *abort_flag = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(v2::TMEM_COLS) : "memory");
  }
  if (c.mode != 2) return;

  // One counter update per owner and CTA (remote atomics on one address are slow when sent per tile): the number of
  // warp-level tile slices this CTA delivered to each owner, recomputed from the tile order.
  if (threadIdx.x == 0 && *abort_flag == 0) {
    unsigned sent[MAX_RANKS];
#pragma unroll
    for (int s = 0; s < MAX_RANKS; ++s) sent[s] = 0u;
    for (int t = cta; t < total_tiles; t += ctas) {
      int m0, n0;
      tile_coords_rot(t, m_tiles, n_tiles, tpr, c, m0, n0);
      const int owner = m0 / c.rows_per_rank;
#pragma unroll
      for (int s = 0; s < MAX_RANKS; ++s)
        if (s == owner) sent[s] += 4u;
    }
#pragma unroll
    for (int s = 0; s < MAX_RANKS; ++s)
      if (s < c.world && sent[s] != 0u) red_release_sys_add(c.sig[s] + SIG_COUNT + parity * MAX_RANKS + c.rank, sent[s]);
  }

  // ------------------------------------------------------------------ reduce the staged partials of this rank's rows
  if (threadIdx.x == 0) {
    const unsigned expected = (unsigned)(tpr * n_tiles * 4);
    bool ok = *abort_flag == 0;
    for (int s = 0; s < c.world && ok; ++s) ok = wait_reach<true>(c.sig[c.rank] + SIG_COUNT + parity * MAX_RANKS + s, expected, c, 0x400u + s);
    *phase_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (*phase_ok) {
    const long long vecs = (long long)c.rows_per_rank * p.N / 8;  // 16-byte vectors of the result
    const uint4* st = reinterpret_cast<const uint4*>(c.stage);
    uint4* out = reinterpret_cast<uint4*>(c.out);
    const long long first = (long long)cta * THREADS + threadIdx.x, step = (long long)ctas * THREADS;
    // eight 16-byte loads in flight per thread whatever the number of ranks
    if (c.world <= 2) reduce_staged<4, 2>(st, out, vecs, first, step, c.world);
    else if (c.world <= 4) reduce_staged<2, 4>(st, out, vecs, first, step, c.world);
    else reduce_staged<1, 8>(st, out, vecs, first, step, c.world);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last CTA to finish clears this parity's counters for the call after next
    const unsigned ticket = atomicAdd(c.sig[c.rank] + SIG_TICKET, 1u);
    if (ticket == (unsigned)ctas - 1u) {
      for (int s = 0; s < MAX_RANKS; ++s) c.sig[c.rank][SIG_COUNT + parity * MAX_RANKS + s] = 0u;
      c.sig[c.rank][SIG_TICKET] = 0u;
      __threadfence_system();
    }
  }
}

int sm_count() { return kb_sm_count(); }

bool prepare_kernel() {
  static bool done[KB_MAX_DEVICES] = {false};
  return kb_allow_smem(gemm_bf16_tcgen05_comm, v2::SMEM_BYTES, done);
}

}  // namespace

KB_API int kb200_gemm_comm_signal_words() { return SIG_WORDS; }

// C[world*Ms, N] = act(gather(A)[world*Ms, K] x B + bias).  `gather[r]` is rank r's gathered-A buffer of this call
// ([world*Ms, K] bf16, contiguous) as mapped here; this rank's slice is already in gather[rank].  B: [K, N] with
// b_mn_major = 1 or [N, K] with b_mn_major = 0, local memory.  `sig[r]`: signal pad of rank r (kb200_gemm_comm_signal_words
// zeroed unsigned words).  Ms must be a multiple of 128.
KB_API int kb200_gemm_allgather(void* const* gather, void* const* sig, const void* b, void* c, const float* bias, int rank, int world, int Ms, int N,
                                int K, long long ldb, long long ldc, int b_mn_major, int act, int out_fp32, unsigned epoch, int copy_ctas,
                                long long timeout_ms, unsigned* status, int* err, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || Ms <= 0 || Ms % v2::BM || N <= 0 || K <= 0 || K % 8 || ldb % 8 || ldc % (out_fp32 ? 4 : 8)) {
    kb200_set_error("gemm_allgather: needs 1..8 ranks, rows per rank a multiple of 128, K and pitches multiples of 8");
    return -2;
  }
  const int M = world * Ms;
  if (M / v2::BM > SIG_WORDS - SIG_CHUNK) {
    kb200_set_error("gemm_allgather: too many row blocks for the signal pad");
    return -2;
  }
  CUtensorMap map_a, map_b;
  CMaps maps_c;
  bool ok = make_map(&map_a, gather[rank], K, M, K, v2::BK, v2::BM);
  ok = ok && (b_mn_major ? make_map(&map_b, b, N, K, ldb, 64, v2::BK) : make_map(&map_b, b, K, N, ldb, v2::BK, v2::BN));
  ok = ok && make_map(&maps_c.m[0], c, N, M, ldc, out_fp32 ? 32 : 64, 32, out_fp32 != 0);
  for (int i = 1; i < MAX_RANKS; ++i) maps_c.m[i] = maps_c.m[0];
  if (!ok || !prepare_kernel()) {
    kb200_set_error("gemm_allgather: tensor map or kernel set-up failed");
    return -3;
  }
  GemmParams p{c, bias, M, N, K, ldc, 0, b_mn_major, act, out_fp32, err, 1, 0};
  CommParams cp{};
  cp.mode = 1;
  cp.rank = rank;
  cp.world = world;
  cp.epoch = epoch;
  cp.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
  cp.status = status;
  for (int i = 0; i < world; ++i) {
    cp.sig[i] = (unsigned*)sig[i];
    cp.gather[i] = (const uint8_t*)gather[i];
  }
  const int sms = sm_count();
  if (world == 1) {
    copy_ctas = 0;
  } else if (copy_ctas < 1) {
    // enough copy CTAs to bring the remote slices in within the time the GEMM takes: one CTA streams about 40 GB/s
    // (four 32 KB pieces in flight), the GEMM runs at roughly 1.3 PFLOP/s
    const double gemm_s = 2.0 * M * (double)N * K / 1.3e15;
    const double remote_bytes = (double)(world - 1) * Ms * K * 2.0;
    copy_ctas = (int)(1.5 * remote_bytes / (gemm_s * 40e9)) + 2;
    if (copy_ctas > 24) copy_ctas = 24;
  }
  if (copy_ctas > sms / 2) copy_ctas = sms / 2;
  cp.copy_ctas = copy_ctas;
  cp.rows_per_rank = Ms;
  const long long tiles = (long long)(M / v2::BM) * ((N + v2::BN - 1) / v2::BN);
  long long compute = tiles < sms - copy_ctas ? tiles : sms - copy_ctas;
  gemm_bf16_tcgen05_comm<<<(unsigned)(compute + copy_ctas), THREADS, v2::SMEM_BYTES, stream>>>(map_a, map_b, maps_c, p, cp);
  KB_CHECK_LAUNCH("gemm_allgather");
  return 0;
}

// out[Ms, N] = sum over ranks s of (A_s x B_s)[rank*Ms : (rank+1)*Ms, :].  A: [world*Ms, K] (a_mn_major = 0) or
// [K, world*Ms] (1), local; B as above.  `stage[r]`: rank r's staging buffer of this call ([world][Ms][N] bf16) as
// mapped here.  `out`: local bf16 [Ms, N], contiguous.  N must be a multiple of 8, Ms of 128.
KB_API int kb200_gemm_reduce_scatter(const void* a, const void* b, void* const* stage, void* const* sig, void* out, int rank, int world, int Ms, int N,
                                     int K, long long lda, long long ldb, int a_mn_major, int b_mn_major, unsigned epoch, long long timeout_ms,
                                     unsigned* status, int* err, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || Ms <= 0 || Ms % v2::BM || N <= 0 || N % 8 || K <= 0 || lda % 8 || ldb % 8) {
    kb200_set_error("gemm_reduce_scatter: needs 1..8 ranks, rows per rank a multiple of 128, N and pitches multiples of 8");
    return -2;
  }
  const int M = world * Ms;
  CUtensorMap map_a, map_b;
  CMaps maps_c;
  bool ok = a_mn_major ? make_map(&map_a, a, M, K, lda, 64, v2::BK) : make_map(&map_a, a, K, M, lda, v2::BK, v2::BM);
  ok = ok && (b_mn_major ? make_map(&map_b, b, N, K, ldb, 64, v2::BK) : make_map(&map_b, b, K, N, ldb, v2::BK, v2::BN));
  for (int o = 0; o < MAX_RANKS; ++o) {
    // this rank's slot inside owner o's staging buffer
    const int oo = o < world ? o : 0;
    const __nv_bfloat16* slot = (const __nv_bfloat16*)stage[oo] + (long long)rank * Ms * N;
    ok = ok && make_map(&maps_c.m[o], slot, N, Ms, N, 64, 32, false);
  }
  if (!ok || !prepare_kernel()) {
    kb200_set_error("gemm_reduce_scatter: tensor map or kernel set-up failed");
    return -3;
  }
  GemmParams p{nullptr, nullptr, M, N, K, N, a_mn_major, b_mn_major, ACT_NONE, 0, err, 1, 0};
  CommParams cp{};
  cp.mode = 2;
  cp.rank = rank;
  cp.world = world;
  cp.epoch = epoch;
  cp.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
  cp.status = status;
  for (int i = 0; i < world; ++i) cp.sig[i] = (unsigned*)sig[i];
  cp.copy_ctas = 0;
  cp.stage = (const __nv_bfloat16*)stage[rank];
  cp.out = (__nv_bfloat16*)out;
  cp.rows_per_rank = Ms;
  const int sms = sm_count();
  const long long tiles = (long long)(M / v2::BM) * ((N + v2::BN - 1) / v2::BN);
  gemm_bf16_tcgen05_comm<<<(unsigned)(tiles < sms ? tiles : sms), THREADS, v2::SMEM_BYTES, stream>>>(map_a, map_b, maps_c, p, cp);
  KB_CHECK_LAUNCH("gemm_reduce_scatter");
  return 0;
}
