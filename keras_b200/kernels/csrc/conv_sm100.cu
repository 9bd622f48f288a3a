// Channels-last 2-D convolution as an implicit GEMM on 5th-generation tensor cores (tcgen05), sm_100a.
//
// Replaces the cuDNN convolutions behind keras/src/backend/torch/nn.py:623-717 (forward) and their autograd
// companions (input gradient, weight gradient), plus the statistics pass of the BatchNormalization that follows a
// convolution (keras/src/backend/torch/nn.py:1020-1043).
//
// The im2col matrix never exists.  Pixels are tiled as boxes (wt x ht x nt, powers of two, 128 or 64 pixels) of the
// NHWC tensor; one TMA box load `cp.async.bulk.tensor.4d` of 64 channels brings such a box into shared memory as 128-byte
// rows in exactly the swizzled layout a tcgen05 operand needs, and the filter tap (r, s) is nothing but an offset added
// to the box's (w, h) coordinates: positions outside the image read as zeros (TMA out-of-bounds fill), which is the zero
// padding.  A strided convolution with a 1x1 filter reads a strided view (the tensor map carries the strides).
//
//   mode "igemm" (forward and input gradient):
//       D[pixel, n] = sum over taps, channels c of  A[pixel + offset(tap), c] * B[tap][c][n]
//       forward:        A = x,  B = kernel[r][s][cin][cout]  (rows are the contraction: MN-major operand)
//       input gradient: A = dy, B = the same kernel array read as [cout -> contraction][cin -> n] (K-major operand),
//                       taps applied with mirrored offsets
//     Epilogue: bias / activation, bf16 TMA box store (or reduce-add into the destination), and per-channel
//     sum / sum of squares of the bf16-rounded outputs for BatchNormalization, accumulated in registers over all tiles
//     of the CTA and written once per warp (deterministic: no atomics).
//   mode "wgrad" (weight gradient):
//       dW[tap][c][n] = sum over pixels  x[pixel + offset(tap), c] * dy[pixel, n]
//     Both operands are MN-major views of the very same pixel boxes; the pixel range is cut into slices that run as
//     separate work units and add their fp32 partial tiles into dW with TMA reduce stores.
//
// Kernel structure as the persistent GEMM (gemm_sm100.cu): warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 =
// epilogue; 4 operand stages; two 256-column TMEM accumulators so an epilogue overlaps the next tile's main loop.
// Every wait is bounded; on expiry an error code is stored and the CTA drains and leaves.
#include "gemm_sm100.cuh"

namespace {
using namespace kbgemm;

constexpr int CV_A_BYTES = 128 * 64 * 2;            // 16 KB: 128 pixels x 64 channels (igemm) / 64 pixels x 128 channels (wgrad)
constexpr int CV_BAR_BYTES = 512;
constexpr int CV_MAX_STAGES = 12;
constexpr int CV_SMEM_BYTES = 227 * 1024;           // everything a CTA may have
constexpr int CV_IGEMM_THREADS = 320;               // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue (two sets of four lane quarters)
// operand bytes (resident kernel slice / dY ring + operand ring) left beside the staging buffers of `epi_sets` sets of four
// epilogue warps (two 4 KB buffers per warp)
constexpr int cv_oper_bytes(int epi_sets) { return (CV_SMEM_BYTES - 1024 /*alignment slack*/ - CV_BAR_BYTES - epi_sets * 4 * 8192) / 1024 * 1024; }
constexpr uint32_t CV_TMEM_COLS = 512;

struct ConvParams {
  int mode;                 // 0: igemm, 1: wgrad
  int lw, lh, lt;           // log2 of the pixel box (wt, ht) and of the pixels per box (7 or 6); nt = 2^(lt - lw - lh)
  int tiles_w, tiles_h, tiles_n;
  int Wo, Ho, No;           // extents of the tiled pixel space
  int n_tiles, bn;          // tiles and tile width along the GEMM N dimension (bn = 64, 128 or 256)
  int Ngemm;                // extent of the GEMM N dimension (channels of the result)
  int kc_blocks;            // igemm: 64-channel blocks of the contraction per tap
  int R, S, dh0, dh_step, dw0, dw_step;
  int b_kmajor;             // igemm: 1 = B rows run along N (input gradient), 0 = along the contraction (forward)
  int rows_per_tap;         // rows of the kernel matrix per tap (input channels)
  const float* bias;
  int act;
  int accumulate;           // igemm: add the bf16 result into the destination
  float* stats;             // igemm: [grid][2][stats_ld] per-CTA partial sums (or null)
  int stats_ld;
  int* err;
  // shared-memory plan: [resident region or dY ring: res_bytes][operand ring: stages x stage_bytes][staging][barriers]
  int stages, stage_bytes, res_bytes;
  int rank2;                // pixels are one flat dimension (1x1 filter, stride 1): 2-D tensor maps, which the TMA unit walks faster
  int oper_bytes, epi_sets; // operand region size; sets of four epilogue warps that share a tile's columns (1 or 2)
  int resident_b;           // igemm: this CTA's column slice of the kernel array stays in shared memory for all tiles
  int epi_alt;              // igemm, 64-column tiles: the two sets of epilogue warps take alternate tiles (each its own accumulator)
  // igemm, rows shared between vertical taps: one box of (ht + R - 1) image rows per (column offset s, channel block) serves
  // the R taps of that column.  A tap's operand is the same shared-memory tile entered `row offset * wt` pixels further on:
  // with wt a multiple of 8 that is a multiple of 1024 bytes, so the 128-byte swizzle pattern of the tile still applies.
  int hshare;
  int a_bytes;              // bytes of the activation box of one stage (16 KB without hshare)
  int h_first;              // hshare: image-row offset of the box relative to the tile's first output row
  int h_sign;               // hshare: +1 when tap r reads box row r, -1 when it reads box row R - 1 - r
  // wgrad
  int m_tiles;              // 128-row tiles over the input channels
  int split, pb_per, total_pb;
  int Mrows;                // R * S * Cin
  int items, group;         // accumulators (128 rows of dW each) in total / per work unit
  int pair_taps;            // Cin == 64: one accumulator holds the rows of two taps
  int b_slots;              // depth of the dY ring
  // wgrad, rows shared between vertical taps: one x box with a halo of image rows per (kernel column s, channel tile) is
  // the operand of several accumulators.  Cin > 64: accumulator a is tap (a, s), its operand the box entered a image rows
  // further on; the two 64-channel halves are two boxes `a_half` bytes apart.  Cin == 64: accumulator a holds the taps
  // (2a, s) and (2a + 1, s); its second 64 rows come from the same box one image row further on, which the descriptor
  // expresses as a leading-dimension offset of one image row (wt * 128 bytes).
  int vshare;
  int n_acc;                // accumulators fed by one stage
  int a_rows;               // image rows of the box
  int a_half;               // bytes of one box
  int acc_step;             // bytes between the operand starts of consecutive accumulators
  int lbo16;                // leading-dimension byte offset of the A descriptor / 16
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// Epilogue of one 32-row slice of an igemm accumulator tile: bf16 output through a swizzled staging buffer and a 4-D TMA
// box store; optional per-channel statistics in `acc` (4 chunks x {sum0, sum1, sq0, sq1} for the two columns a lane owns).
template <int CHUNKS>
__device__ __forceinline__ void conv_store_rows(uint32_t tmem_row, int ng0, int q, int w0, int h0, int n0, uint32_t stage, uint32_t& stores,
                                                const CUtensorMap* map_c, const ConvParams& p, int lane, float* acc, int c_begin) {
  const int wt_mask = (1 << p.lw) - 1, ht_mask = (1 << p.lh) - 1;
  const int r = q * 32 + lane;
  const bool valid = (w0 + (r & wt_mask) < p.Wo) && (h0 + ((r >> p.lw) & ht_mask) < p.Ho) && (n0 + (r >> (p.lw + p.lh)) < p.No);
  const int r0 = q * 32;
  const int bw0 = w0 + (r0 & wt_mask), bh0 = h0 + ((r0 >> p.lw) & ht_mask), bn0 = n0 + (r0 >> (p.lw + p.lh));
  const bool box_ok = bw0 < p.Wo && bh0 < p.Ho && bn0 < p.No;
  const uint32_t sw = (uint32_t)(lane & 7);
  // two register sets: the tensor-memory load of chunk c+1 is in flight while chunk c is converted and staged
  uint32_t ra[64], rb[64];
  tmem_row += (uint32_t)(c_begin * 64);
  ng0 += c_begin * 64;
  tmem_ld32(tmem_row, ra);
  tmem_ld32(tmem_row + 32u, ra + 32);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col0 = ng0 + c * 64;
    uint32_t* rr = (c & 1) ? rb : ra;
    uint32_t* rn = (c & 1) ? ra : rb;
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (c + 1 < CHUNKS) {
      tmem_ld32(tmem_row + (uint32_t)((c + 1) * 64), rn);
      tmem_ld32(tmem_row + (uint32_t)((c + 1) * 64 + 32), rn + 32);
    }
    if (col0 < p.Ngemm) {
      // the staging buffer about to be reused must have been read out by the TMA engine
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      __syncwarp();
      const uint32_t buf0 = stage + (stores & 1u) * 4096u;
      const uint32_t buf = buf0 + (uint32_t)lane * 128u;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[h * 32 + j]);
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += __ldg(p.bias + min(col0 + h * 32 + j, p.Ngemm - 1));
        }
        if (p.act != ACT_NONE) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
        }
        if (!valid) {  // pixels beyond the image: clipped by the store, and they must not enter the statistics
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const bf16x8 pk = pack8(v + u * 8);
          const uint4 w = *reinterpret_cast<const uint4*>(&pk);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + (((uint32_t)(h * 4 + u) ^ sw) << 4)), "r"(w.x), "r"(w.y), "r"(w.z),
                       "r"(w.w) : "memory");
        }
      }
      if (p.stats != nullptr) {
        // column sums over the 32 rows just staged: lane L owns columns 2L and 2L+1 of the chunk
        __syncwarp();
        float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
        const uint32_t cbase = buf0 + (uint32_t)(lane & 3) * 4u;
        const uint32_t cch = (uint32_t)(lane >> 2);
#pragma unroll 8
        for (int i = 0; i < 32; ++i) {
          uint32_t w;
          asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w) : "r"(cbase + (uint32_t)i * 128u + ((cch ^ (uint32_t)(i & 7)) << 4)) : "memory");
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
          s0 += f.x; q0 = fmaf(f.x, f.x, q0);
          s1 += f.y; q1 = fmaf(f.y, f.y, q1);
        }
        acc[c * 4 + 0] += s0; acc[c * 4 + 1] += s1; acc[c * 4 + 2] += q0; acc[c * 4 + 3] += q1;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0 && box_ok) {
        if (p.rank2) {
          if (p.accumulate) {
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c), "r"(buf0),
                         "r"(col0), "r"(bw0) : "memory");
          } else {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c), "r"(buf0), "r"(col0), "r"(bw0)
                         : "memory");
          }
        } else if (p.accumulate) {
          asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map_c), "r"(buf0),
                       "r"(col0), "r"(bw0), "r"(bh0), "r"(bn0) : "memory");
        } else {
          asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map_c), "r"(buf0), "r"(col0),
                       "r"(bw0), "r"(bh0), "r"(bn0) : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
      if (box_ok) ++stores;  // buffers alternate per committed store group (see store_rows_tma)
    }
  }
}

__device__ __forceinline__ void pixel_tile_origin(const ConvParams& p, int ptile, int& w0, int& h0, int& n0) {
  const int tw = ptile % p.tiles_w;
  const int rest = ptile / p.tiles_w;
  const int th = rest % p.tiles_h;
  const int tn = rest / p.tiles_h;
  w0 = tw << p.lw;
  h0 = th << p.lh;
  n0 = tn << (p.lt - p.lw - p.lh);
}


// Shared-memory carve-up common to both kernels.
struct ConvSmem {
  uint32_t res, ring, out, bar;
  uint8_t* bar_ptr;
};
__device__ __forceinline__ ConvSmem conv_smem(uint8_t* smem_raw, const ConvParams& p) {
  ConvSmem s;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  s.res = base;
  s.ring = base + (uint32_t)p.res_bytes;
  s.out = base + (uint32_t)p.oper_bytes;
  s.bar = s.out + (uint32_t)((p.epi_alt ? 2 : p.epi_sets) * 4 * 8192);
  s.bar_ptr = smem_raw + (s.bar - smem_u32(smem_raw));
  return s;
}
// barrier slots (8 bytes each): full[12] empty[12] acc_full[2] acc_empty[2] b_full[4] b_empty[4] | tmem slot | abort flag
__device__ __forceinline__ uint32_t bar_full(const ConvSmem& s, int i) { return s.bar + 8u * (uint32_t)i; }
__device__ __forceinline__ uint32_t bar_empty(const ConvSmem& s, int i) { return s.bar + 8u * (uint32_t)(CV_MAX_STAGES + i); }
__device__ __forceinline__ uint32_t bar_acc_full(const ConvSmem& s, int i) { return s.bar + 8u * (uint32_t)(2 * CV_MAX_STAGES + i); }
__device__ __forceinline__ uint32_t bar_acc_empty(const ConvSmem& s, int i) { return s.bar + 8u * (uint32_t)(2 * CV_MAX_STAGES + 2 + i); }
__device__ __forceinline__ uint32_t bar_b_full(const ConvSmem& s, int i) { return s.bar + 8u * (uint32_t)(2 * CV_MAX_STAGES + 4 + i); }
__device__ __forceinline__ uint32_t bar_b_empty(const ConvSmem& s, int i) { return s.bar + 8u * (uint32_t)(2 * CV_MAX_STAGES + 8 + i); }

__device__ __forceinline__ void conv_prologue(const ConvSmem& s, const ConvParams& p, int acc_empty_count, volatile uint32_t*& tmem_slot,
                                              volatile int*& abort_flag) {
  uint64_t* bars = reinterpret_cast<uint64_t*>(s.bar_ptr);
  tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * CV_MAX_STAGES + 12);
  abort_flag = reinterpret_cast<volatile int*>(bars + 2 * CV_MAX_STAGES + 13);
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(bar_full(s, i), 1);
      mbar_init(bar_empty(s, i), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_acc_full(s, a), 1);
      mbar_init(bar_acc_empty(s, a), acc_empty_count);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_b_full(s, i), 1);
      mbar_init(bar_b_empty(s, i), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if ((threadIdx.x >> 5) == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(CV_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Give copies that were issued before an abort a bounded time to land (the CTA must not exit under them).
__device__ __forceinline__ void conv_drain(const ConvSmem& s, const ConvParams& p, uint32_t issued) {
  const uint32_t first = issued > (uint32_t)p.stages ? issued - (uint32_t)p.stages : 0;
  for (uint32_t i = first; i < issued; ++i) {
    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
      if (mbar_try_wait(bar_full(s, (int)(i % (uint32_t)p.stages)), (i / (uint32_t)p.stages) & 1)) break;
  }
}

// ------------------------------------------------------------------------------------------------ forward / input gradient
__global__ void __launch_bounds__(CV_IGEMM_THREADS, 1)
conv_igemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                          const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  const ConvSmem s = conv_smem(smem_raw, p);
  volatile uint32_t* tmem_slot;
  volatile int* abort_flag;
  conv_prologue(s, p, p.epi_alt ? 4 : 8, tmem_slot, abort_flag);
  const uint32_t tmem_base = *tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = p.R * p.S;
  const int STAGES = p.stages;
  const int total_units = p.tiles_w * p.tiles_h * p.tiles_n * p.n_tiles;
  const int ng0 = (blockIdx.x % p.n_tiles) * p.bn;  // the grid is a multiple of n_tiles: one column tile per CTA
  const uint32_t b_block = (uint32_t)p.bn * 128u;   // bytes of one 64-deep slice of the kernel tile

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0, issued = 0;
      bool ok = true;
      if (p.resident_b) {
        mbar_expect_tx(bar_b_full(s, 0), (uint32_t)p.res_bytes);
        for (int tap = 0; tap < taps; ++tap) {
          const int brow = tap * p.rows_per_tap;
          for (int kc = 0; kc < p.kc_blocks; ++kc) {
            const uint32_t sb = s.res + (uint32_t)(tap * p.kc_blocks + kc) * b_block;
            if (p.b_kmajor) {
              tma_load_2d(sb, &map_b, bar_b_full(s, 0), kc * 64, brow + ng0);
            } else {
              for (int j = 0; j < (p.bn >> 6); ++j) tma_load_2d(sb + j * 8192, &map_b, bar_b_full(s, 0), ng0 + j * 64, brow + kc * 64);
            }
          }
        }
      }
      for (int u = blockIdx.x; u < total_units && ok && p.hshare; u += gridDim.x) {
        int w0, h0, n0;
        pixel_tile_origin(p, u / p.n_tiles, w0, h0, n0);
        for (int sc = 0; sc < p.S && ok; ++sc) {
          const int dw = p.dw0 + sc * p.dw_step;
          for (int kc = 0; kc < p.kc_blocks; ++kc, ++it) {
            const int st = it % STAGES;
            ok = mbar_wait(bar_empty(s, st), ((it / STAGES) & 1) ^ 1, abort_flag);
            if (!ok) break;
            const uint32_t sa = s.ring + (uint32_t)(st * p.stage_bytes);
            mbar_expect_tx(bar_full(s, st), (uint32_t)p.stage_bytes);
            tma_load_4d(sa, &map_a, bar_full(s, st), kc * 64, w0 + dw, h0 + p.h_first, n0);
            if (!p.resident_b) {
              for (int r = 0; r < p.R; ++r) {
                const uint32_t sb = sa + (uint32_t)p.a_bytes + (uint32_t)r * b_block;
                const int brow = (r * p.S + sc) * p.rows_per_tap;
                if (p.b_kmajor) {
                  tma_load_2d(sb, &map_b, bar_full(s, st), kc * 64, brow + ng0);
                } else {
                  for (int j = 0; j < (p.bn >> 6); ++j) tma_load_2d(sb + j * 8192, &map_b, bar_full(s, st), ng0 + j * 64, brow + kc * 64);
                }
              }
            }
            issued = it + 1;
          }
        }
      }
      for (int u = blockIdx.x; u < total_units && ok && !p.hshare; u += gridDim.x) {
        int w0, h0, n0;
        pixel_tile_origin(p, u / p.n_tiles, w0, h0, n0);
        for (int tap = 0; tap < taps && ok; ++tap) {
          const int dh = p.dh0 + (tap / p.S) * p.dh_step, dw = p.dw0 + (tap % p.S) * p.dw_step;
          const int brow = tap * p.rows_per_tap;
          for (int kc = 0; kc < p.kc_blocks; ++kc, ++it) {
            const int st = it % STAGES;
            ok = mbar_wait(bar_empty(s, st), ((it / STAGES) & 1) ^ 1, abort_flag);
            if (!ok) break;
            const uint32_t sa = s.ring + (uint32_t)(st * p.stage_bytes);
            mbar_expect_tx(bar_full(s, st), (uint32_t)p.stage_bytes);
            if (p.rank2) tma_load_2d(sa, &map_a, bar_full(s, st), kc * 64, w0 + dw);
            else tma_load_4d(sa, &map_a, bar_full(s, st), kc * 64, w0 + dw, h0 + dh, n0);
            if (!p.resident_b) {
              const uint32_t sb = sa + (uint32_t)p.a_bytes;
              if (p.b_kmajor) {
                tma_load_2d(sb, &map_b, bar_full(s, st), kc * 64, brow + ng0);
              } else {
                for (int j = 0; j < (p.bn >> 6); ++j) tma_load_2d(sb + j * 8192, &map_b, bar_full(s, st), ng0 + j * 64, brow + kc * 64);
              }
            }
            issued = it + 1;
          }
        }
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 21);
        *abort_flag = 1;
        conv_drain(s, p, issued);
      }
      if (p.resident_b) {  // the kernel slice must have landed before the CTA may exit
        for (uint32_t spin = 0; spin < (1u << 20); ++spin)
          if (mbar_try_wait(bar_b_full(s, 0), 0)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t b_mn = p.b_kmajor ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (b_mn << 16) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t a_step = 32u >> 4;
      const uint32_t b_step = b_mn ? (2048u >> 4) : (32u >> 4);
      uint32_t it = 0, local = 0;
      bool ok = true;
      if (p.resident_b) {
        ok = mbar_wait(bar_b_full(s, 0), 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      const int steps = p.hshare ? p.S * p.kc_blocks : taps * p.kc_blocks;
      const uint32_t row_bytes = (uint32_t)(128u << p.lw);  // one image row of the tile: wt pixels of 128 bytes
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++local) {
        const uint32_t acc = local & 1;
        ok = mbar_wait(bar_acc_empty(s, acc), ((local >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * 256u;
        for (int k = 0; k < steps; ++k, ++it) {
          const int st = it % STAGES;
          ok = mbar_wait(bar_full(s, st), (it / STAGES) & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = s.ring + (uint32_t)(st * p.stage_bytes);
          if (p.hshare) {
            const int sc = k / p.kc_blocks, kc = k - sc * p.kc_blocks;
            for (int r = 0; r < p.R; ++r) {
              const int box_row = p.h_sign > 0 ? r : p.R - 1 - r;
              const uint32_t sb = p.resident_b ? s.res + (uint32_t)((r * p.S + sc) * p.kc_blocks + kc) * b_block
                                               : sa + (uint32_t)p.a_bytes + (uint32_t)r * b_block;
              const uint64_t adesc = make_smem_desc(sa + (uint32_t)box_row * row_bytes, false), bdesc = make_smem_desc(sb, b_mn != 0);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_bf16(tmem_d, adesc + (uint64_t)(a_step * kk), bdesc + (uint64_t)(b_step * kk), idesc, (k > 0 || r > 0 || kk > 0) ? 1u : 0u);
            }
          } else {
            const uint32_t sb = p.resident_b ? s.res + (uint32_t)k * b_block : sa + (uint32_t)p.a_bytes;
            const uint64_t adesc = make_smem_desc(sa, false), bdesc = make_smem_desc(sb, b_mn != 0);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_bf16(tmem_d, adesc + (uint64_t)(a_step * kk), bdesc + (uint64_t)(b_step * kk), idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty(s, st));
        }
        if (ok) umma_commit(bar_acc_full(s, acc));
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 22);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Two sets of four warps (one warp per tensor-memory lane quarter in each set).  With epi_sets == 2 the sets split the
    // tile's 64-column chunks between them; with epi_sets == 1 the second set only takes part in the barriers.
    const int q = warp & 3;
    const int ew = warp - 2, set = ew >> 2;
    // With 64-column tiles one set of four warps would do all the work: the sets then take alternate tiles instead, set k
    // always reading accumulator k.
    const bool alt = p.epi_alt != 0;
    const bool active = alt || set < p.epi_sets;
    const int cps = (p.bn >> 6) / p.epi_sets;  // chunks per set
    const int c_begin = alt ? 0 : set * cps;
    const uint32_t my_stage = s.out + (uint32_t)ew * 8192u;
    uint32_t local = 0, stores = 0;
    bool ok = true;
    float acc_stats[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc_stats[i] = 0.f;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++local) {
      const uint32_t acc = local & 1;
      if (alt && (int)acc != set) continue;
      ok = mbar_wait(bar_acc_full(s, acc), (local >> 1) & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (active) {
        const uint32_t tmem_row = tmem_base + acc * 256u + ((uint32_t)(q * 32) << 16);
        int w0, h0, n0;
        pixel_tile_origin(p, u / p.n_tiles, w0, h0, n0);
        if (cps == 4) conv_store_rows<4>(tmem_row, ng0, q, w0, h0, n0, my_stage, stores, &map_c, p, lane, acc_stats, c_begin);
        else if (cps == 2) conv_store_rows<2>(tmem_row, ng0, q, w0, h0, n0, my_stage, stores, &map_c, p, lane, acc_stats, c_begin);
        else conv_store_rows<1>(tmem_row, ng0, q, w0, h0, n0, my_stage, stores, &map_c, p, lane, acc_stats, c_begin);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(s, acc));
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (p.stats != nullptr) {
      // combine the warps' column sums in a fixed order (reproducible) and write one row pair per CTA
      __syncwarp();  // lane 0 has waited for this warp's stores: the staging buffers are free
      if (active) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c < cps) {
            const uint32_t o = my_stage + (uint32_t)((c_begin + c) * 64 + 2 * lane) * 4u;
            asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(o), "f"(acc_stats[c * 4 + 0]), "f"(acc_stats[c * 4 + 1]) : "memory");
            asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(o + 1024u), "f"(acc_stats[c * 4 + 2]), "f"(acc_stats[c * 4 + 3]) : "memory");
          }
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight epilogue warps
      const int tid = threadIdx.x - 64;
      float* dst = p.stats + (size_t)blockIdx.x * 2 * p.stats_ld + ng0;
      for (int col = tid; col < p.bn; col += 256) {
        const uint32_t owner = s.out + (uint32_t)(((col >> 6) / cps) * 4) * 8192u + (uint32_t)col * 4u;
        float sum = 0.f, sq = 0.f;
        const int contributors = alt ? 8 : 4;  // alternating sets: both sets hold sums of this column
        for (int w = 0; w < contributors; ++w) {
          float a, b;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a) : "r"(owner + (uint32_t)w * 8192u) : "memory");
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(b) : "r"(owner + (uint32_t)w * 8192u + 1024u) : "memory");
          sum += a;
          sq += b;
        }
        dst[col] = sum;
        dst[p.stats_ld + col] = sq;
      }
    }
    if (!ok) {
      if (lane == 0 && p.err) atomicExch(p.err, 23);
      *abort_flag = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(CV_TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ weight gradient
// Work unit = (group of up to `group` accumulators, column tile, slice of the pixel range).  An accumulator holds 128 rows
// of dW: one (tap, 128-channel tile) pair, or two taps when Cin == 64.  For every 64-pixel block of its slice the unit
// loads the dY box once (dY ring) and one shifted x box per accumulator (operand ring), so dY crosses L2 -> shared memory
// once per group instead of once per tap.  All accumulators of the unit live in tensor memory until the slice is done.
__device__ __forceinline__ void wgrad_unit(const ConvParams& p, int u, int& item0, int& cnt, int& ng0, int& pb0, int& pb1) {
  const int groups = (p.items + p.group - 1) / p.group;
  const int grp = u % groups;
  const int rest = u / groups;
  ng0 = (rest % p.n_tiles) * p.bn;
  const int slice = rest / p.n_tiles;
  item0 = grp * p.group;
  cnt = min(p.group, p.items - item0);
  pb0 = slice * p.pb_per;
  pb1 = min(pb0 + p.pb_per, p.total_pb);
}

__global__ void __launch_bounds__(THREADS, 1)
conv_wgrad_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                          const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  const ConvSmem s = conv_smem(smem_raw, p);
  volatile uint32_t* tmem_slot;
  volatile int* abort_flag;
  conv_prologue(s, p, 4, tmem_slot, abort_flag);
  const uint32_t tmem_base = *tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = p.R * p.S;
  const int STAGES = p.stages, BSLOTS = p.b_slots;
  const int groups = (p.items + p.group - 1) / p.group;
  const int total_units = groups * p.n_tiles * p.split;
  const uint32_t b_bytes = (uint32_t)p.bn * 128u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0, bit = 0, issued = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        int item0, cnt, ng0, pb0, pb1;
        wgrad_unit(p, u, item0, cnt, ng0, pb0, pb1);
        for (int pb = pb0; pb < pb1 && ok; ++pb, ++bit) {
          int w0, h0, n0;
          pixel_tile_origin(p, pb, w0, h0, n0);
          const int bs = bit % BSLOTS;
          ok = mbar_wait(bar_b_empty(s, bs), ((bit / BSLOTS) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t sb = s.res + (uint32_t)bs * b_bytes;
          mbar_expect_tx(bar_b_full(s, bs), b_bytes);
          if (p.rank2) {
            for (int j = 0; j < (p.bn >> 6); ++j) tma_load_2d(sb + j * 8192, &map_b, bar_b_full(s, bs), ng0 + j * 64, w0);
          } else {
            for (int j = 0; j < (p.bn >> 6); ++j) tma_load_4d(sb + j * 8192, &map_b, bar_b_full(s, bs), ng0 + j * 64, w0, h0, n0);
          }
          for (int i = 0; i < cnt; ++i, ++it) {
            const int st = it % STAGES;
            ok = mbar_wait(bar_empty(s, st), ((it / STAGES) & 1) ^ 1, abort_flag);
            if (!ok) break;
            const uint32_t sa = s.ring + (uint32_t)(st * p.stage_bytes);
            mbar_expect_tx(bar_full(s, st), (uint32_t)p.stage_bytes);
            const int item = item0 + i;
            if (p.vshare) {
              const int sc = item / p.m_tiles, c0 = (item % p.m_tiles) * 128;
              const int dw = p.dw0 + sc * p.dw_step;
              tma_load_4d(sa, &map_a, bar_full(s, st), c0, w0 + dw, h0 + p.dh0, n0);
              if (!p.pair_taps) tma_load_4d(sa + (uint32_t)p.a_half, &map_a, bar_full(s, st), c0 + 64, w0 + dw, h0 + p.dh0, n0);
            } else if (p.pair_taps) {
              const int ta = 2 * item, tb = 2 * item + 1;
              tma_load_4d(sa, &map_a, bar_full(s, st), 0, w0 + p.dw0 + (ta % p.S) * p.dw_step, h0 + p.dh0 + (ta / p.S) * p.dh_step, n0);
              if (tb < taps) {
                tma_load_4d(sa + 8192, &map_a, bar_full(s, st), 0, w0 + p.dw0 + (tb % p.S) * p.dw_step, h0 + p.dh0 + (tb / p.S) * p.dh_step, n0);
              } else {
                tma_load_4d(sa + 8192, &map_a, bar_full(s, st), 64, w0, h0, n0);  // channels 64.. do not exist: zero fill
              }
            } else {
              const int tap = item / p.m_tiles, c0 = (item % p.m_tiles) * 128;
              const int dh = p.dh0 + (tap / p.S) * p.dh_step, dw = p.dw0 + (tap % p.S) * p.dw_step;
              if (p.rank2) {
                tma_load_2d(sa, &map_a, bar_full(s, st), c0, w0 + dw);
                tma_load_2d(sa + 8192, &map_a, bar_full(s, st), c0 + 64, w0 + dw);
              } else {
                tma_load_4d(sa, &map_a, bar_full(s, st), c0, w0 + dw, h0 + dh, n0);
                tma_load_4d(sa + 8192, &map_a, bar_full(s, st), c0 + 64, w0 + dw, h0 + dh, n0);
              }
            }
            issued = it + 1;
          }
        }
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 31);
        *abort_flag = 1;
        conv_drain(s, p, issued);
        for (int i = 0; i < BSLOTS; ++i)
          for (uint32_t spin = 0; spin < (1u << 14); ++spin)
            if (mbar_try_wait(bar_b_full(s, i), 0) || mbar_try_wait(bar_b_full(s, i), 1)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t step = 2048u >> 4;
      uint32_t it = 0, bit = 0, local = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++local) {
        int item0, cnt, ng0, pb0, pb1;
        wgrad_unit(p, u, item0, cnt, ng0, pb0, pb1);
        ok = mbar_wait(bar_acc_empty(s, 0), (local & 1) ^ 1, abort_flag);  // the epilogue has drained the previous unit
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int pb = pb0; pb < pb1 && ok; ++pb, ++bit) {
          const int bs = bit % BSLOTS;
          ok = mbar_wait(bar_b_full(s, bs), (bit / BSLOTS) & 1, abort_flag);
          if (!ok) break;
          const uint64_t bdesc = make_smem_desc(s.res + (uint32_t)bs * b_bytes, true);
          for (int i = 0; i < cnt; ++i, ++it) {
            const int st = it % STAGES;
            ok = mbar_wait(bar_full(s, st), (it / STAGES) & 1, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = s.ring + (uint32_t)(st * p.stage_bytes);
            if (p.vshare) {
              for (int a = 0; a < p.n_acc; ++a) {
                // same descriptor as make_smem_desc(.., true) with the leading-dimension offset of this mode
                uint64_t adesc = make_smem_desc(sa + (uint32_t)(a * p.acc_step), true);
                adesc = (adesc & ~(0x3FFFull << 16)) | ((uint64_t)p.lbo16 << 16);
                const uint32_t tmem_d = tmem_base + (uint32_t)((i * p.n_acc + a) * p.bn);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                  umma_bf16(tmem_d, adesc + (uint64_t)(step * kk), bdesc + (uint64_t)(step * kk), idesc, (pb > pb0 || kk > 0) ? 1u : 0u);
              }
            } else {
              const uint64_t adesc = make_smem_desc(sa, true);
              const uint32_t tmem_d = tmem_base + (uint32_t)(i * p.bn);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_bf16(tmem_d, adesc + (uint64_t)(step * kk), bdesc + (uint64_t)(step * kk), idesc, (pb > pb0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(bar_empty(s, st));
          }
          if (ok) umma_commit(bar_b_empty(s, bs));
        }
        if (ok) umma_commit(bar_acc_full(s, 0));
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 32);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const uint32_t my_stage = s.out + (uint32_t)(warp - 2) * 8192u;
    uint32_t local = 0, stores = 0;
    bool ok = true;
    GemmParams gp{};
    gp.M = p.Mrows; gp.N = p.Ngemm; gp.out_fp32 = 1; gp.split_k = 2;  // every unit adds its partial tiles (TMA reduce stores)
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++local) {
      int item0, cnt, ng0, pb0, pb1;
      wgrad_unit(p, u, item0, cnt, ng0, pb0, pb1);
      ok = mbar_wait(bar_acc_full(s, 0), local & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int i = 0; i < cnt; ++i) {
        const int item = item0 + i;
        if (p.vshare) {
          const int sc = item / p.m_tiles, ctile = item % p.m_tiles;
          for (int a = 0; a < p.n_acc; ++a) {
            // rows of dW that this warp's 32 accumulator rows are: tap (r, sc), channels from `ch`
            const int r = p.pair_taps ? 2 * a + (q >> 1) : a;
            const int ch = p.pair_taps ? (q & 1) * 32 : ctile * 128 + q * 32;
            if (r >= p.R) continue;  // the odd tap out of a pair: rows of a tap that does not exist
            const int row0 = (r * p.S + sc) * p.rows_per_tap + ch;
            const uint32_t tmem_row = tmem_base + (uint32_t)((i * p.n_acc + a) * p.bn) + ((uint32_t)(q * 32) << 16);
            store_rows_tma(tmem_row, p.bn, ng0, row0, my_stage, stores, &map_c, gp, lane);
          }
          continue;
        }
        const int row0 = (p.pair_taps ? item * 128 : (item / p.m_tiles) * p.rows_per_tap + (item % p.m_tiles) * 128) + q * 32;
        const uint32_t tmem_row = tmem_base + (uint32_t)(i * p.bn) + ((uint32_t)(q * 32) << 16);
        store_rows_tma(tmem_row, p.bn, ng0, row0, my_stage, stores, &map_c, gp, lane);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(s, 0));
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (!ok) {
      if (lane == 0 && p.err) atomicExch(p.err, 33);
      *abort_flag = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(CV_TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host side

// 4-D bf16 tensor map over (channels, w, h, n) with element strides (sw, sh, sn); box = (64, bw, bh, bn).
bool make_map_4d(CUtensorMap* map, const void* ptr, long long C, long long W, long long H, long long N, long long sw, long long sh, long long sn,
                 int bw, int bh, int bnn) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)sw * 2, (cuuint64_t)sh * 2, (cuuint64_t)sn * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bnn};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int ilog2i(int v) {
  int l = 0;
  while ((1 << (l + 1)) <= v) ++l;
  return l;
}

// Power-of-two box (wt, ht, nt) of `pixels` pixels that covers W x H x N with the least padding (ties: widest, then tallest).
void pick_box(int pixels, int W, int H, int N, int& lw, int& lh) {
  const int lt = ilog2i(pixels);
  long long best = -1;
  for (int a = lt; a >= 0; --a) {
    for (int b = lt - a; b >= 0; --b) {
      const int wt = 1 << a, ht = 1 << b, nt = 1 << (lt - a - b);
      const long long vol = (long long)((W + wt - 1) / wt) * ((H + ht - 1) / ht) * ((N + nt - 1) / nt);
      if (best < 0 || vol < best) {
        best = vol;
        lw = a;
        lh = b;
      }
    }
  }
}

int conv_sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (counts[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    counts[dev] = n;
  }
  return counts[dev];
}

bool conv_set_attr() {
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return false;
  if (!done[dev]) {
    if (cudaFuncSetAttribute(conv_igemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CV_SMEM_BYTES) != cudaSuccess) return false;
    if (cudaFuncSetAttribute(conv_wgrad_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CV_SMEM_BYTES) != cudaSuccess) return false;
    done[dev] = true;
  }
  return true;
}

int pick_bn(int n) { return n <= 64 ? 64 : (n <= 128 ? 128 : 256); }

// igemm: 64-column tiles let the two sets of epilogue warps take alternate tiles (KERAS_B200_CONV_EPI_ALT=0: one set works)
bool igemm_epi_alt(int bn) {
  static const int allow = [] { const char* e = getenv("KERAS_B200_CONV_EPI_ALT"); return (e != nullptr && e[0] == '0') ? 0 : 1; }();
  return allow && bn == 64;
}
// igemm: sets of epilogue warps that need staging buffers
int igemm_staging_sets(int bn, int steps) { return (igemm_epi_alt(bn) || (bn >= 128 && steps <= 12)) ? 2 : 1; }

bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

}  // namespace

namespace {
// Pixel tile of the forward / input-gradient kernel.  Vertical taps can share one box of (ht + R - 1) rows when the tile lies
// inside one image and is a multiple of 8 pixels wide: taken when it cuts the 128-byte rows the TMA unit has to fetch for the
// whole problem by a quarter or more.  Measured cost of a 4-D box is about 6 cycles per 128-byte row, which is what bounds the
// 3x3 layers with 64 and 128 channels.
void igemm_box(int Wo, int Ho, int N, int R, int S, int dh_step, int Ca, int Cn, int& lw, int& lh, int& hshare) {
  static const int allow = [] { const char* e = getenv("KERAS_B200_CONV_HSHARE"); return (e != nullptr && e[0] == '0') ? 0 : 1; }();
  pick_box(128, Wo, Ho, N, lw, lh);
  hshare = 0;
  if (!allow || R < 2 || R > 8 || (dh_step != 1 && dh_step != -1)) return;
  const int wt0 = 1 << lw, ht0 = 1 << lh, nt0 = 1 << (7 - lw - lh);
  const long long tiles_plain = (long long)((Wo + wt0 - 1) / wt0) * ((Ho + ht0 - 1) / ht0) * ((N + nt0 - 1) / nt0);
  const long long rows_plain = tiles_plain * R * S * 128;
  // KERAS_B200_CONV_HSHARE_LW=3..7 pins log2 of the tile width (for measurements)
  static const int pinned = [] { const char* e = getenv("KERAS_B200_CONV_HSHARE_LW"); return (e != nullptr && e[0] >= '3' && e[0] <= '7') ? e[0] - '0' : 0; }();
  long long best = -1;
  int best_lw = 0;
  for (int a = 3; a <= 7; ++a) {
    if (pinned && a != pinned) continue;
    const int wt1 = 1 << a, ht1 = 128 >> a;
    const long long tiles = (long long)((Wo + wt1 - 1) / wt1) * ((Ho + ht1 - 1) / ht1) * N;
    if (tiles * 4 > tiles_plain * 5) continue;  // at most a quarter more tiles (tensor-core and epilogue work) than the plain tiling
    const long long rows = tiles * S * wt1 * (ht1 + R - 1);
    if (best < 0 || rows < best) { best = rows; best_lw = a; }
  }
  if (best < 0 || best * 4 > rows_plain * 3) return;
  // the operand ring must still hold two stages (four when the kernel slice is resident): same arithmetic as the launcher's
  const int bn = pick_bn(Cn), kc_blocks = (Ca + 63) / 64;
  const int a_bytes = (1 << best_lw) * ((128 >> best_lw) + R - 1) * 128;
  const int oper = cv_oper_bytes(igemm_staging_sets(bn, R * S * kc_blocks));
  const long long bbytes = (long long)R * S * kc_blocks * bn * 128;
  if (bbytes > oper - 4 * a_bytes && 2 * (a_bytes + R * bn * 128) > oper) return;
  hshare = 1;
  lw = best_lw;
  lh = 7 - best_lw;
}
}  // namespace

// Launch plan of kb200_conv_igemm for a result of N x Ho x Wo pixels and Cn channels from Ca input channels and R x S taps: plan_out = {grid, n_tiles, bn}.
// The statistics buffer of that call needs grid * 2 * (n_tiles * bn) floats.
KB_API int kb200_conv_igemm_plan(int N, int Ho, int Wo, int Ca, int Cn, int R, int S, int dh_step, int* plan_out) {
  int lw = 0, lh = 0, hshare = 0;
  igemm_box(Wo, Ho, N, R, S, dh_step, Ca, Cn, lw, lh, hshare);
  const int wt = 1 << lw, ht = 1 << lh, nt = 1 << (7 - lw - lh);
  const int bn = pick_bn(Cn);
  const int n_tiles = (Cn + bn - 1) / bn;
  const long long total = (long long)((Wo + wt - 1) / wt) * ((Ho + ht - 1) / ht) * ((N + nt - 1) / nt) * n_tiles;
  const int sms = conv_sm_count();
  int grid = total <= sms ? (int)total : sms - sms % n_tiles;
  if (grid <= 0) grid = (int)(total < n_tiles ? total : n_tiles);
  plan_out[0] = grid;
  plan_out[1] = n_tiles;
  plan_out[2] = bn;
  return 0;
}

// 1 when the most recent kb200_conv_wgrad call of this process shared image rows between vertical taps (for tests; the call
// comes from autograd's worker thread, so the flag is per process).
static volatile int g_last_wgrad_shared = 0;
KB_API int kb200_conv_wgrad_last_shared() { return g_last_wgrad_shared; }

// 1 when kb200_conv_igemm would share image rows between the vertical taps for this problem.
KB_API int kb200_conv_igemm_shares_rows(int N, int Ho, int Wo, int Ca, int Cn, int R, int S, int dh_step) {
  int lw = 0, lh = 0, hshare = 0;
  igemm_box(Wo, Ho, N, R, S, dh_step, Ca, Cn, lw, lh, hshare);
  return hshare;
}

// Implicit-GEMM convolution, forward or input-gradient form.
//
//   a:   bf16 activations seen as (n, h, w, c) with element strides (a_sn, a_sh, a_sw, 1) and extents (N, H, W, Ca)
//   wgt: bf16 kernel array [R][S][rows_per_tap][w_cols] (Keras layout: rows = input channels, columns = filters)
//   out: bf16 result seen as (n, h, w, c) with element strides (c_sn, c_sh, c_sw, 1) and extents (N, Ho, Wo, Cn)
//   out[n, h, w, :] = act(bias + sum over r, s:  a[n, h + dh0 + r*dh_step, w + dw0 + s*dw_step, :] x B[r][s])
//   b_kmajor = 0: B[r][s] = wgt[r][s] (Ca = rows_per_tap contracted, Cn = w_cols)            -> forward
//   b_kmajor = 1: B[r][s] = wgt[r][s] transposed (Ca = w_cols contracted, Cn = rows_per_tap) -> input gradient
//   accumulate: add into `out` instead of overwriting it.
//   stats (optional): fp32 [grid][2][stats_ld] per-CTA partial sums of out and out^2 per channel over all pixels;
//   plan_out (optional) receives {grid, n_tiles, bn} so that the caller can reduce them (kb200_bn_finalize_partials).
// All channel counts and strides must be multiples of 8 elements and all base pointers 16-byte aligned.
KB_API int kb200_conv_igemm(const void* a, const void* wgt, void* out, const float* bias, float* stats, int stats_ld, int* plan_out, int N, int H, int W,
                            int Ca, long long a_sw, long long a_sh, long long a_sn, int Ho, int Wo, int Cn, long long c_sw, long long c_sh,
                            long long c_sn, int R, int S, int dh0, int dh_step, int dw0, int dw_step, int b_kmajor, int rows_per_tap, int w_cols,
                            int act, int accumulate, int* err, cudaStream_t stream) {
  if (N <= 0 || Ho <= 0 || Wo <= 0 || Cn <= 0 || Ca <= 0) return 0;
  if ((Ca % 8) || (Cn % 8) || (w_cols % 8) || (a_sw % 8) || (a_sh % 8) || (a_sn % 8) || (c_sw % 8) || (c_sh % 8) || (c_sn % 8) || !aligned16(a) ||
      !aligned16(wgt) || !aligned16(out)) {
    kb200_set_error("conv_igemm: channel counts and strides must be multiples of 8 and pointers 16-byte aligned");
    return -2;
  }
  if (!conv_set_attr()) {
    kb200_set_error("conv_igemm: cannot raise the shared-memory limit");
    return -5;
  }
  ConvParams p{};
  p.mode = 0;
  p.lt = 7;
  igemm_box(Wo, Ho, N, R, S, dh_step, Ca, Cn, p.lw, p.lh, p.hshare);
  p.a_bytes = CV_A_BYTES;
  if (p.hshare) {
    p.h_first = dh_step > 0 ? dh0 : dh0 + (R - 1) * dh_step;
    p.h_sign = dh_step > 0 ? 1 : -1;
    p.a_bytes = (1 << p.lw) * ((1 << p.lh) + R - 1) * 128;
  }
  const int wt = 1 << p.lw, ht = 1 << p.lh, nt = 1 << (p.lt - p.lw - p.lh);
  p.tiles_w = (Wo + wt - 1) / wt;
  p.tiles_h = (Ho + ht - 1) / ht;
  p.tiles_n = (N + nt - 1) / nt;
  p.Wo = Wo; p.Ho = Ho; p.No = N;
  p.bn = pick_bn(Cn);
  p.n_tiles = (Cn + p.bn - 1) / p.bn;
  p.Ngemm = Cn;
  p.kc_blocks = (Ca + 63) / 64;
  p.R = R; p.S = S; p.dh0 = dh0; p.dh_step = dh_step; p.dw0 = dw0; p.dw_step = dw_step;
  p.b_kmajor = b_kmajor;
  p.rows_per_tap = rows_per_tap;
  p.bias = bias; p.act = act; p.accumulate = accumulate;
  p.stats = stats; p.stats_ld = stats_ld;
  p.err = err;
  const long long total = (long long)p.tiles_w * p.tiles_h * p.tiles_n * p.n_tiles;
  if (total > 0x7fffffffLL) {
    kb200_set_error("conv_igemm: too many tiles");
    return -6;
  }
  const int sms = conv_sm_count();
  int grid = total <= sms ? (int)total : sms - sms % p.n_tiles;
  if (grid <= 0) grid = (int)(total < p.n_tiles ? total : p.n_tiles);
  if (plan_out != nullptr) {
    plan_out[0] = grid; plan_out[1] = p.n_tiles; plan_out[2] = p.bn;
  }
  if (stats != nullptr && stats_ld < p.n_tiles * p.bn) {
    kb200_set_error("conv_igemm: stats_ld is smaller than the padded channel count");
    return -7;
  }
  // shared-memory plan.  With few MMAs per tile the epilogue (about 1500 cycles per 64-column chunk and warp) is the
  // bottleneck: both sets of epilogue warps then work on a tile.  The kernel slice of this CTA's column tile stays resident
  // in shared memory when that leaves a ring of at least six 16 KB stages.
  const long long bbytes = (long long)R * S * p.kc_blocks * p.bn * 128;
  const int steps = R * S * p.kc_blocks;
  p.epi_sets = (p.bn >= 128 && steps <= 12) ? 2 : 1;
  p.epi_alt = igemm_epi_alt(p.bn) ? 1 : 0;
  p.oper_bytes = cv_oper_bytes(igemm_staging_sets(p.bn, steps));
  const int b_per_stage = (p.hshare ? R : 1) * p.bn * 128;
  if (bbytes <= p.oper_bytes - (p.hshare ? 4 : 6) * p.a_bytes) {
    p.resident_b = 1;
    p.res_bytes = (int)bbytes;
    p.stage_bytes = p.a_bytes;
  } else {
    p.resident_b = 0;
    p.res_bytes = 0;
    p.stage_bytes = p.a_bytes + b_per_stage;
  }
  p.stages = (p.oper_bytes - p.res_bytes) / p.stage_bytes;
  if (p.stages > CV_MAX_STAGES) p.stages = CV_MAX_STAGES;
  if (p.stages < 2) {
    kb200_set_error("conv_igemm: the operand ring does not fit two stages");
    return -8;
  }
  p.rank2 = (R == 1 && S == 1 && H == 1 && N == 1 && Ho == 1) ? 1 : 0;
  CUtensorMap map_a, map_b, map_c;
  bool ok = p.rank2 ? make_map(&map_a, a, Ca, W, a_sw, 64, 128)
                    : make_map_4d(&map_a, a, Ca, W, H, N, a_sw, a_sh, a_sn, wt, p.hshare ? ht + R - 1 : ht, nt);
  const long long wrows = (long long)R * S * rows_per_tap;
  ok = ok && (b_kmajor ? make_map(&map_b, wgt, w_cols, wrows, w_cols, 64, p.bn) : make_map(&map_b, wgt, w_cols, wrows, w_cols, 64, 64));
  const int sbw = wt < 32 ? wt : 32;
  const int sbh = (32 / sbw) < ht ? (32 / sbw) : ht;
  const int sbn = 32 / (sbw * sbh);
  ok = ok && (p.rank2 ? make_map(&map_c, out, Cn, Wo, c_sw, 64, 32) : make_map_4d(&map_c, out, Cn, Wo, Ho, N, c_sw, c_sh, c_sn, sbw, sbh, sbn));
  if (!ok) {
    kb200_set_error("conv_igemm: cuTensorMapEncodeTiled failed");
    return -3;
  }
  conv_igemm_tcgen05_kernel<<<(unsigned)grid, CV_IGEMM_THREADS, CV_SMEM_BYTES, stream>>>(map_a, map_b, map_c, p);
  KB_CHECK_LAUNCH("conv_igemm");
  return 0;
}

// Weight gradient: dw[r][s][c][n] += sum over pixels x[n_, h + dh0 + r*dh_step, w + dw0 + s*dw_step, c] * dy[n_, h, w, n].
//   x:  bf16 (N, H, W, Cin) with element strides (x_sn, x_sh, x_sw, 1);  dy: bf16 (N, Ho, Wo, Cout) with strides (d_sn, d_sh, d_sw, 1)
//   dw: fp32 [R*S*Cin, Cout] contiguous, ADDED to (zero it for a plain gradient).
KB_API int kb200_conv_wgrad(const void* x, const void* dy, float* dw, int N, int H, int W, int Cin, long long x_sw, long long x_sh, long long x_sn,
                            int Ho, int Wo, int Cout, long long d_sw, long long d_sh, long long d_sn, int R, int S, int dh0, int dh_step, int dw0,
                            int dw_step, int* err, cudaStream_t stream) {
  if (N <= 0 || Ho <= 0 || Wo <= 0 || Cin <= 0 || Cout <= 0) return 0;
  if ((Cin % 8) || (Cout % 8) || (x_sw % 8) || (x_sh % 8) || (x_sn % 8) || (d_sw % 8) || (d_sh % 8) || (d_sn % 8) || !aligned16(x) || !aligned16(dy) ||
      !aligned16(dw)) {
    kb200_set_error("conv_wgrad: channel counts and strides must be multiples of 8 and pointers 16-byte aligned");
    return -2;
  }
  if (!conv_set_attr()) {
    kb200_set_error("conv_wgrad: cannot raise the shared-memory limit");
    return -5;
  }
  ConvParams p{};
  p.mode = 1;
  p.lt = 6;
  pick_box(64, Wo, Ho, N, p.lw, p.lh);
  p.bn = pick_bn(Cout);
  {
    // Rows shared between vertical taps (see ConvParams::vshare): the pixel block lies inside one image and is a multiple
    // of 8 pixels wide; taken when it cuts the x rows the TMA unit fetches by a quarter or more with at most a quarter more
    // pixel blocks, and the accumulators of one stage fit the 512 tensor-memory columns.
    static const int allow = [] { const char* e = getenv("KERAS_B200_CONV_WGRAD_SHARE"); return (e != nullptr && e[0] == '0') ? 0 : 1; }();
    const bool pair = Cin == 64;
    const int n_acc = pair ? (R + 1) / 2 : R;
    const bool rank2_call = R == 1 && S == 1;
    if (allow && !rank2_call && R >= 2 && R <= 8 && dh_step == 1 && Cin >= 64 && n_acc * p.bn <= 512) {
      const int wt0 = 1 << p.lw, ht0 = 1 << p.lh, nt0 = 1 << (p.lt - p.lw - p.lh);
      const long long blocks_plain = (long long)((Wo + wt0 - 1) / wt0) * ((Ho + ht0 - 1) / ht0) * ((N + nt0 - 1) / nt0);
      const long long rows_plain = blocks_plain * R * S * 64;
      long long best = -1;
      int best_lw = 0;
      for (int a = 3; a <= 6; ++a) {
        const int wt1 = 1 << a, ht1 = 64 >> a;
        const long long blocks = (long long)((Wo + wt1 - 1) / wt1) * ((Ho + ht1 - 1) / ht1) * N;
        if (blocks * 4 > blocks_plain * 5) continue;
        const int box_rows = pair ? ht1 + 2 * n_acc - 1 : ht1 + R - 1;
        const long long rows = blocks * S * wt1 * box_rows;
        if (best < 0 || rows < best) { best = rows; best_lw = a; }
      }
      if (best > 0 && best * 4 <= rows_plain * 3) {
        p.vshare = 1;
        p.lw = best_lw;
        p.lh = 6 - best_lw;
        p.n_acc = n_acc;
        const int wt1 = 1 << p.lw, ht1 = 1 << p.lh;
        p.a_rows = pair ? ht1 + 2 * n_acc - 1 : ht1 + R - 1;  // a pair reaches one image row past its first tap
        p.a_half = wt1 * p.a_rows * 128;
        p.acc_step = (pair ? 2 : 1) * wt1 * 128;
        p.lbo16 = (pair ? wt1 * 128 : p.a_half) >> 4;
      }
    }
  }
  const int wt = 1 << p.lw, ht = 1 << p.lh, nt = 1 << (p.lt - p.lw - p.lh);
  p.tiles_w = (Wo + wt - 1) / wt;
  p.tiles_h = (Ho + ht - 1) / ht;
  p.tiles_n = (N + nt - 1) / nt;
  p.Wo = Wo; p.Ho = Ho; p.No = N;
  p.n_tiles = (Cout + p.bn - 1) / p.bn;
  p.Ngemm = Cout;
  p.R = R; p.S = S; p.dh0 = dh0; p.dh_step = dh_step; p.dw0 = dw0; p.dw_step = dw_step;
  p.rows_per_tap = Cin;
  p.m_tiles = (Cin + 127) / 128;
  p.Mrows = R * S * Cin;
  p.err = err;
  const long long pbs = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
  if (pbs > 0x7fffffffLL) {
    kb200_set_error("conv_wgrad: too many pixel blocks");
    return -6;
  }
  p.total_pb = (int)pbs;
  const int taps = R * S;
  p.pair_taps = (Cin == 64 && taps > 1) ? 1 : 0;
  p.b_slots = p.bn == 256 ? 2 : 3;
  p.res_bytes = p.b_slots * p.bn * 128;
  p.epi_sets = 1;
  p.oper_bytes = cv_oper_bytes(1);
  if (p.vshare) {
    p.items = S * p.m_tiles;                    // stage loads per pixel block; each feeds n_acc accumulators
    p.group = 512 / (p.bn * p.n_acc);
    if (p.group > p.items) p.group = p.items;
    p.stage_bytes = (p.pair_taps ? 1 : 2) * p.a_half;
  } else {
    p.items = p.pair_taps ? (taps + 1) / 2 : taps * p.m_tiles;
    p.group = 512 / p.bn < p.items ? 512 / p.bn : p.items;
    p.stage_bytes = CV_A_BYTES;
  }
  p.stages = (p.oper_bytes - p.res_bytes) / p.stage_bytes;
  if (p.stages > CV_MAX_STAGES) p.stages = CV_MAX_STAGES;
  if (p.stages < 2 || p.group < 1) {
    kb200_set_error("conv_wgrad: the operand ring does not fit two stages");
    return -8;
  }
  const int tiles = ((p.items + p.group - 1) / p.group) * p.n_tiles;
  const int sms = conv_sm_count();
  // slices of the pixel range: one wave of work units, at least 4 pixel blocks each
  int split = tiles >= sms ? 1 : sms / tiles;
  if (split > p.total_pb / 4) split = p.total_pb / 4;
  if (split < 1) split = 1;
  p.pb_per = (p.total_pb + split - 1) / split;
  p.split = (p.total_pb + p.pb_per - 1) / p.pb_per;
  const long long units = (long long)tiles * p.split;
  CUtensorMap map_a, map_b, map_c;
  p.rank2 = (R == 1 && S == 1 && H == 1 && N == 1 && Ho == 1) ? 1 : 0;
  bool ok = p.rank2 ? make_map(&map_a, x, Cin, W, x_sw, 64, 64) : make_map_4d(&map_a, x, Cin, W, H, N, x_sw, x_sh, x_sn, wt, p.vshare ? p.a_rows : ht, nt);
  ok = ok && (p.rank2 ? make_map(&map_b, dy, Cout, Wo, d_sw, 64, 64) : make_map_4d(&map_b, dy, Cout, Wo, Ho, N, d_sw, d_sh, d_sn, wt, ht, nt));
  ok = ok && make_map(&map_c, dw, Cout, p.Mrows, Cout, 32, 32, true);
  if (!ok) {
    kb200_set_error("conv_wgrad: cuTensorMapEncodeTiled failed");
    return -3;
  }
  const unsigned grid = (unsigned)(units < sms ? units : sms);
  g_last_wgrad_shared = p.vshare;
  conv_wgrad_tcgen05_kernel<<<grid, THREADS, CV_SMEM_BYTES, stream>>>(map_a, map_b, map_c, p);
  KB_CHECK_LAUNCH("conv_wgrad");
  return 0;
}

namespace {
// Patch matrix of a convolution with few input channels (the 7x7 stem on RGB): row = output pixel, columns = R groups of
// `seg` elements, the first S*C of which are the contiguous input run x[n, ih, iw0 .. iw0+S-1, :] and the rest zeros.
template <typename T>
__global__ void __launch_bounds__(256) im2col_rows_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out, int N, int H, int W, int C, int Ho, int Wo,
                                                          int R, int S, int sh, int sw, int pt, int pl, int seg, long long total) {
  // one thread per 16-byte vector of the patch matrix: consecutive threads write consecutive vectors and read
  // consecutive runs of the same input row
  const int run = S * C, vecs = seg >> 3, row_len = W * C;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(t % vecs);
    long long rest = t / vecs;
    const int r = (int)(rest % R);
    const long long pix = rest / R;
    const int ow = (int)(pix % Wo);
    rest = pix / Wo;
    const int oh = (int)(rest % Ho);
    const int n = (int)(rest / Ho);
    const int ih = oh * sh - pt + r;
    const int e0 = v << 3;
    const int off0 = (ow * sw - pl) * C + e0;  // element offset inside the input row
    float f[8];
    if (ih >= 0 && ih < H) {
      const T* src = x + ((long long)n * H + ih) * row_len;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int off = off0 + j;
        f[j] = (e0 + j < run && off >= 0 && off < row_len) ? to_f32<T>(src[off]) : 0.f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
    *reinterpret_cast<bf16x8*>(out + t * 8) = pack8(f);
  }
}
}  // namespace

// out[N*Ho*Wo, R*seg] (bf16) from x[N, H, W, C] (dtype 0: fp32, 1: bf16); seg >= S*C, a multiple of 8.
KB_API int kb200_im2col_rows(const void* x, void* out, int N, int H, int W, int C, int Ho, int Wo, int R, int S, int sh, int sw, int pt, int pl, int seg,
                             int dtype, cudaStream_t stream) {
  if (seg % 8 || seg < S * C || !aligned16(out)) {
    kb200_set_error("im2col_rows: seg must be a multiple of 8 and at least S*C");
    return -2;
  }
  const long long total = (long long)N * Ho * Wo * R * (seg / 8);
  if (total <= 0) return 0;
  const unsigned grid = (unsigned)((total + 255) / 256 < 148LL * 32 ? (total + 255) / 256 : 148LL * 32);
  if (dtype == 1)
    im2col_rows_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, N, H, W, C, Ho, Wo, R, S, sh, sw, pt, pl, seg, total);
  else
    im2col_rows_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (__nv_bfloat16*)out, N, H, W, C, Ho, Wo, R, S, sh, sw, pt, pl, seg, total);
  KB_CHECK_LAUNCH("im2col_rows");
  return 0;
}
