// Flash attention forward on tcgen05 tensor cores: O = softmax(scale * Q K^T [+ causal mask]) V without materialising the
// score matrix.  Layout [batch, time, heads, head_dim] for Q, K, V and O (the layout of the attention layers), bf16 in and
// out, fp32 statistics; grouped-query attention by mapping query head h to key/value head h / (H / Hkv).
// Replaces the einsum -> masked softmax -> einsum chain (keras/src/layers/attention/multi_head_attention.py:574-608) and the
// library call behind keras/src/backend/torch/nn.py:1124-1175.
//
// One CTA per (128 query rows, head, batch element); 192 threads:
//   warp 0   TMA producer: Q once, then K/V blocks of 128 keys into a two-stage ring (4-D tiled copies, 128-byte swizzle)
//   warp 1   one elected thread issues S = Q K^T (128 x 128 x D) into TMEM, and, once the softmax warps have written the
//            probabilities P (bf16, shared memory, K-major) O_blk = P V (128 x D x 128) into a second TMEM region
//   warps 2-5 one thread per query row (= TMEM lane): running maximum and sum in the log2 domain without any shuffle, two
//            passes over S in TMEM (maximum, then exponentials), O accumulated and rescaled in registers; finally O / l is
//            staged in shared memory and written with TMA stores, and the log-sum-exp per row is stored for a backward pass.
// The tensor pipe runs S(j+1) while the softmax warps fold O_blk(j) into their registers; with head_dim 64 two CTAs share an
// SM and overlap one CTA's softmax with the other's matrix products.
//
// Every mbarrier wait is bounded (iteration limit + abort flag): on expiry the kernel writes a code to *err, lets its
// outstanding copies land, frees TMEM and returns.
#include "gemm_sm100.cuh"

namespace {
using namespace kbgemm;

struct FlashParams {
  int B, H, Hkv, Tq, Tk;
  float scale_log2;  // softmax scale times log2(e)
  int causal;
  float* lse;        // [B, H, Tq] natural-log sum of exponentials of the scaled scores
  int* err;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

template <int D>
struct FlashCfg {
  static constexpr int CH = D / 64;                 // 64-column chunks of the head dimension
  static constexpr int Q_BYTES = CH * 16384;        // [chunk][128 rows][128 B]
  static constexpr int KV_BYTES = CH * 16384;       // K: [chunk][128 keys][128 B];  V: [64-key block][chunk][64 keys][128 B]
  static constexpr int P_BYTES = 2 * 16384;         // [64-key chunk][128 rows][128 B]
  static constexpr int SMEM = Q_BYTES + 4 * KV_BYTES + P_BYTES + 256;  // no alignment slack: two CTAs of the D = 64 variant fit one SM
  static constexpr uint32_t TMEM_COLS = 256;        // S: columns 0-127, O block: columns 128..128+D
};

template <int D>
__global__ void __launch_bounds__(THREADS, D == 64 ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                 const __grid_constant__ CUtensorMap map_o, const FlashParams p) {
  using C = FlashCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // the 128-byte swizzle needs 1024-byte aligned tiles; without static shared memory the window starts aligned
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 30);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t sQ = base, sK = sQ + C::Q_BYTES, sV = sK + 2 * C::KV_BYTES, sP = sV + 2 * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + C::Q_BYTES + 4 * C::KV_BYTES + C::P_BYTES);
  const uint32_t bar_base = sP + C::P_BYTES;
  const uint32_t q_bar = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (3 + s); };
  const uint32_t s_full = bar_base + 8u * 5, p_ready = bar_base + 8u * 6, o_full = bar_base + 8u * 7, o_free = bar_base + 8u * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 128, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (p.H / p.Hkv);
  int n_blocks = (p.Tk + 127) / 128;
  if (p.causal) n_blocks = min(n_blocks, (q0 + 128 + 127) / 128);

  if (threadIdx.x == 0) {
    mbar_init(q_bar, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    mbar_init(o_full, 1);
    mbar_init(o_free, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(q_bar, C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < C::CH; ++c) tma_load_4d(sQ + c * 16384, &map_q, q_bar, c * 64, q0, h, b);
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_blocks; ++j) {
        const int s = j & 1;
        ok = mbar_wait(kv_empty(s), ((j >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(kv_full(s), 2 * C::KV_BYTES);
        const uint32_t k_dst = sK + s * C::KV_BYTES, v_dst = sV + s * C::KV_BYTES;
#pragma unroll
        for (int c = 0; c < C::CH; ++c) tma_load_4d(k_dst + c * 16384, &map_k, kv_full(s), c * 64, j * 128, hkv, b);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int c = 0; c < C::CH; ++c) tma_load_4d(v_dst + (kb * C::CH + c) * 8192, &map_v, kv_full(s), c * 64, j * 128 + kb * 64, hkv, b);
        issued = j + 1;
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 31);
        *abort_flag = 1;
        for (int j = max(0, issued - 2); j < issued; ++j)
          for (uint32_t spin = 0; spin < (1u << 16); ++spin)
            if (mbar_try_wait(kv_full(j & 1), (j >> 1) & 1)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = mbar_wait(q_bar, 0, abort_flag);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait(kv_full(s), (j >> 1) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // S = Q K^T; the softmax warps finished reading the previous S before they announced the previous P
#pragma unroll
        for (int c = 0; c < C::CH; ++c) {
          const uint64_t adesc = make_smem_desc(sQ + c * 16384, false), bdesc = make_smem_desc(sK + s * C::KV_BYTES + c * 16384, false);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_S, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(s_full);
        // O_blk = P V once P is in shared memory and the previous O block has been folded into the registers
        ok = mbar_wait(p_ready, j & 1, abort_flag);
        if (ok && j > 0) ok = mbar_wait(o_free, (j - 1) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t adesc = make_smem_desc(sP + kb * 16384, false);
          const uint64_t bdesc = make_smem_desc(sV + s * C::KV_BYTES + kb * C::CH * 8192, true);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_O, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)((2048u >> 4) * k), idesc_o, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(kv_empty(s));
      }
      if (!ok) {
        if (p.err) atomicExch(p.err, 32);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output (warps 2..5), one thread per query row
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(s_full, j & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int k0 = j * 128;
      const bool need_mask = (k0 + 127 >= p.Tk) || (p.causal && k0 + 127 > q0);
      // pass 1: row maximum of the scaled scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[64];
        tmem_ld32(tmem_S + lane_base + (uint32_t)(c * 64), r);
        tmem_ld32(tmem_S + lane_base + (uint32_t)(c * 64 + 32), r + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float s = __uint_as_float(r[i]) * p.scale_log2;
          if (need_mask) {
            const int kc = k0 + c * 64 + i;
            if (kc >= p.Tk || (p.causal && kc > qi)) s = -INFINITY;
          }
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // a fully masked row keeps zeros instead of NaNs
      const float alpha = exp2f(m - m_use);
      // fold the previous O block into the registers: O = (O + O_blk) * alpha
      if (j > 0) {
        ok = mbar_wait(o_full, (j - 1) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          uint32_t r[64];
          tmem_ld32(tmem_O + lane_base + (uint32_t)(c * 64), r);
          tmem_ld32(tmem_O + lane_base + (uint32_t)(c * 64 + 32), r + 32);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 64; ++i) o_acc[c * 64 + i] = (o_acc[c * 64 + i] + __uint_as_float(r[i])) * alpha;
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free);
      }
      l *= alpha;
      // pass 2: probabilities, their sum, and P (bf16) into shared memory as the K-major A operand of P V
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {  // 64 keys = one 128-byte row of P per step
        uint32_t r[64];
        tmem_ld32(tmem_S + lane_base + (uint32_t)(c * 64), r);
        tmem_ld32(tmem_S + lane_base + (uint32_t)(c * 64 + 32), r + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const uint32_t chunk = sP + (uint32_t)c * 16384u + (uint32_t)row * 128u;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float pv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float s = __uint_as_float(r[u * 8 + i]) * p.scale_log2;
            if (need_mask) {
              const int kc = k0 + c * 64 + u * 8 + i;
              if (kc >= p.Tk || (p.causal && kc > qi)) s = -INFINITY;
            }
            const float e = exp2f(s - m_use);
            pv[i] = e;
            l += e;
          }
          const bf16x8 pk = pack8(pv);
          const uint4 w = *reinterpret_cast<const uint4*>(&pk);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(chunk + (((uint32_t)u ^ (uint32_t)(row & 7)) << 4)), "r"(w.x), "r"(w.y), "r"(w.z),
                       "r"(w.w) : "memory");
        }
      }
      m = m_new;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && n_blocks > 0) {
      ok = mbar_wait(o_full, (n_blocks - 1) & 1, abort_flag);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_O + lane_base + (uint32_t)(c * 32), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = (o_acc[c * 32 + i] + __uint_as_float(r[i])) * inv_l;
        }
        // every P V product has completed (o_full of the last block), so the P buffer is free: stage O there
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          const uint32_t chunk = sP + (uint32_t)c * 16384u + (uint32_t)row * 128u;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const bf16x8 pk = pack8(o_acc + c * 64 + u * 8);
            const uint4 w = *reinterpret_cast<const uint4*>(&pk);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(chunk + (((uint32_t)u ^ (uint32_t)(row & 7)) << 4)), "r"(w.x), "r"(w.y),
                         "r"(w.z), "r"(w.w) : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && q0 + q * 32 < p.Tq) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_store_4d(&map_o, sP + (uint32_t)c * 16384u + (uint32_t)(q * 32) * 128u, c * 64, q0 + q * 32, h, b);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
        if (qi < p.Tq && p.lse != nullptr)
          p.lse[((long long)b * p.H + h) * p.Tq + qi] = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    }
    if (!ok) {
      if (lane == 0 && p.err) atomicExch(p.err, 33);
      *abort_flag = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

// 4-D bf16 tensor map over [batch, time, heads, head_dim] storage: dims (head_dim, time, heads, batch).
bool make_map_bthd(CUtensorMap* map, const void* ptr, int D, int T, int H, int B, long long stride_t, long long stride_h, long long stride_b, int box_d,
                   int box_t) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)stride_t * 2, (cuuint64_t)stride_h * 2, (cuuint64_t)stride_b * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_d, (cuuint32_t)box_t, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

// q, o: [B, Tq, H, D]; k, v: [B, Tk, Hkv, D]; bf16, unit stride on D, the other strides (in elements) multiples of 8 and the
// base pointers 16-byte aligned.  D is 64 or 128, H a multiple of Hkv.  lse: [B, H, Tq] fp32 (may be null).
KB_API int kb200_flash_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int H, int Hkv, int D,
                                     long long q_st, long long q_sh, long long q_sb, long long k_st, long long k_sh, long long k_sb, long long v_st,
                                     long long v_sh, long long v_sb, long long o_st, long long o_sh, long long o_sb, float scale, int causal, int* err,
                                     cudaStream_t stream) {
  if (B <= 0 || Tq <= 0 || Tk <= 0 || H <= 0) return 0;
  if ((D != 64 && D != 128) || Hkv <= 0 || H % Hkv) {
    kb200_set_error("flash_attention_fwd: head_dim must be 64 or 128 and the query heads a multiple of the key/value heads");
    return -2;
  }
  const long long strides[12] = {q_st, q_sh, q_sb, k_st, k_sh, k_sb, v_st, v_sh, v_sb, o_st, o_sh, o_sb};
  for (int i = 0; i < 12; ++i)
    if (strides[i] % 8) {
      kb200_set_error("flash_attention_fwd: strides must be multiples of 8 elements");
      return -2;
    }
  if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) != 0) {
    kb200_set_error("flash_attention_fwd: base pointers must be 16-byte aligned");
    return -2;
  }
  CUtensorMap map_q, map_k, map_v, map_o;
  bool ok = make_map_bthd(&map_q, q, D, Tq, H, B, q_st, q_sh, q_sb, 64, 128) && make_map_bthd(&map_k, k, D, Tk, Hkv, B, k_st, k_sh, k_sb, 64, 128) &&
            make_map_bthd(&map_v, v, D, Tk, Hkv, B, v_st, v_sh, v_sb, 64, 64) && make_map_bthd(&map_o, o, D, Tq, H, B, o_st, o_sh, o_sb, 64, 32);
  if (!ok) {
    kb200_set_error("flash_attention_fwd: cuTensorMapEncodeTiled failed");
    return -3;
  }
  FlashParams p{B, H, Hkv, Tq, Tk, scale * 1.4426950408889634f, causal, lse, err};
  dim3 grid((Tq + 127) / 128, H, B);
  static bool attr64[KB_MAX_DEVICES] = {false}, attr128[KB_MAX_DEVICES] = {false};
  if (D == 64) {
    if (!kb_allow_smem(flash_fwd_kernel<64>, FlashCfg<64>::SMEM, attr64)) { kb200_set_error("flash_attention: shared-memory limit"); return -3; }
    flash_fwd_kernel<64><<<grid, THREADS, FlashCfg<64>::SMEM, stream>>>(map_q, map_k, map_v, map_o, p);
  } else {
    if (!kb_allow_smem(flash_fwd_kernel<128>, FlashCfg<128>::SMEM, attr128)) { kb200_set_error("flash_attention: shared-memory limit"); return -3; }
    flash_fwd_kernel<128><<<grid, THREADS, FlashCfg<128>::SMEM, stream>>>(map_q, map_k, map_v, map_o, p);
  }
  KB_CHECK_LAUNCH("flash_attention_fwd");
  return 0;
}
