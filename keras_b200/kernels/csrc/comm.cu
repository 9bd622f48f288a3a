// Collectives over NVLink peer memory for one-process-per-GPU jobs on a single NVSwitch node.
//
// The reference delegates gradient reduction to torch DistributedDataParallel, i.e. bucketed NCCL
// all-reduces (keras/src/backend/torch/trainer.py:83-92), and reduces every metric variable with its
// own NCCL call (:207-244).  Here every rank maps the other ranks' gradient arenas with CUDA IPC
// and a single kernel per step does a two-shot all-reduce in place: rank r sums slice r of all
// arenas with plain peer loads (fixed rank order, so all ranks hold bit-identical results) and
// stores the sum into slice r of every arena with peer stores.  Ranks meet at an entry and an exit
// barrier made of release/acquire flags in a small IPC-shared signal pad.
//
// Every wait is bounded (iteration count and wall-clock): when it runs out the kernel raises the
// status word, leaves the data untouched and returns, so a lost peer surfaces as a Python
// exception rather than a hung GPU.  Peer data is read with plain vector loads only.
#include "common.cuh"

namespace {

constexpr int KB_MAX_RANKS = 16;

struct KbPeers {
  float* base[KB_MAX_RANKS];      // arena of every rank as mapped into this process (base[rank] is local)
  unsigned* signal[KB_MAX_RANKS];  // signal pad of every rank
};

// Signal pad layout (unsigned words): [0, 16) entry flags, [16, 32) exit flags, [32] finished-block counter
constexpr int SIG_ENTRY = 0, SIG_EXIT = 16, SIG_COUNTER = 32;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// All threads of the block call this.  Threads t < n wait until flags[t] has reached `epoch`.
// Returns false (and raises *status) when the wait ran out.
__device__ bool wait_flags(const unsigned* flags, int n, unsigned epoch, unsigned long long timeout_ns, unsigned* status, int code) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < n) {
    const unsigned long long t0 = global_ns();
    for (long long it = 0;; ++it) {
      if ((int)(ld_acquire_sys(flags + threadIdx.x) - epoch) >= 0) break;
      if ((it & 63) == 63 && *(volatile unsigned*)status != 0u) { ok = 0; break; }  // another block already gave up
      if (it > (1ll << 26) || global_ns() - t0 > timeout_ns) {
        ok = 0;
        atomicCAS(status, 0u, (unsigned)(code * 256 + threadIdx.x + 1));
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  return ok != 0;
}

__device__ __forceinline__ float4 ld_peer(const float* p) { return __ldcv(reinterpret_cast<const float4*>(p)); }

// In-place collective on `n` floats (n % 4 == 0) living at the same offset in every rank's arena.  The region is cut into
// `world` slices; rank r works on slice r (broadcast: the root works on the whole region).
//   mode 0  all-reduce       slice r of every arena := scale * sum over ranks of slice r
//   mode 1  reduce-scatter   slice r of this arena  := scale * sum over ranks of slice r
//   mode 2  all-gather       slice r of every arena := slice r of this arena
//   mode 3  broadcast        every arena := arena of rank `root`
enum { COMM_ALLREDUCE = 0, COMM_REDUCE_SCATTER = 1, COMM_ALLGATHER = 2, COMM_BROADCAST = 3 };

// The epoch of a collective is `epoch` plus, when `epoch_ctr` is given, the value of that device-side counter: the counter
// holds the epoch of the last completed collective of this communicator and allreduce_wait_kernel advances it.  With the
// counter in device memory the launch arguments are the same for every call, so a recorded (CUDA graph) step can be
// replayed.
__global__ void __launch_bounds__(512) allreduce_twoshot_kernel(KbPeers peers, int rank, int world, long long n, float scale, unsigned epoch,
                                                               const unsigned* epoch_ctr, unsigned long long timeout_ns, unsigned* status, int mode,
                                                               int root) {
  unsigned* my_sig = peers.signal[rank];
  if (epoch_ctr != nullptr) epoch += *epoch_ctr;
  // entry: tell every rank that this arena is complete, wait until every arena is
  if (blockIdx.x == 0 && (int)threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(peers.signal[threadIdx.x] + SIG_ENTRY + rank, epoch);
  }
  const bool entered = wait_flags(my_sig + SIG_ENTRY, world, epoch, timeout_ns, status, 1);

  const long long vecs = entered ? n / 4 : 0;  // a rank that gave up moves no data but still keeps its block counter consistent
  const long long per = (vecs + world - 1) / world;
  long long lo = per * rank, hi = min(vecs, lo + per);
  if (mode == COMM_BROADCAST) {
    lo = 0;
    hi = rank == root ? vecs : 0;
  }
  const bool reduce = mode == COMM_ALLREDUCE || mode == COMM_REDUCE_SCATTER;
  const bool spread = mode != COMM_REDUCE_SCATTER;
  for (long long v = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; v < hi; v += (long long)gridDim.x * blockDim.x) {
    float4 acc;
    if (reduce) {
      acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float4 part[KB_MAX_RANKS];
#pragma unroll
      for (int p = 0; p < KB_MAX_RANKS; ++p)
        if (p < world) part[p] = ld_peer(peers.base[p] + v * 4);
#pragma unroll
      for (int p = 0; p < KB_MAX_RANKS; ++p)
        if (p < world) { acc.x += part[p].x; acc.y += part[p].y; acc.z += part[p].z; acc.w += part[p].w; }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    } else {
      acc = *reinterpret_cast<const float4*>(peers.base[rank] + v * 4);
    }
    if (spread) {
#pragma unroll
      for (int p = 0; p < KB_MAX_RANKS; ++p)
        if (p < world && (reduce || p != rank)) *reinterpret_cast<float4*>(peers.base[p] + v * 4) = acc;
    } else {
      *reinterpret_cast<float4*>(peers.base[rank] + v * 4) = acc;
    }
  }
  // exit: the last block of this rank publishes "my slice is stored everywhere"
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = (atomicAdd(my_sig + SIG_COUNTER, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) my_sig[SIG_COUNTER] = 0u;
    if ((int)threadIdx.x < world && *(volatile unsigned*)status == 0u) {
      __threadfence_system();
      st_release_sys(peers.signal[threadIdx.x] + SIG_EXIT + rank, epoch);
    }
  }
}

// Waits until every rank has stored its slice (follows allreduce_twoshot_kernel on the same stream).
__global__ void allreduce_wait_kernel(KbPeers peers, int rank, int world, unsigned epoch, unsigned* epoch_ctr, unsigned long long timeout_ns,
                                      unsigned* status) {
  if (epoch_ctr != nullptr) epoch += *epoch_ctr;
  if (*(volatile unsigned*)status == 0u) wait_flags(peers.signal[rank] + SIG_EXIT, world, epoch, timeout_ns, status, 2);
  __syncthreads();
  if (epoch_ctr != nullptr && threadIdx.x == 0) *epoch_ctr = epoch;  // also after a time-out: later calls must not reuse an epoch
}

}  // namespace

// ---------------------------------------------------------------------------------------------------
// CUDA IPC plumbing: buffers that peers may map.  Allocation happens once per engine, never per step.
KB_API int kb200_ipc_alloc(long long bytes, void** ptr, void* handle64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) { kb200_set_error(cudaGetErrorString(e)); return -1; }
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { kb200_set_error(cudaGetErrorString(e)); cudaFree(p); return -1; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}

KB_API int kb200_ipc_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { kb200_set_error(cudaGetErrorString(e)); return -1; }
  *ptr = p;
  return 0;
}

KB_API int kb200_ipc_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) { kb200_set_error(cudaGetErrorString(e)); return -1; }
  return 0;
}

KB_API int kb200_ipc_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) { kb200_set_error(cudaGetErrorString(e)); return -1; }
  return 0;
}

// bases / signals: arrays of `world` device pointers (as mapped in this process).  `offset_floats` selects a region
// of the arenas (same in every rank), `n` its length in floats; both multiples of 4.  status: one unsigned word
// that the host can read (0 = fine).  The reduction is complete on `stream` when both kernels have run.
KB_API int kb200_collective_p2p(void* const* bases, void* const* signals, int rank, int world, long long offset_floats, long long n, float scale,
                                unsigned epoch, unsigned* epoch_ctr, long long timeout_ms, unsigned* status, int mode, int root, cudaStream_t stream);

KB_API int kb200_allreduce_p2p(void* const* bases, void* const* signals, int rank, int world, long long offset_floats, long long n, float scale,
                               unsigned epoch, long long timeout_ms, unsigned* status, cudaStream_t stream) {
  return kb200_collective_p2p(bases, signals, rank, world, offset_floats, n, scale, epoch, nullptr, timeout_ms, status, COMM_ALLREDUCE, 0, stream);
}

// mode: 0 all-reduce, 1 reduce-scatter, 2 all-gather, 3 broadcast from `root` (see allreduce_twoshot_kernel).
// epoch_ctr: optional device word owned by this rank's communicator; the call's epoch is then `epoch + *epoch_ctr` (pass
// epoch = 1) and the counter is advanced on the device when the call completes.
KB_API int kb200_collective_p2p(void* const* bases, void* const* signals, int rank, int world, long long offset_floats, long long n, float scale,
                                unsigned epoch, unsigned* epoch_ctr, long long timeout_ms, unsigned* status, int mode, int root, cudaStream_t stream) {
  if (mode < 0 || mode > 3 || root < 0 || root >= world) { kb200_set_error("collective_p2p: bad mode or root"); return -2; }
  if (world < 1 || world > KB_MAX_RANKS) { kb200_set_error("allreduce_p2p: world size must be in [1, 16]"); return -2; }
  if ((n & 3) != 0 || (offset_floats & 3) != 0) { kb200_set_error("allreduce_p2p: offset and length must be multiples of 4 floats"); return -2; }
  if (n == 0) return 0;
  KbPeers peers;
  for (int p = 0; p < KB_MAX_RANKS; ++p) {
    peers.base[p] = p < world ? (float*)bases[p] + offset_floats : nullptr;
    peers.signal[p] = p < world ? (unsigned*)signals[p] : nullptr;
  }
  const long long vecs_per_rank = mode == COMM_BROADCAST ? n / 4 : (n / 4 + world - 1) / world;
  long long blocks = (vecs_per_rank + 511) / 512;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  const unsigned long long timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
  allreduce_twoshot_kernel<<<(int)blocks, 512, 0, stream>>>(peers, rank, world, n, scale, epoch, epoch_ctr, timeout_ns, status, mode, root);
  KB_CHECK_LAUNCH("allreduce_twoshot");
  allreduce_wait_kernel<<<1, 32, 0, stream>>>(peers, rank, world, epoch, epoch_ctr, timeout_ns, status);
  KB_CHECK_LAUNCH("allreduce_wait");
  return 0;
}

// Bounded-wait self-test: waits `timeout_ms` for a flag that nothing sets and reports through *status.
// Used by tests of the failure path; it touches no peer memory.
KB_API int kb200_wait_selftest(unsigned* flag, unsigned* status, long long timeout_ms, cudaStream_t stream) {
  KbPeers peers;
  for (int p = 0; p < KB_MAX_RANKS; ++p) { peers.base[p] = nullptr; peers.signal[p] = nullptr; }
  peers.signal[0] = flag - SIG_EXIT;
  allreduce_wait_kernel<<<1, 32, 0, stream>>>(peers, 0, 1, 1u, nullptr, (unsigned long long)timeout_ms * 1000000ull, status);
  KB_CHECK_LAUNCH("wait_selftest");
  return 0;
}
