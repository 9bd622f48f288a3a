// Fused multi-tensor optimizer kernels (one launch updates every variable of a model).
//
// A descriptor table in device memory lists, per tensor, the parameter / gradient / slot pointers;
// a chunk table maps each thread block to (tensor, chunk).  The kernels fuse: gradient unscale,
// non-finite detection, decoupled weight decay, the moment updates, the parameter update, an
// optional bf16 shadow-weight write and zeroing of the consumed gradient.
// Update rules: Adam/AdamW as keras/src/optimizers/adam.py:101-138 (epsilon outside the sqrt, bias
// correction folded into alpha); SGD as keras/src/optimizers/sgd.py:96-128.
#include "common.cuh"

struct KbTensorDesc {
  float* param;
  float* grad;
  float* slot0;  // Adam m / SGD momentum (may be null for plain SGD)
  float* slot1;  // Adam v
  __nv_bfloat16* shadow;  // optional bf16 copy of the parameter
  long long numel;
  float decay;  // decoupled weight-decay coefficient of this tensor (0 when excluded): param *= 1 - lr*decay
  int pad;
};

struct KbChunk {
  int tensor;
  int pad;
  long long start;
};

constexpr int KB_OPT_THREADS = 256;
constexpr int KB_OPT_CHUNK = KB_OPT_THREADS * 4 * 8;  // 8192 elements per block

// Step scalars come either by value (`lr`, `alpha`) or, when `lr_ptr` is set, from device memory: the learning-rate
// variable and the iteration counter.  With device-resident scalars a captured CUDA graph of the step stays correct when
// the learning rate is reassigned or the counter advances between replays.
struct AdamArgs {
  float alpha, lr, beta1, beta2, eps, grad_scale;
  double beta1d, beta2d;
  const float* lr_ptr;
  const int* step_ptr;
  int zero_grad;
};

struct StepScalars {
  float lr, alpha;
};

// thread 0 resolves the scalars, every thread of the block gets them
__device__ __forceinline__ StepScalars adam_scalars(const AdamArgs& a) {
  __shared__ StepScalars s;
  if (threadIdx.x == 0) {
    s.lr = a.lr;
    s.alpha = a.alpha;
    if (a.lr_ptr != nullptr) {
      const double lr = (double)(*a.lr_ptr);
      const double t = (double)(*a.step_ptr) + 1.0;
      s.lr = (float)lr;
      s.alpha = (float)(lr * sqrt(1.0 - pow(a.beta2d, t)) / (1.0 - pow(a.beta1d, t)));
    }
  }
  __syncthreads();
  return s;
}

__device__ __forceinline__ float decay_factor(float wd, float lr) { return (float)(1.0 - (double)wd * (double)lr); }

__device__ __forceinline__ void adam_elem(float& p, float g, float& m, float& v, const AdamArgs& a, float alpha, float decay) {
  p *= decay;
  m += (g - m) * (1.f - a.beta1);
  v += (g * g - v) * (1.f - a.beta2);
  p -= alpha * m / (sqrtf(v) + a.eps);
}

__global__ void __launch_bounds__(KB_OPT_THREADS) adam_kernel(const KbTensorDesc* __restrict__ descs, const KbChunk* __restrict__ chunks,
                                                              AdamArgs a, int* __restrict__ found_inf) {
  const StepScalars sc = adam_scalars(a);
  const float alpha = sc.alpha;
  const KbChunk c = chunks[blockIdx.x];
  const KbTensorDesc d = descs[c.tensor];
  const float decay = decay_factor(d.decay, sc.lr);
  const long long end = min(d.numel, c.start + (long long)KB_OPT_CHUNK);
  const bool vec = ((((uintptr_t)d.param | (uintptr_t)d.grad | (uintptr_t)d.slot0 | (uintptr_t)d.slot1) & 15) == 0) && ((c.start & 3) == 0) &&
                   (d.shadow == nullptr || (((uintptr_t)d.shadow & 7) == 0));
  bool bad = false;
  if (vec) {
    for (long long i = c.start + threadIdx.x * 4ll; i + 3 < end; i += KB_OPT_THREADS * 4ll) {
      float4 p = *reinterpret_cast<float4*>(d.param + i);
      float4 g = *reinterpret_cast<const float4*>(d.grad + i);
      float4 m = *reinterpret_cast<float4*>(d.slot0 + i);
      float4 v = *reinterpret_cast<float4*>(d.slot1 + i);
      g.x *= a.grad_scale; g.y *= a.grad_scale; g.z *= a.grad_scale; g.w *= a.grad_scale;
      bad |= !(isfinite(g.x) && isfinite(g.y) && isfinite(g.z) && isfinite(g.w));
      adam_elem(p.x, g.x, m.x, v.x, a, alpha, decay);
      adam_elem(p.y, g.y, m.y, v.y, a, alpha, decay);
      adam_elem(p.z, g.z, m.z, v.z, a, alpha, decay);
      adam_elem(p.w, g.w, m.w, v.w, a, alpha, decay);
      *reinterpret_cast<float4*>(d.param + i) = p;
      *reinterpret_cast<float4*>(d.slot0 + i) = m;
      *reinterpret_cast<float4*>(d.slot1 + i) = v;
      if (a.zero_grad) *reinterpret_cast<float4*>(d.grad + i) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d.shadow) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
        *reinterpret_cast<__nv_bfloat162*>(d.shadow + i) = lo;
        *reinterpret_cast<__nv_bfloat162*>(d.shadow + i + 2) = hi;
      }
    }
    // tail (numel not a multiple of 4) handled by the scalar loop below
    const long long tail = c.start + ((end - c.start) & ~3ll);
    for (long long i = tail + threadIdx.x; i < end; i += KB_OPT_THREADS) {
      float p = d.param[i], g = d.grad[i] * a.grad_scale, m = d.slot0[i], v = d.slot1[i];
      bad |= !isfinite(g);
      adam_elem(p, g, m, v, a, alpha, decay);
      d.param[i] = p; d.slot0[i] = m; d.slot1[i] = v;
      if (a.zero_grad) d.grad[i] = 0.f;
      if (d.shadow) d.shadow[i] = __float2bfloat16_rn(p);
    }
  } else {
    for (long long i = c.start + threadIdx.x; i < end; i += KB_OPT_THREADS) {
      float p = d.param[i], g = d.grad[i] * a.grad_scale, m = d.slot0[i], v = d.slot1[i];
      bad |= !isfinite(g);
      adam_elem(p, g, m, v, a, alpha, decay);
      d.param[i] = p; d.slot0[i] = m; d.slot1[i] = v;
      if (a.zero_grad) d.grad[i] = 0.f;
      if (d.shadow) d.shadow[i] = __float2bfloat16_rn(p);
    }
  }
  if (found_inf != nullptr && bad) atomicOr(found_inf, 1);
}

struct SgdArgs {
  float lr, momentum, grad_scale;
  const float* lr_ptr;  // when set, the learning rate is read from device memory
  int nesterov, zero_grad;
};

__device__ __forceinline__ void sgd_elem(float& p, float g, float* m, const SgdArgs& a, float lr, float decay) {
  p *= decay;
  if (m != nullptr) {
    float mv = a.momentum * (*m) - lr * g;
    *m = mv;
    p += a.nesterov ? (a.momentum * mv - lr * g) : mv;
  } else {
    p -= lr * g;
  }
}

__global__ void __launch_bounds__(KB_OPT_THREADS) sgd_kernel(const KbTensorDesc* __restrict__ descs, const KbChunk* __restrict__ chunks,
                                                             SgdArgs a, int* __restrict__ found_inf) {
  const float lr = a.lr_ptr != nullptr ? *a.lr_ptr : a.lr;
  const KbChunk c = chunks[blockIdx.x];
  const KbTensorDesc d = descs[c.tensor];
  const float decay = decay_factor(d.decay, lr);
  const long long end = min(d.numel, c.start + (long long)KB_OPT_CHUNK);
  const bool has_m = d.slot0 != nullptr;
  const bool vec = ((((uintptr_t)d.param | (uintptr_t)d.grad | (uintptr_t)d.slot0) & 15) == 0) && ((c.start & 3) == 0) &&
                   (d.shadow == nullptr || (((uintptr_t)d.shadow & 7) == 0));
  bool bad = false;
  long long scalar_from = c.start;
  if (vec) {
    for (long long i = c.start + threadIdx.x * 4ll; i + 3 < end; i += KB_OPT_THREADS * 4ll) {
      float4 p = *reinterpret_cast<float4*>(d.param + i);
      float4 g = *reinterpret_cast<const float4*>(d.grad + i);
      float4 m = has_m ? *reinterpret_cast<float4*>(d.slot0 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      g.x *= a.grad_scale; g.y *= a.grad_scale; g.z *= a.grad_scale; g.w *= a.grad_scale;
      bad |= !(isfinite(g.x) && isfinite(g.y) && isfinite(g.z) && isfinite(g.w));
      sgd_elem(p.x, g.x, has_m ? &m.x : nullptr, a, lr, decay);
      sgd_elem(p.y, g.y, has_m ? &m.y : nullptr, a, lr, decay);
      sgd_elem(p.z, g.z, has_m ? &m.z : nullptr, a, lr, decay);
      sgd_elem(p.w, g.w, has_m ? &m.w : nullptr, a, lr, decay);
      *reinterpret_cast<float4*>(d.param + i) = p;
      if (has_m) *reinterpret_cast<float4*>(d.slot0 + i) = m;
      if (a.zero_grad) *reinterpret_cast<float4*>(d.grad + i) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d.shadow) {
        *reinterpret_cast<__nv_bfloat162*>(d.shadow + i) = __floats2bfloat162_rn(p.x, p.y);
        *reinterpret_cast<__nv_bfloat162*>(d.shadow + i + 2) = __floats2bfloat162_rn(p.z, p.w);
      }
    }
    scalar_from = c.start + ((end - c.start) & ~3ll);
  }
  for (long long i = scalar_from + threadIdx.x; i < end; i += KB_OPT_THREADS) {
    float p = d.param[i], g = d.grad[i] * a.grad_scale;
    bad |= !isfinite(g);
    float m = has_m ? d.slot0[i] : 0.f;
    sgd_elem(p, g, has_m ? &m : nullptr, a, lr, decay);
    d.param[i] = p;
    if (has_m) d.slot0[i] = m;
    if (a.zero_grad) d.grad[i] = 0.f;
    if (d.shadow) d.shadow[i] = __float2bfloat16_rn(p);
  }
  if (found_inf != nullptr && bad) atomicOr(found_inf, 1);
}

KB_API int kb200_opt_chunk_elems() { return KB_OPT_CHUNK; }
KB_API int kb200_opt_desc_bytes() { return (int)sizeof(KbTensorDesc); }

// lr_ptr / step_ptr (both or neither): the fp32 learning rate and the int32 count of completed updates in device memory;
// alpha is then computed on the device as lr * sqrt(1 - beta2^t) / (1 - beta1^t) with t = *step_ptr + 1.
KB_API int kb200_fused_adam(const void* descs, const void* chunks, int n_chunks, float alpha, float lr, double beta1, double beta2, float eps,
                            float grad_scale, int zero_grad, int* found_inf, const float* lr_ptr, const int* step_ptr, cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  if ((lr_ptr == nullptr) != (step_ptr == nullptr)) {
    kb200_set_error("fused_adam: lr_ptr and step_ptr must be given together");
    return -2;
  }
  AdamArgs a{alpha, lr, (float)beta1, (float)beta2, eps, grad_scale, beta1, beta2, lr_ptr, step_ptr, zero_grad};
  adam_kernel<<<n_chunks, KB_OPT_THREADS, 0, stream>>>((const KbTensorDesc*)descs, (const KbChunk*)chunks, a, found_inf);
  KB_CHECK_LAUNCH("fused_adam");
  return 0;
}

KB_API int kb200_fused_sgd(const void* descs, const void* chunks, int n_chunks, float lr, float momentum, int nesterov, float grad_scale,
                           int zero_grad, int* found_inf, const float* lr_ptr, cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  SgdArgs a{lr, momentum, grad_scale, lr_ptr, nesterov, zero_grad};
  sgd_kernel<<<n_chunks, KB_OPT_THREADS, 0, stream>>>((const KbTensorDesc*)descs, (const KbChunk*)chunks, a, found_inf);
  KB_CHECK_LAUNCH("fused_sgd");
  return 0;
}

// bf16 shadow refresh for tensors updated outside the fused path: dst = bf16(src)
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n && ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0)) {
    float4 v = *reinterpret_cast<const float4*>(src + i);
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(dst + i + 2) = __floats2bfloat162_rn(v.z, v.w);
  } else {
    for (long long k = i; k < min(n, i + 4); ++k) dst[k] = __float2bfloat16_rn(src[k]);
  }
}

KB_API int kb200_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long threads = (n + 3) / 4;
  int blocks = (int)((threads + 255) / 256);
  cast_f32_bf16_kernel<<<blocks, 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
  KB_CHECK_LAUNCH("cast_f32_bf16");
  return 0;
}
