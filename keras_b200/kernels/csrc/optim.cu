// Fused multi-tensor optimizer kernels (one launch updates every variable of a model).
//
// A descriptor table in device memory lists, per tensor, the parameter / gradient / slot pointers;
// a chunk table maps each thread block to (tensor, chunk).  The kernels fuse: gradient unscale,
// non-finite detection, decoupled weight decay, the moment updates, the parameter update, an
// optional bf16 shadow-weight write and zeroing of the consumed gradient.
// Update rules: Adam/AdamW as keras/src/optimizers/adam.py:101-138 (epsilon outside the sqrt, bias
// correction folded into alpha); SGD as keras/src/optimizers/sgd.py:96-128; RMSprop, Adagrad, Adadelta, Adamax, Nadam and
// Lion through one rule template further down.
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

// ------------------------------------------------------------------------------------------------ other update rules
// One kernel template for the optimizers whose rule touches a parameter, its gradient and at most two slots:
//   RMSprop   keras/src/optimizers/rmsprop.py:120-160     slot0 velocity, slot1 momentum or average gradient
//   Adagrad   keras/src/optimizers/adagrad.py:82-99       slot0 accumulator
//   Adadelta  keras/src/optimizers/adadelta.py:98-130     slot0 accumulated gradient, slot1 accumulated delta
//   Adamax    keras/src/optimizers/adamax.py:110-135      slot0 momentum, slot1 norm
//   Nadam     keras/src/optimizers/nadam.py:110-160       slot0 momentum, slot1 velocity, u_product on the device
//   Lion      keras/src/optimizers/lion.py:110-135        slot0 momentum
// (the reference runs these as chains of torch._foreach_* calls: keras/src/backend/torch/optimizers/torch_*.py).
enum KbRule { RULE_RMSPROP = 0, RULE_ADAGRAD = 1, RULE_ADADELTA = 2, RULE_ADAMAX = 3, RULE_NADAM = 4, RULE_LION = 5 };

struct RuleArgs {
  float lr, grad_scale;
  float c[4];            // rule constants (see rule_elem)
  double b1, b2;         // beta_1 / beta_2 in double for the powers
  float k[4];            // step-dependent scalars when they come by value
  const float* lr_ptr;   // learning rate in device memory (or null)
  const int* step_ptr;   // count of completed updates in device memory (or null: k[] is used)
  const float* aux;      // Nadam: {u_t, u_{t+1}, u_product_t, 1 - beta_2^t} written by nadam_prepare_kernel
  int flags;             // RMSprop: bit 0 momentum slot, bit 1 centered
  int zero_grad;
};

struct RuleScalars {
  float lr, k0, k1, k2, k3;
};

template <int RULE>
__device__ __forceinline__ RuleScalars rule_scalars(const RuleArgs& a) {
  __shared__ RuleScalars s;
  if (threadIdx.x == 0) {
    s.lr = a.lr_ptr != nullptr ? *a.lr_ptr : a.lr;
    s.k0 = a.k[0]; s.k1 = a.k[1]; s.k2 = a.k[2]; s.k3 = a.k[3];
    if (RULE == RULE_ADAMAX && a.step_ptr != nullptr) s.k0 = (float)(1.0 - pow(a.b1, (double)(*a.step_ptr) + 1.0));
    if (RULE == RULE_NADAM && a.aux != nullptr) {
      s.k0 = a.aux[0]; s.k1 = a.aux[1]; s.k2 = a.aux[2]; s.k3 = a.aux[3];
    }
  }
  __syncthreads();
  return s;
}

// s0 / s1 are the slot values (unused ones are dummies that are not written back)
template <int RULE>
__device__ __forceinline__ void rule_elem(float& p, float g, float& s0, float& s1, const RuleArgs& a, const RuleScalars& sc, float decay) {
  p *= decay;
  if (RULE == RULE_RMSPROP) {  // c0 rho, c1 momentum, c2 epsilon
    s0 = a.c[0] * s0 + (1.f - a.c[0]) * g * g;
    float denom = s0 + a.c[2];
    if (a.flags & 2) {
      s1 = a.c[0] * s1 + (1.f - a.c[0]) * g;
      denom = s0 - s1 * s1 + a.c[2];
    }
    const float inc = g * sc.lr * rsqrtf(denom);
    if (a.flags & 1) {
      s1 = a.c[1] * s1 + inc;
      p -= s1;
    } else {
      p -= inc;
    }
  } else if (RULE == RULE_ADAGRAD) {  // c0 epsilon
    s0 += g * g;
    p -= sc.lr * g / sqrtf(s0 + a.c[0]);
  } else if (RULE == RULE_ADADELTA) {  // c0 rho, c1 epsilon
    s0 = a.c[0] * s0 + (1.f - a.c[0]) * g * g;
    const float delta = -sqrtf(s1 + a.c[1]) * g / sqrtf(s0 + a.c[1]);
    s1 = a.c[0] * s1 + (1.f - a.c[0]) * delta * delta;
    p += sc.lr * delta;
  } else if (RULE == RULE_ADAMAX) {  // c0 beta_1, c1 beta_2, c2 epsilon; k0 = 1 - beta_1^t
    s0 += (g - s0) * (1.f - a.c[0]);
    s1 = fmaxf(a.c[1] * s1, fabsf(g));
    p -= (sc.lr * s0) / (sc.k0 * (s1 + a.c[2]));
  } else if (RULE == RULE_NADAM) {  // c0 beta_1, c1 beta_2, c2 epsilon; k0 u_t, k1 u_{t+1}, k2 u_product_t, k3 1 - beta_2^t
    s0 += (g - s0) * (1.f - a.c[0]);
    s1 += (g * g - s1) * (1.f - a.c[1]);
    const float m_hat = (sc.k1 * s0) / (1.f - sc.k2 * sc.k1) + ((1.f - sc.k0) * g) / (1.f - sc.k2);
    const float v_hat = s1 / sc.k3;
    p -= (m_hat * sc.lr) / (sqrtf(v_hat) + a.c[2]);
  } else {  // Lion: c0 beta_1, c1 beta_2
    const float dir = s0 * a.c[0] + g * (1.f - a.c[0]);
    p -= sc.lr * (dir > 0.f ? 1.f : (dir < 0.f ? -1.f : 0.f));
    s0 = a.c[1] * s0 + (1.f - a.c[1]) * g;
  }
}

template <int RULE>
__global__ void __launch_bounds__(KB_OPT_THREADS) rule_kernel(const KbTensorDesc* __restrict__ descs, const KbChunk* __restrict__ chunks, RuleArgs a,
                                                              int* __restrict__ found_inf) {
  const RuleScalars sc = rule_scalars<RULE>(a);
  const KbChunk c = chunks[blockIdx.x];
  const KbTensorDesc d = descs[c.tensor];
  const float decay = decay_factor(d.decay, sc.lr);
  const long long end = min(d.numel, c.start + (long long)KB_OPT_CHUNK);
  const bool has1 = d.slot1 != nullptr;
  const bool vec = ((((uintptr_t)d.param | (uintptr_t)d.grad | (uintptr_t)d.slot0 | (uintptr_t)d.slot1) & 15) == 0) && ((c.start & 3) == 0) &&
                   (d.shadow == nullptr || (((uintptr_t)d.shadow & 7) == 0));
  bool bad = false;
  long long scalar_from = c.start;
  if (vec) {
    for (long long i = c.start + threadIdx.x * 4ll; i + 3 < end; i += KB_OPT_THREADS * 4ll) {
      float4 p = *reinterpret_cast<float4*>(d.param + i);
      float4 g = *reinterpret_cast<const float4*>(d.grad + i);
      float4 s0 = *reinterpret_cast<float4*>(d.slot0 + i);
      float4 s1 = has1 ? *reinterpret_cast<float4*>(d.slot1 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      g.x *= a.grad_scale; g.y *= a.grad_scale; g.z *= a.grad_scale; g.w *= a.grad_scale;
      bad |= !(isfinite(g.x) && isfinite(g.y) && isfinite(g.z) && isfinite(g.w));
      rule_elem<RULE>(p.x, g.x, s0.x, s1.x, a, sc, decay);
      rule_elem<RULE>(p.y, g.y, s0.y, s1.y, a, sc, decay);
      rule_elem<RULE>(p.z, g.z, s0.z, s1.z, a, sc, decay);
      rule_elem<RULE>(p.w, g.w, s0.w, s1.w, a, sc, decay);
      *reinterpret_cast<float4*>(d.param + i) = p;
      *reinterpret_cast<float4*>(d.slot0 + i) = s0;
      if (has1) *reinterpret_cast<float4*>(d.slot1 + i) = s1;
      if (a.zero_grad) *reinterpret_cast<float4*>(d.grad + i) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d.shadow) {
        *reinterpret_cast<__nv_bfloat162*>(d.shadow + i) = __floats2bfloat162_rn(p.x, p.y);
        *reinterpret_cast<__nv_bfloat162*>(d.shadow + i + 2) = __floats2bfloat162_rn(p.z, p.w);
      }
    }
    scalar_from = c.start + ((end - c.start) & ~3ll);
  }
  for (long long i = scalar_from + threadIdx.x; i < end; i += KB_OPT_THREADS) {
    float p = d.param[i], g = d.grad[i] * a.grad_scale, s0 = d.slot0[i], s1 = has1 ? d.slot1[i] : 0.f;
    bad |= !isfinite(g);
    rule_elem<RULE>(p, g, s0, s1, a, sc, decay);
    d.param[i] = p;
    d.slot0[i] = s0;
    if (has1) d.slot1[i] = s1;
    if (a.zero_grad) d.grad[i] = 0.f;
    if (d.shadow) d.shadow[i] = __float2bfloat16_rn(p);
  }
  if (found_inf != nullptr && bad) atomicOr(found_inf, 1);
}

// Nadam's per-step scalars from the device-resident iteration counter; multiplies u_product by u_t as the host path does
// before its update (keras/src/optimizers/nadam.py:100-108).  out = {u_t, u_{t+1}, u_product_t, 1 - beta_2^t}.
__global__ void nadam_prepare_kernel(const int* __restrict__ step_ptr, double b1, double b2, float* __restrict__ u_product, float* __restrict__ out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const double t = (double)(*step_ptr) + 1.0;
  const double u_t = b1 * (1.0 - 0.5 * pow(0.96, t));
  const double u_t1 = b1 * (1.0 - 0.5 * pow(0.96, t + 1.0));
  const float prod = (float)((double)(*u_product) * u_t);
  *u_product = prod;
  out[0] = (float)u_t;
  out[1] = (float)u_t1;
  out[2] = prod;
  out[3] = (float)(1.0 - pow(b2, t));
}

// rule: KbRule.  c[4]: rule constants; k[4]: step-dependent scalars by value (used when step_ptr is null).
// Nadam with step_ptr: `u_product` (device float) is advanced and `scratch` (4 device floats) receives the step scalars.
KB_API int kb200_fused_rule(const void* descs, const void* chunks, int n_chunks, int rule, float lr, const float* c, const float* k, double beta1,
                            double beta2, int flags, float grad_scale, int zero_grad, int* found_inf, const float* lr_ptr, const int* step_ptr,
                            float* u_product, float* scratch, cudaStream_t stream) {
  if (n_chunks <= 0) return 0;
  RuleArgs a{};
  a.lr = lr;
  a.grad_scale = grad_scale;
  for (int i = 0; i < 4; ++i) {
    a.c[i] = c[i];
    a.k[i] = k[i];
  }
  a.b1 = beta1;
  a.b2 = beta2;
  a.lr_ptr = lr_ptr;
  a.step_ptr = step_ptr;
  a.aux = nullptr;
  a.flags = flags;
  a.zero_grad = zero_grad;
  const KbTensorDesc* d = (const KbTensorDesc*)descs;
  const KbChunk* ch = (const KbChunk*)chunks;
  switch (rule) {
    case RULE_RMSPROP: rule_kernel<RULE_RMSPROP><<<n_chunks, KB_OPT_THREADS, 0, stream>>>(d, ch, a, found_inf); break;
    case RULE_ADAGRAD: rule_kernel<RULE_ADAGRAD><<<n_chunks, KB_OPT_THREADS, 0, stream>>>(d, ch, a, found_inf); break;
    case RULE_ADADELTA: rule_kernel<RULE_ADADELTA><<<n_chunks, KB_OPT_THREADS, 0, stream>>>(d, ch, a, found_inf); break;
    case RULE_ADAMAX: rule_kernel<RULE_ADAMAX><<<n_chunks, KB_OPT_THREADS, 0, stream>>>(d, ch, a, found_inf); break;
    case RULE_NADAM:
      if (step_ptr != nullptr) {
        if (u_product == nullptr || scratch == nullptr) {
          kb200_set_error("fused_rule: Nadam with a device step counter needs u_product and scratch");
          return -2;
        }
        nadam_prepare_kernel<<<1, 32, 0, stream>>>(step_ptr, beta1, beta2, u_product, scratch);
        a.aux = scratch;
      }
      rule_kernel<RULE_NADAM><<<n_chunks, KB_OPT_THREADS, 0, stream>>>(d, ch, a, found_inf);
      break;
    case RULE_LION: rule_kernel<RULE_LION><<<n_chunks, KB_OPT_THREADS, 0, stream>>>(d, ch, a, found_inf); break;
    default:
      kb200_set_error("fused_rule: unknown rule");
      return -2;
  }
  KB_CHECK_LAUNCH("fused_rule");
  return 0;
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
