// Allocation-free BatchNorm backward: see bn_static.h for the contract.
#include "bn_static.h"

#include <mutex>

#include "common.cuh"

// Existing launchers (bn.cu); they take the temporaries as pointers and allocate nothing themselves.
extern "C" int kb200_bn_bwd_reduce(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, long long M, int C,
                                   int dtype, float* sums, cudaStream_t stream);
extern "C" int kb200_bn_bwd_apply(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, const float* gamma,
                                  const float* sums, float* coef, void* dx, void* dres, long long M, int C, int dtype, cudaStream_t stream);

// [0, 2C): per-channel sums (must be zero when the reduction starts); [2C, 5C): dx coefficients.
static __device__ __align__(256) float g_bn_static_scratch[5 * KB200_BN_STATIC_MAX_C];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mu;

int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { kb200_set_error(cudaGetErrorString(e)); return -1; }
  if (dev < 0 || dev >= kMaxDevices) { kb200_set_error("bn_bwd_static: device ordinal out of range"); return -1; }
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_bn_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      kb200_set_error(e != cudaSuccess ? cudaGetErrorString(e) : "bn_bwd_static: null scratch address");
      return -1;
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

KB_API int kb200_bn_bwd_static_max_channels(void) { return KB200_BN_STATIC_MAX_C; }

KB_API int kb200_bn_bwd_static_setup(void) {
  float* p = nullptr;
  return scratch_for_current_device(&p);
}

KB_API int kb200_bn_bwd_static(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, const float* gamma, void* dx,
                               void* dres, float* dgamma, float* dbeta, long long M, int C, int dtype, cudaStream_t stream) {
  if (C <= 0 || M <= 0) { kb200_set_error("bn_bwd_static: empty input"); return -2; }
  if (C > KB200_BN_STATIC_MAX_C) {
    kb200_set_error("bn_bwd_static: C exceeds KB200_BN_STATIC_MAX_C (4096); use kb200_bn_bwd_reduce/kb200_bn_bwd_apply with caller scratch");
    return -3;
  }
  if (C % (dtype == 1 ? 8 : 4) != 0) { kb200_set_error("bn: C must be a multiple of the vector width"); return -2; }
  float* scratch = nullptr;
  if (scratch_for_current_device(&scratch) != 0) return -1;
  float* sums = scratch;
  float* coef = scratch + 2 * (size_t)C;
  int rc = kb200_bn_bwd_reduce(dy, x, y, mean, invstd, M, C, dtype, sums, stream);  // clears sums[0:2C] on `stream` first
  if (rc != 0) return rc;
  rc = kb200_bn_bwd_apply(dy, x, y, mean, invstd, gamma, sums, coef, dx, dres, M, C, dtype, stream);
  if (rc != 0) return rc;
  cudaError_t e = cudaSuccess;
  if (dbeta != nullptr) e = cudaMemcpyAsync(dbeta, sums, sizeof(float) * C, cudaMemcpyDeviceToDevice, stream);
  if (e == cudaSuccess && dgamma != nullptr) e = cudaMemcpyAsync(dgamma, sums + C, sizeof(float) * C, cudaMemcpyDeviceToDevice, stream);
  if (e != cudaSuccess) { kb200_set_error(cudaGetErrorString(e)); return -1; }
  return 0;
}
