#include <string.h>

#include "common.cuh"

static thread_local char g_last_error[512] = {0};

void kb200_set_error(const char* msg) {
  strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
}

KB_API const char* kb200_last_error() { return g_last_error; }

KB_API int kb200_abi_version() { return 1; }

// Make `device`'s primary context current on the calling thread.  Launchers are reached through
// ctypes from arbitrary Python threads (e.g. the autograd engine's), which may not have touched
// the CUDA runtime yet; driver-API helpers such as tensor-map encoding need a current context.
KB_API int kb200_bind_device(int device) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) {
    kb200_set_error(cudaGetErrorString(e));
    return -1;
  }
  cudaFree(0);
  return 0;
}
