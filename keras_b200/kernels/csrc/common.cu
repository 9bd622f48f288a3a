#include <string.h>

#include "common.cuh"

static thread_local char g_last_error[512] = {0};

void kb200_set_error(const char* msg) {
  strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
}

KB_API const char* kb200_last_error() { return g_last_error; }

KB_API int kb200_abi_version() { return 1; }
