// Host-side helpers shared by the translation units of libdmlx_b200.
#pragma once
#include <cstdarg>
#include <cstdint>

#include "dmlx_b200.h"

// printf-style setter for the calling thread's last-error string.
void b200_set_error(const char* fmt, ...);

#ifdef __CUDACC__
#include <cuda_runtime.h>
#define B200_CUDA_TRY(expr)                                                                 \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) {                                                                \
      b200_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return B200_ERR_CUDA;                                                                 \
    }                                                                                       \
  } while (0)
// Every kernel launch of the library passes through B200_LAUNCH_CHECK, which also counts it.
extern long long g_b200_launch_counter;
#define B200_LAUNCH_CHECK()                                                                 \
  do {                                                                                      \
    ++g_b200_launch_counter;                                                                \
    cudaError_t _e = cudaGetLastError();                                                    \
    if (_e != cudaSuccess) {                                                                \
      b200_set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
      return B200_ERR_CUDA;                                                                 \
    }                                                                                       \
  } while (0)
// Returns B200_ERR_NO_DEVICE (with a message) unless a CUDA device is usable, and B200_ERR_UNSUPPORTED
// when the current device is not the one this process first used the library on.
b200_status b200_require_device();
// The same without binding the process to a device (entry points that keep per-device state).
b200_status b200_require_any_device();
#endif
