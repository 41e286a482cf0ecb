// Error / launch bookkeeping shared by the files that implement the C-ABI (l3_api.cu, layerlist.cu).
#pragma once
#include <cuda_runtime.h>

#include "model.h"

void set_err(L3Model* m, const char* fmt, ...);  // l3_api.cu
extern const bool g_l3_debug_sync;               // L3_DEBUG_SYNC=1: synchronise after every launch

#define CK(m, call)                                                                         \
  do {                                                                                      \
    cudaError_t e__ = (call);                                                               \
    if (e__ != cudaSuccess) {                                                               \
      set_err(m, "CUDA error %s at %s:%d: %s", cudaGetErrorName(e__), __FILE__, __LINE__,   \
              cudaGetErrorString(e__));                                                     \
      return L3_ECUDA;                                                                      \
    }                                                                                       \
  } while (0)
// a kernel launch: counted (gpu_launches in bench.py is this counter)
#define LAUNCH(m, call)                                                                        \
  do {                                                                                         \
    CK(m, call);                                                                               \
    (m)->launch_acc += 1;                                                                      \
    if (g_l3_debug_sync) { /* L3_DEBUG_SYNC=1: attribute an asynchronous fault to its launch */ \
      cudaError_t e2__ = cudaStreamSynchronize((m)->stream);                                   \
      if (e2__ != cudaSuccess) {                                                               \
        set_err(m, "kernel launched at %s:%d (launch #%lld) failed: %s", __FILE__, __LINE__,   \
                (long long)(m)->launch_acc, cudaGetErrorString(e2__));                         \
        return L3_ECUDA;                                                                       \
      }                                                                                        \
    }                                                                                          \
  } while (0)
#define REQUIRE(m, cond, ...)    \
  do {                           \
    if (!(cond)) {               \
      set_err(m, __VA_ARGS__);   \
      return L3_EINVAL;          \
    }                            \
  } while (0)
