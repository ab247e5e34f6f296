// Shared host-side helpers of the cagnet_b200 C ABI (error reporting, launch checks).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/cagnet_b200.h"

namespace cagnet {

// Last error text of the calling thread (returned by cagnet_last_error_string).
char* last_error_buf();

inline int fail(int code, const char* fmt, const char* a = "", long long b = 0, long long c = 0) {
  snprintf(last_error_buf(), 256, fmt, a, b, c);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(last_error_buf(), 256, "%s: CUDA launch failed: %s", what, cudaGetErrorString(e));
    return CAGNET_E_LAUNCH;
  }
  return CAGNET_OK;
}

__host__ __device__ inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

constexpr int kNumSMs = 148;  // B200

// k length of one tensor-core accumulation of the dense-core multiply (tuning knob "core_chunk")
int core_chunk();
int set_core_chunk(int value);
// the same for the integer-core multiply (tuning knob "core_chunk_int")
int core_chunk_int();
int set_core_chunk_int(int value);


}  // namespace cagnet
