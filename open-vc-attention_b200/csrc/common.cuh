// Shared helpers for the libovc.so translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ovc.h"

namespace ovc {

// Last CUDA error code seen by a failing entry point (per host thread).
void set_last_cuda_error(int code);

inline int check_launch() {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        set_last_cuda_error(static_cast<int>(err));
        return OVC_ERR_CUDA;
    }
    return OVC_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kTile = 128;  // tokens per quantisation block and per key tile
constexpr int kDim = 128;   // head dimension

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

#ifdef __CUDACC__
// a / b as the reference's Triton kernels compute it on a GPU: div.full.f32, the dividend times the
// hardware's approximate reciprocal of b, rounded once (not the IEEE quotient).
__device__ __forceinline__ float div_full(float a, float b) {
    float q;
    asm("div.full.f32 %0, %1, %2;" : "=f"(q) : "f"(a), "f"(b));
    return q;
}
#endif

}  // namespace ovc
