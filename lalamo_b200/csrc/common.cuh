// Shared helpers of the sm_100a kernels: element types, conversions, reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {

// Element type codes shared with the Python bindings.
enum DType : int { kFloat32 = 0, kBFloat16 = 1 };

// Error codes written to the device-side status word (first error wins).
enum KernelError : int {
    kOk = 0,
    kBadPage = 1,       // a block-table entry outside the pool was about to be used
    kBadSlot = 2,       // a state slot outside the slot array
    kBadToken = 3,      // a token id outside the vocabulary
    kWaitTimeout = 4,   // a bounded wait on a barrier gave up
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Rounds a 32-bit value to the activation type and back: marks the places where the
// activation type limits precision (a no-op on the 32-bit path).
template <typename T>
__device__ __forceinline__ float round_to(float v) { return to_float(from_float<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Block-wide sum with a fixed reduction order (the result does not depend on what else runs).
// `scratch` holds at least 33 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < warps ? scratch[lane] : 0.0f;
        w = warp_sum(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < warps ? scratch[lane] : -INFINITY;
        w = warp_max(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ void report_error(int* status, int code) {
    if (status != nullptr) atomicCAS(status, 0, code);
}

}  // namespace lb

// Every launcher returns 0 or the CUDA error code of its launch.
#define LB_LAUNCH_RESULT() static_cast<int>(cudaGetLastError())

#define LB_DISPATCH_DTYPE(dtype, ...)                    \
    if ((dtype) == lb::kFloat32) {                       \
        using T = float;                                 \
        __VA_ARGS__                                      \
    } else if ((dtype) == lb::kBFloat16) {               \
        using T = __nv_bfloat16;                         \
        __VA_ARGS__                                      \
    } else {                                             \
        return -1;                                       \
    }
