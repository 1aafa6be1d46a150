// Shared helpers of the sm_100a kernels: element types, conversions, reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

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

// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation attribute may
// start while the kernel before it on the stream still runs; whatever it does before
// `wait_for_previous_kernel()` must not depend on (or disturb) that kernel's work.  It is used to pull
// weights, which no kernel writes, towards L2 early.  `allow_next_kernel()` lets the kernel after this one
// start early in turn; it does nothing if that kernel was launched the ordinary way.
__device__ __forceinline__ void allow_next_kernel() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_previous_kernel() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void prefetch_to_l2(const void* address) { asm volatile("prefetch.global.L2 [%0];" ::"l"(address)); }

__device__ __forceinline__ void report_error(int* status, int code) {
    if (status != nullptr) atomicCAS(status, 0, code);
}

// Launches `kernel` with the programmatic-serialisation attribute (see wait_for_previous_kernel): only
// for kernels that call wait_for_previous_kernel() before they touch anything another kernel produces.
// LALAMO_B200_OVERLAP_LAUNCH=0 in the environment launches the ordinary way.
inline bool overlap_launches() {
    static const bool overlap = []() {
        const char* setting = getenv("LALAMO_B200_OVERLAP_LAUNCH");
        return setting == nullptr || setting[0] != '0';
    }();
    return overlap;
}

template <typename... Parameters, typename... Arguments>
inline cudaError_t launch_overlapped(void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                                     Arguments&&... arguments) {
    const bool overlap = overlap_launches();
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = overlap ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Parameters>(arguments)...);
}

// Something a launcher must do once on every device before its first launch there (a kernel's
// attributes belong to the device's copy of the kernel): `run(f)` calls `f` under a lock the first
// time the current device is seen and remembers the device once `f` has returned cudaSuccess.
class OncePerDevice {
   public:
    template <typename Setup>
    cudaError_t run(Setup&& setup) {
        int device = 0;
        const cudaError_t error = cudaGetDevice(&device);
        if (error != cudaSuccess) return error;
        if (device < 0 || device >= kDevices) return setup();   // beyond the table: every time
        if (done_[device].load(std::memory_order_acquire)) return cudaSuccess;
        std::lock_guard<std::mutex> guard(mutex_);
        if (done_[device].load(std::memory_order_relaxed)) return cudaSuccess;
        const cudaError_t result = setup();
        if (result == cudaSuccess) done_[device].store(true, std::memory_order_release);
        return result;
    }

   private:
    static constexpr int kDevices = 64;
    std::atomic<bool> done_[kDevices] = {};
    std::mutex mutex_;
};

// Raises a kernel's dynamic shared memory limit, once per device.
template <typename Kernel>
inline cudaError_t allow_shared_memory(OncePerDevice& once, Kernel kernel, int bytes) {
    return once.run([&]() { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); });
}

// Multiprocessors of the current device (asked once per device).
inline int multiprocessor_count() {
    constexpr int kDevices = 64;
    static std::atomic<int> counts[kDevices] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDevices) return 1;
    int count = counts[device].load(std::memory_order_relaxed);
    if (count == 0) {
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 1) count = 1;
        counts[device].store(count, std::memory_order_relaxed);
    }
    return count;
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
