// Shared by every kernel file: dtype conversion, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TAU_EXPORT extern "C" __attribute__((visibility("default")))

// Dtype codes shared with the Python side.
enum TauDType : int { TAU_F32 = 0, TAU_BF16 = 1 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float value) { return value; }
__device__ __forceinline__ float to_float(bf16 value) { return __bfloat162float(value); }

template <typename T> __device__ __forceinline__ T from_float(float value);
template <> __device__ __forceinline__ float from_float<float>(float value) { return value; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float value) { return __float2bfloat16_rn(value); }

// Rounds to the storage type and widens again: the value that a store followed by a load would give.
template <typename T> __device__ __forceinline__ float round_through(float value) {
    return to_float(from_float<T>(value));
}

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
    return value;
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
    return value;
}

// Sum over a block of up to 1024 threads; every thread receives the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float value, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    value = warp_sum(value);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = value;
    __syncthreads();
    if (warp == 0) {
        float partial = lane < warps ? scratch[lane] : 0.0f;
        partial = warp_sum(partial);
        if (lane == 0) scratch[32] = partial;
    }
    __syncthreads();
    return scratch[32];
}

static inline int tau_launch_status() { return static_cast<int>(cudaGetLastError()); }

// Programmatic dependent launch.  Every kernel of this library starts with `grid_dependents_launch()` (the next
// kernel in the stream may be scheduled as soon as all blocks of this one have started) and calls
// `grid_dependency_wait()` before it reads anything an earlier kernel wrote or writes anything at all (the wait
// returns when the previous kernel has completed and its writes are visible).  What a kernel does before the
// wait therefore overlaps the previous kernel's tail: in the products, that is the prefetch of the weights.
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#include <cstdlib>
#include <utility>

static inline bool tau_dependent_launch_enabled() {
    static const bool enabled = std::getenv("TAU_NO_DEPENDENT_LAUNCH") == nullptr;
    return enabled;
}

// Launches `kernel`; with `dependent` it may begin before the previous kernel of the stream has finished.
template <typename... Parameters, typename... Arguments>
static inline int tau_launch_as(bool dependent, void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                                Arguments&&... arguments) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = (dependent && tau_dependent_launch_enabled()) ? 1 : 0;
    return static_cast<int>(cudaLaunchKernelEx(&config, kernel, Parameters(std::forward<Arguments>(arguments))...));
}

// The same with thread-block clusters of `cluster` blocks along x (the grid's x must be a multiple of it).
template <typename... Parameters, typename... Arguments>
static inline int tau_launch_clusters_as(bool dependent, unsigned cluster, void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes,
                                         cudaStream_t stream, Arguments&&... arguments) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = (dependent && tau_dependent_launch_enabled()) ? 2 : 1;
    return static_cast<int>(cudaLaunchKernelEx(&config, kernel, Parameters(std::forward<Arguments>(arguments))...));
}

template <typename... Parameters, typename... Arguments>
static inline int tau_launch_clusters(unsigned cluster, void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes,
                                      cudaStream_t stream, Arguments&&... arguments) {
    return tau_launch_clusters_as(true, cluster, kernel, grid, block, shared_bytes, stream, std::forward<Arguments>(arguments)...);
}

// Launches `kernel` so that it may begin before the previous kernel of the stream has finished.
template <typename... Parameters, typename... Arguments>
static inline int tau_launch(void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                             Arguments&&... arguments) {
    return tau_launch_as(true, kernel, grid, block, shared_bytes, stream, std::forward<Arguments>(arguments)...);
}

TAU_EXPORT const char* tau_error_string(int code);
