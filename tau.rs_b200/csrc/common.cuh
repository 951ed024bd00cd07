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

TAU_EXPORT const char* tau_error_string(int code);
