// Weight-streaming product for a few rows of activations (decode): out[M, N] = x[M, K] * w[N, K]^T + bias, M <= 32.
//
// The reference runs these products through cuBLAS as m x 1 x k problems (crates/models/src/components/cuda/
// decode/operation.rs:150-193).  Here the step is bound by reading `w` once from HBM, so the kernel is shaped
// around that stream: a block owns 16 consecutive output features, its 8 warps split K in interleaved chunks of
// 64 elements, every thread keeps several 16-byte weight loads in flight, and the few activation rows are
// re-read from L1/L2.  The arithmetic is mma.sync m16n8k16 (bfloat16 in, float accumulate) with the weight
// rows as the A operand and the activations as B; a thread's 16-byte load is used as the fragments of two
// consecutive MMAs, which permutes K inside a chunk identically for both operands and so leaves every dot
// product unchanged.  Partial sums of the 8 warps meet in shared memory.
//
// Needs K % 8 == 0, 16-byte aligned rows of x and w (row strides multiples of 8 elements); other shapes go
// to the plain tiled kernel.
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kRows = 16;       // output features per block
constexpr int kChunk = 64;      // K elements per warp iteration

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NB, typename TOut>
__global__ void __launch_bounds__(kWarps * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias, TOut* __restrict__ out,
                   int M, int N, int K, long long x_stride, long long w_stride, long long out_stride) {
    grid_dependents_launch();
    __shared__ float partial[kWarps][NB * 8][kRows + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * kRows;
    // The weights do not depend on the previous kernel: ask L2 for this block's rows, then wait for the activations.
    if (threadIdx.x < kRows && row0 + threadIdx.x < N) {
        const bf16* row = w + static_cast<size_t>(row0 + threadIdx.x) * w_stride;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row), "r"(static_cast<unsigned>(K) * 2u) : "memory");
    }
    grid_dependency_wait();
    // Rows beyond N are clamped for loading and dropped when storing.
    const bf16* w_lo = w + static_cast<size_t>(min(row0 + g, N - 1)) * w_stride;
    const bf16* w_hi = w + static_cast<size_t>(min(row0 + g + 8, N - 1)) * w_stride;
    const bf16* x_row[NB];
    bool x_live[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const int token = j * 8 + g;
        x_live[j] = token < M;
        x_row[j] = x + static_cast<size_t>(x_live[j] ? token : 0) * x_stride;
    }
    float acc[NB][4];
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 4
    for (int chunk = warp * kChunk; chunk < K; chunk += kWarps * kChunk) {
        const int k_first = chunk + t * 8, k_second = chunk + 32 + t * 8;
        const bool first_live = k_first < K, second_live = k_second < K;   // K % 8 == 0: a group of 8 is whole or absent
        const uint4 lo1 = first_live ? __ldcs(reinterpret_cast<const uint4*>(w_lo + k_first)) : zero;
        const uint4 hi1 = first_live ? __ldcs(reinterpret_cast<const uint4*>(w_hi + k_first)) : zero;
        const uint4 lo2 = second_live ? __ldcs(reinterpret_cast<const uint4*>(w_lo + k_second)) : zero;
        const uint4 hi2 = second_live ? __ldcs(reinterpret_cast<const uint4*>(w_hi + k_second)) : zero;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const uint4 x1 = (x_live[j] && first_live) ? __ldg(reinterpret_cast<const uint4*>(x_row[j] + k_first)) : zero;
            const uint4 x2 = (x_live[j] && second_live) ? __ldg(reinterpret_cast<const uint4*>(x_row[j] + k_second)) : zero;
            mma_bf16(acc[j], lo1.x, hi1.x, lo1.y, hi1.y, x1.x, x1.y);
            mma_bf16(acc[j], lo1.z, hi1.z, lo1.w, hi1.w, x1.z, x1.w);
            mma_bf16(acc[j], lo2.x, hi2.x, lo2.y, hi2.y, x2.x, x2.y);
            mma_bf16(acc[j], lo2.z, hi2.z, lo2.w, hi2.w, x2.z, x2.w);
        }
    }
    // acc[j] = {D[g][2t], D[g][2t+1], D[g+8][2t], D[g+8][2t+1]} with D[feature][token within block j].
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        partial[warp][j * 8 + 2 * t][g] = acc[j][0];
        partial[warp][j * 8 + 2 * t + 1][g] = acc[j][1];
        partial[warp][j * 8 + 2 * t][g + 8] = acc[j][2];
        partial[warp][j * 8 + 2 * t + 1][g + 8] = acc[j][3];
    }
    __syncthreads();
    for (int index = threadIdx.x; index < NB * 8 * kRows; index += kWarps * 32) {
        const int token = index / kRows, r = index % kRows;
        const int feature = row0 + r;
        if (token >= M || feature >= N) continue;
        float sum = 0.0f;
#pragma unroll
        for (int wi = 0; wi < kWarps; ++wi) sum += partial[wi][token][r];
        if (bias) sum += bias[feature];
        out[static_cast<size_t>(token) * out_stride + feature] = from_float<TOut>(sum);
    }
}

template <int NB>
int launch(int out_dtype, const void* x, const void* w, const float* bias, void* out, int M, int N, int K, long long x_stride,
           long long w_stride, long long out_stride, cudaStream_t stream) {
    const unsigned blocks = (N + kRows - 1) / kRows;
    if (out_dtype == TAU_BF16)
        tau_launch(gemm_skinny_kernel<NB, bf16>, dim3(blocks), dim3(kWarps * 32), 0, stream, static_cast<const bf16*>(x), static_cast<const bf16*>(w), bias,
                                                                        static_cast<bf16*>(out), M, N, K, x_stride, w_stride, out_stride);
    else
        tau_launch(gemm_skinny_kernel<NB, float>, dim3(blocks), dim3(kWarps * 32), 0, stream, static_cast<const bf16*>(x), static_cast<const bf16*>(w), bias,
                                                                         static_cast<float*>(out), M, N, K, x_stride, w_stride, out_stride);
    return tau_launch_status();
}

}  // namespace

TAU_EXPORT int tau_gemm_skinny_max_rows() { return 32; }

// bfloat16 inputs; `out_dtype` bfloat16 or float32.  Strides in elements.
TAU_EXPORT int tau_gemm_skinny(int out_dtype, const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                               long long x_stride, long long w_stride, long long out_stride, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!x || !w || !out || K <= 0 || M > 32 || (K & 7) || (x_stride & 7) || (w_stride & 7) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (out_dtype != TAU_BF16 && out_dtype != TAU_F32))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (M <= 8) return launch<1>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    if (M <= 16) return launch<2>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    return launch<4>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
}
