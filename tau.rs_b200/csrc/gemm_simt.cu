// Plain tiled matrix product on the ordinary 32-bit pipes: out[M, N] = x[M, K] * w[N, K]^T + bias.
//
// This is the true 32-bit product (fused multiply-add in float, no tensor cores, no reduced-precision
// mode) and the fallback for bfloat16 shapes that the tensor-core kernels refuse.  The weight is the
// checkpoint's `[out, in]` matrix used as it lies (crates/cuda-kernels/src/kernels/
// linear_bf16_fp32.cuh:31-33).  Any M, N, K.
#include "common.cuh"

namespace {

constexpr int kTile = 64;     // output tile is kTile x kTile
constexpr int kDepth = 16;    // K elements per stage
constexpr int kThreads = 256; // each thread owns a 4 x 4 patch

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kThreads)
gemm_simt_kernel(const TIn* __restrict__ x, const TIn* __restrict__ w, const float* __restrict__ bias,
                 TOut* __restrict__ out, int M, int N, int K, long long x_stride, long long w_stride,
                 long long out_stride) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ float xs[kDepth][kTile + 4];
    __shared__ float ws[kDepth][kTile + 4];
    const int row0 = blockIdx.y * kTile, col0 = blockIdx.x * kTile;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    // Loading: thread t brings element (t / 16 + 16 * i, t % 16) of each 64 x 16 tile, i = 0..3.
    const int load_k = threadIdx.x % kDepth, load_r = threadIdx.x / kDepth;
    for (int k0 = 0; k0 < K; k0 += kDepth) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = load_r + 16 * i;
            const int k = k0 + load_k;
            const int xr = row0 + r, wr = col0 + r;
            xs[load_k][r] = (xr < M && k < K) ? to_float(x[xr * x_stride + k]) : 0.0f;
            ws[load_k][r] = (wr < N && k < K) ? to_float(w[wr * w_stride + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kDepth; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx * 4 + j;
            if (c >= N) continue;
            const float value = acc[i][j] + (bias ? bias[c] : 0.0f);
            out[r * out_stride + c] = from_float<TOut>(value);
        }
    }
}

template <typename TIn, typename TOut>
int launch(const void* x, const void* w, const float* bias, void* out, int M, int N, int K, long long x_stride,
           long long w_stride, long long out_stride, cudaStream_t stream) {
    dim3 grid((N + kTile - 1) / kTile, (M + kTile - 1) / kTile);
    tau_launch(gemm_simt_kernel<TIn, TOut>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const TIn*>(x), static_cast<const TIn*>(w), bias,
                                                              static_cast<TOut*>(out), M, N, K, x_stride, w_stride, out_stride);
    return tau_launch_status();
}

}  // namespace

// Strides are in elements between consecutive rows.  `out_dtype` may be float32 for a bfloat16 product (logits).
TAU_EXPORT int tau_gemm_simt(int in_dtype, int out_dtype, const void* x, const void* w, const float* bias, void* out, int M,
                             int N, int K, long long x_stride, long long w_stride, long long out_stride, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!x || !w || !out || K <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_dtype == TAU_F32 && out_dtype == TAU_F32) return launch<float, float>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    if (in_dtype == TAU_BF16 && out_dtype == TAU_BF16) return launch<bf16, bf16>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    if (in_dtype == TAU_BF16 && out_dtype == TAU_F32) return launch<bf16, float>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    return cudaErrorInvalidValue;
}
