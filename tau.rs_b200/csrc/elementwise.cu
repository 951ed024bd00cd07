// Embedding rows, RMSNorm (plain and fused with the residual sum) and SiLU*mul, for float32 and bfloat16.
//
// Reference counterparts: crates/cuda-kernels/src/kernels/decode_attention.cu:25 (embedding row copy),
// centered_rms_norm.cu:75-115 and :267-308 (norm, and the fused form that rounds the residual sum to the
// storage type before normalising it), silu_and_mul.cu:51-76.  The norm here scales by `w`, not `1 + w`.
#include "common.cuh"

const char* tau_error_string(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }

namespace {

constexpr int kNormThreads = 256;

template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table, T* __restrict__ out,
                                 int width, int vocab) {
    const int row = blockIdx.x;
    const int token = tokens[row];
    T* target = out + static_cast<size_t>(row) * width;
    if (token < 0 || token >= vocab) {  // refused on the host already; never read outside the table
        for (int column = threadIdx.x; column < width; column += blockDim.x) target[column] = from_float<T>(0.0f);
        return;
    }
    const T* source = table + static_cast<size_t>(token) * width;
    for (int column = threadIdx.x; column < width; column += blockDim.x) target[column] = source[column];
}

// out[i] = norm(round(x[r] + branch[r])) * w with r = rows ? rows[i] : i; x is left unchanged.
template <typename T>
__global__ void rms_norm_kernel(const T* __restrict__ values, const T* __restrict__ branch, const int* __restrict__ rows,
                                const float* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    const int source_row = rows ? rows[blockIdx.x] : blockIdx.x;
    const T* source = values + static_cast<size_t>(source_row) * width;
    const T* extra = branch ? branch + static_cast<size_t>(source_row) * width : nullptr;
    float squares = 0.0f;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        float value = to_float(source[column]);
        if (extra) value = round_through<T>(value + to_float(extra[column]));
        squares += value * value;
    }
    const float inverse = rsqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    T* target = out + static_cast<size_t>(blockIdx.x) * width;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        float value = to_float(source[column]);
        if (extra) value = round_through<T>(value + to_float(extra[column]));
        target[column] = from_float<T>(value * inverse * weight[column]);
    }
}

// residual = round(residual + branch); out = norm(residual) * w.
template <typename T>
__global__ void add_rms_norm_kernel(const T* __restrict__ branch, T* __restrict__ residual,
                                    const float* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    const size_t base = static_cast<size_t>(blockIdx.x) * width;
    float squares = 0.0f;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        const T sum = from_float<T>(to_float(residual[base + column]) + to_float(branch[base + column]));
        residual[base + column] = sum;
        const float value = to_float(sum);
        squares += value * value;
    }
    const float inverse = rsqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    // Each thread reads back only what it wrote itself.
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        out[base + column] = from_float<T>(to_float(residual[base + column]) * inverse * weight[column]);
    }
}

// out[r, c] = silu(in[r, c]) * in[r, width + c]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ stacked, T* __restrict__ out, size_t rows, int width) {
    const size_t total = rows * static_cast<size_t>(width);
    for (size_t index = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; index < total;
         index += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = index / width;
        const int column = static_cast<int>(index - row * width);
        const float gate = to_float(stacked[row * 2 * width + column]);
        const float up = to_float(stacked[row * 2 * width + width + column]);
        out[index] = from_float<T>(gate / (1.0f + expf(-gate)) * up);
    }
}

}  // namespace

TAU_EXPORT int tau_embedding(int dtype, const int* tokens, const void* table, void* out, int rows, int width, int vocab,
                             void* stream) {
    if (rows <= 0) return 0;
    if (!tokens || !table || !out || width <= 0 || vocab <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32)
        embedding_kernel<float><<<rows, 256, 0, s>>>(tokens, static_cast<const float*>(table), static_cast<float*>(out), width, vocab);
    else if (dtype == TAU_BF16)
        embedding_kernel<bf16><<<rows, 256, 0, s>>>(tokens, static_cast<const bf16*>(table), static_cast<bf16*>(out), width, vocab);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_rms_norm(int dtype, const void* values, const void* branch, const int* rows, const float* weight,
                            void* out, int out_rows, int width, float eps, void* stream) {
    if (out_rows <= 0) return 0;
    if (!values || !weight || !out || width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32)
        rms_norm_kernel<float><<<out_rows, kNormThreads, 0, s>>>(static_cast<const float*>(values), static_cast<const float*>(branch),
                                                                rows, weight, static_cast<float*>(out), width, eps);
    else if (dtype == TAU_BF16)
        rms_norm_kernel<bf16><<<out_rows, kNormThreads, 0, s>>>(static_cast<const bf16*>(values), static_cast<const bf16*>(branch),
                                                               rows, weight, static_cast<bf16*>(out), width, eps);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_add_rms_norm(int dtype, const void* branch, void* residual, const float* weight, void* out, int rows,
                                int width, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (!branch || !residual || !weight || !out || width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32)
        add_rms_norm_kernel<float><<<rows, kNormThreads, 0, s>>>(static_cast<const float*>(branch), static_cast<float*>(residual),
                                                                weight, static_cast<float*>(out), width, eps);
    else if (dtype == TAU_BF16)
        add_rms_norm_kernel<bf16><<<rows, kNormThreads, 0, s>>>(static_cast<const bf16*>(branch), static_cast<bf16*>(residual),
                                                               weight, static_cast<bf16*>(out), width, eps);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_silu_mul(int dtype, const void* stacked, void* out, long long rows, int width, void* stream) {
    if (rows <= 0) return 0;
    if (!stacked || !out || width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long total = rows * width;
    const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
    if (dtype == TAU_F32)
        silu_mul_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(stacked), static_cast<float*>(out), rows, width);
    else if (dtype == TAU_BF16)
        silu_mul_kernel<bf16><<<blocks, 256, 0, s>>>(static_cast<const bf16*>(stacked), static_cast<bf16*>(out), rows, width);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}
