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
    grid_dependents_launch();
    grid_dependency_wait();
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
    grid_dependents_launch();
    grid_dependency_wait();
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
    grid_dependents_launch();
    grid_dependency_wait();
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


// ---- vectorised forms: 16-byte loads, the row kept in registers between the reduction and the scaling ---------
template <typename T> struct Vec16;
template <> struct Vec16<bf16> { static constexpr int n = 8; };
template <> struct Vec16<float> { static constexpr int n = 4; };

template <typename T> __device__ __forceinline__ void unpack16(const uint4& raw, float (&out)[Vec16<T>::n]);
template <> __device__ __forceinline__ void unpack16<bf16>(const uint4& raw, float (&out)[8]) {
    const unsigned words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(words[i] << 16);
        out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
}
template <> __device__ __forceinline__ void unpack16<float>(const uint4& raw, float (&out)[4]) {
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y); out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
}
template <typename T> __device__ __forceinline__ uint4 pack16(const float (&in)[Vec16<T>::n]);
template <> __device__ __forceinline__ uint4 pack16<bf16>(const float (&in)[8]) {
    unsigned words[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 pair = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
        words[i] = *reinterpret_cast<const unsigned*>(&pair);
    }
    return make_uint4(words[0], words[1], words[2], words[3]);
}
template <> __device__ __forceinline__ uint4 pack16<float>(const float (&in)[4]) {
    return make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]), __float_as_uint(in[3]));
}

// One block per output row, ITEMS vectors per thread (width <= threads * ITEMS * n, width % n == 0).
// MODE 0: out = norm(x[row]); MODE 1: out = norm(round(x[row] + branch[row])), x unchanged;
// MODE 2: x[row] = round(x[row] + branch[row]) in place, out = norm(x[row]).
template <typename T, int ITEMS, int MODE>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_vec_kernel(T* __restrict__ values, const T* __restrict__ branch, const int* __restrict__ rows, const float* __restrict__ weight,
                    T* __restrict__ out, int width, float eps) {
    grid_dependents_launch();
    constexpr int n = Vec16<T>::n;
    __shared__ float scratch[33];
    // The norm's weight is a parameter of the model and the row numbers came with the step, before its first kernel: both are
    // read while the kernel before this one is still at work, so that nothing but the rows themselves is waited for afterwards.
    const int source_row = rows ? rows[blockIdx.x] : blockIdx.x;
    float w[ITEMS][n];
#pragma unroll
    for (int item = 0; item < ITEMS; ++item) {
        const int column = (item * kNormThreads + threadIdx.x) * n;
        if (column < width) {
#pragma unroll
            for (int i = 0; i < n; i += 4) {
                const float4 part = *reinterpret_cast<const float4*>(weight + column + i);
                w[item][i] = part.x; w[item][i + 1] = part.y; w[item][i + 2] = part.z; w[item][i + 3] = part.w;
            }
        }
    }
    grid_dependency_wait();
    const size_t base = static_cast<size_t>(source_row) * width;
    float kept[ITEMS][n];
    float squares = 0.0f;
#pragma unroll
    for (int item = 0; item < ITEMS; ++item) {
        const int column = (item * kNormThreads + threadIdx.x) * n;
        if (column < width) {
            unpack16<T>(*reinterpret_cast<const uint4*>(values + base + column), kept[item]);
            if (MODE != 0) {
                float extra[n];
                unpack16<T>(*reinterpret_cast<const uint4*>(branch + base + column), extra);
#pragma unroll
                for (int i = 0; i < n; ++i) kept[item][i] = round_through<T>(kept[item][i] + extra[i]);
                if (MODE == 2) *reinterpret_cast<uint4*>(values + base + column) = pack16<T>(kept[item]);
            }
#pragma unroll
            for (int i = 0; i < n; ++i) squares += kept[item][i] * kept[item][i];
        }
    }
    const float inverse = rsqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    T* target = out + static_cast<size_t>(blockIdx.x) * width;
#pragma unroll
    for (int item = 0; item < ITEMS; ++item) {
        const int column = (item * kNormThreads + threadIdx.x) * n;
        if (column < width) {
            float scaled[n];
#pragma unroll
            for (int i = 0; i < n; ++i) scaled[i] = kept[item][i] * inverse * w[item][i];
            *reinterpret_cast<uint4*>(target + column) = pack16<T>(scaled);
        }
    }
}

template <typename T, int MODE>
bool launch_norm_vec(T* values, const T* branch, const int* rows, const float* weight, T* out, int out_rows, int width, float eps,
                     cudaStream_t stream) {
    constexpr int n = Vec16<T>::n;
    if (width % n != 0) return false;
    const int items = (width + kNormThreads * n - 1) / (kNormThreads * n);
    switch (items) {
        case 1: tau_launch(rms_norm_vec_kernel<T, 1, MODE>, dim3(out_rows), dim3(kNormThreads), 0, stream, values, branch, rows, weight, out, width, eps); return true;
        case 2: tau_launch(rms_norm_vec_kernel<T, 2, MODE>, dim3(out_rows), dim3(kNormThreads), 0, stream, values, branch, rows, weight, out, width, eps); return true;
        case 3: tau_launch(rms_norm_vec_kernel<T, 3, MODE>, dim3(out_rows), dim3(kNormThreads), 0, stream, values, branch, rows, weight, out, width, eps); return true;
        case 4: tau_launch(rms_norm_vec_kernel<T, 4, MODE>, dim3(out_rows), dim3(kNormThreads), 0, stream, values, branch, rows, weight, out, width, eps); return true;
        default: return false;
    }
}

// 16 bytes of gate and of up per thread.
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ stacked, T* __restrict__ out, size_t rows, int width) {
    grid_dependents_launch();
    grid_dependency_wait();
    constexpr int n = Vec16<T>::n;
    const int vectors_per_row = width / n;
    const size_t total = rows * static_cast<size_t>(vectors_per_row);
    for (size_t index = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; index < total;
         index += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = index / vectors_per_row;
        const int column = static_cast<int>(index - row * vectors_per_row) * n;
        float gate[n], up[n], result[n];
        unpack16<T>(*reinterpret_cast<const uint4*>(stacked + row * 2 * width + column), gate);
        unpack16<T>(*reinterpret_cast<const uint4*>(stacked + row * 2 * width + width + column), up);
#pragma unroll
        for (int i = 0; i < n; ++i) result[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
        *reinterpret_cast<uint4*>(out + row * width + column) = pack16<T>(result);
    }
}

// out[r, c] = silu(in[r, c]) * in[r, width + c]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ stacked, T* __restrict__ out, size_t rows, int width) {
    grid_dependents_launch();
    grid_dependency_wait();
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
        tau_launch(embedding_kernel<float>, dim3(rows), dim3(256), 0, s, tokens, static_cast<const float*>(table), static_cast<float*>(out), width, vocab);
    else if (dtype == TAU_BF16)
        tau_launch(embedding_kernel<bf16>, dim3(rows), dim3(256), 0, s, tokens, static_cast<const bf16*>(table), static_cast<bf16*>(out), width, vocab);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_rms_norm(int dtype, const void* values, const void* branch, const int* rows, const float* weight,
                            void* out, int out_rows, int width, float eps, void* stream) {
    if (out_rows <= 0) return 0;
    if (!values || !weight || !out || width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32 && (branch ? launch_norm_vec<float, 1>(const_cast<float*>(static_cast<const float*>(values)), static_cast<const float*>(branch), rows, weight, static_cast<float*>(out), out_rows, width, eps, s)
                                    : launch_norm_vec<float, 0>(const_cast<float*>(static_cast<const float*>(values)), nullptr, rows, weight, static_cast<float*>(out), out_rows, width, eps, s)))
        return tau_launch_status();
    if (dtype == TAU_BF16 && (branch ? launch_norm_vec<bf16, 1>(const_cast<bf16*>(static_cast<const bf16*>(values)), static_cast<const bf16*>(branch), rows, weight, static_cast<bf16*>(out), out_rows, width, eps, s)
                                     : launch_norm_vec<bf16, 0>(const_cast<bf16*>(static_cast<const bf16*>(values)), nullptr, rows, weight, static_cast<bf16*>(out), out_rows, width, eps, s)))
        return tau_launch_status();
    if (dtype == TAU_F32)
        tau_launch(rms_norm_kernel<float>, dim3(out_rows), dim3(kNormThreads), 0, s, static_cast<const float*>(values), static_cast<const float*>(branch),
                                                                rows, weight, static_cast<float*>(out), width, eps);
    else if (dtype == TAU_BF16)
        tau_launch(rms_norm_kernel<bf16>, dim3(out_rows), dim3(kNormThreads), 0, s, static_cast<const bf16*>(values), static_cast<const bf16*>(branch),
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
    if (dtype == TAU_F32 && launch_norm_vec<float, 2>(static_cast<float*>(residual), static_cast<const float*>(branch), nullptr, weight, static_cast<float*>(out), rows, width, eps, s))
        return tau_launch_status();
    if (dtype == TAU_BF16 && launch_norm_vec<bf16, 2>(static_cast<bf16*>(residual), static_cast<const bf16*>(branch), nullptr, weight, static_cast<bf16*>(out), rows, width, eps, s))
        return tau_launch_status();
    if (dtype == TAU_F32)
        tau_launch(add_rms_norm_kernel<float>, dim3(rows), dim3(kNormThreads), 0, s, static_cast<const float*>(branch), static_cast<float*>(residual),
                                                                weight, static_cast<float*>(out), width, eps);
    else if (dtype == TAU_BF16)
        tau_launch(add_rms_norm_kernel<bf16>, dim3(rows), dim3(kNormThreads), 0, s, static_cast<const bf16*>(branch), static_cast<bf16*>(residual),
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
    if (dtype == TAU_F32 && width % 4 == 0) {
        tau_launch(silu_mul_vec_kernel<float>, dim3(blocks), dim3(256), 0, s, static_cast<const float*>(stacked), static_cast<float*>(out), rows, width);
        return tau_launch_status();
    }
    if (dtype == TAU_BF16 && width % 8 == 0) {
        tau_launch(silu_mul_vec_kernel<bf16>, dim3(blocks), dim3(256), 0, s, static_cast<const bf16*>(stacked), static_cast<bf16*>(out), rows, width);
        return tau_launch_status();
    }
    if (dtype == TAU_F32)
        tau_launch(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, static_cast<const float*>(stacked), static_cast<float*>(out), rows, width);
    else if (dtype == TAU_BF16)
        tau_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s, static_cast<const bf16*>(stacked), static_cast<bf16*>(out), rows, width);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}
