// Attention over the paged cache, for every head size, head count and dtype: the prepare step (per-head
// q/k RMSNorm, rotation, cache write) and a plain attention kernel with an online softmax.
//
// Reference counterparts: crates/cuda-kernels/src/kernels/decode_attention.cu:120-181 (`attention_prepare`:
// one block per query or key head of one token: norm, rotate, write Q / append K and V) and :186-250
// (`attention`: 32-bit dot per key, `* rsqrt(d)`, max, exp, sum, probabilities times V).  Here a launch
// covers every token of a step, each with its own sequence, position and page list.
//
// Cache layout of one layer: keys[page][kv_head][slot_in_page][d], the same for values; position `p` of
// sequence `s` lies in page `page_rows[s * page_stride + p / page_tokens]` at `p % page_tokens`.
#include "common.cuh"

namespace {

constexpr int kMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void attention_prepare_kernel(
    const T* __restrict__ projected, long long projected_stride, T* __restrict__ queries, T* __restrict__ keys,
    T* __restrict__ values, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rotary_dim,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows,
    int page_stride, int page_tokens, int n_heads, int n_kv_heads, int head_dim, int write_cache) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int position = positions[token];
    const int heads_total = write_cache ? n_heads + 2 * n_kv_heads : n_heads;
    const T* row = projected + static_cast<size_t>(token) * projected_stride;
    const int half = rotary_dim / 2;
    size_t cache_base = 0;
    if (write_cache) {
        const int page = page_rows[static_cast<size_t>(token_seq[token]) * page_stride + position / page_tokens];
        cache_base = (static_cast<size_t>(page) * n_kv_heads * page_tokens + position % page_tokens) * head_dim;
    }
    for (int head = warp; head < heads_total; head += warps) {
        const T* source = row + static_cast<size_t>(head) * head_dim;
        T* target;
        const float* weight;
        bool rotate = true;
        if (head < n_heads) {
            target = queries + (static_cast<size_t>(token) * n_heads + head) * head_dim;
            weight = q_weight;
        } else {
            const int kv_head = (head - n_heads) % n_kv_heads;
            const bool is_key = head < n_heads + n_kv_heads;
            target = (is_key ? keys : values) + cache_base + static_cast<size_t>(kv_head) * page_tokens * head_dim;
            weight = is_key ? k_weight : nullptr;
            rotate = is_key;
            if (!is_key) {  // values are stored as projected
                for (int e = lane; e < head_dim; e += 32) target[e] = source[e];
                continue;
            }
        }
        float inverse = 1.0f;
        if (weight) {
            float squares = 0.0f;
            for (int e = lane; e < head_dim; e += 32) {
                const float value = to_float(source[e]);
                squares += value * value;
            }
            inverse = rsqrtf(warp_sum(squares) / static_cast<float>(head_dim) + eps);
        }
        // Normalised values are rounded to the storage type, rotated in 32-bit and rounded once more.
        auto normalized = [&](int e) {
            const float value = to_float(source[e]);
            return weight ? round_through<T>(value * inverse * weight[e]) : value;
        };
        if (rotate && half > 0) {
            const float* cos_row = cos_table + static_cast<size_t>(position) * half;
            const float* sin_row = sin_table + static_cast<size_t>(position) * half;
            for (int j = lane; j < half; j += 32) {
                const float first = normalized(j), second = normalized(j + half);
                const float c = cos_row[j], s = sin_row[j];
                target[j] = from_float<T>(first * c - second * s);
                target[j + half] = from_float<T>(second * c + first * s);
            }
            for (int e = rotary_dim + lane; e < head_dim; e += 32) target[e] = from_float<T>(normalized(e));
        } else {
            for (int e = lane; e < head_dim; e += 32) target[e] = from_float<T>(normalized(e));
        }
    }
}

// The same for head sizes of 32 * PER elements that are rotated whole (or not at all): a lane holds PER neighbouring
// elements, loaded and stored as one vector; the element it is paired with by the rotation lies in lane ^ 16.
template <typename T, int PER> struct alignas(sizeof(T) * PER) HeadVector { T v[PER]; };

template <typename T, int PER>
__global__ void attention_prepare_vec_kernel(
    const T* __restrict__ projected, long long projected_stride, T* __restrict__ queries, T* __restrict__ keys,
    T* __restrict__ values, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rotary_dim,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows,
    int page_stride, int page_tokens, int n_heads, int n_kv_heads, int write_cache) {
    grid_dependents_launch();
    grid_dependency_wait();
    constexpr int head_dim = 32 * PER;
    typedef HeadVector<T, PER> Vector;
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int position = positions[token];
    const int heads_total = write_cache ? n_heads + 2 * n_kv_heads : n_heads;
    const T* row = projected + static_cast<size_t>(token) * projected_stride;
    size_t cache_base = 0;
    if (write_cache) {
        const int page = page_rows[static_cast<size_t>(token_seq[token]) * page_stride + position / page_tokens];
        cache_base = (static_cast<size_t>(page) * n_kv_heads * page_tokens + position % page_tokens) * head_dim;
    }
    // This lane's rotation coefficients: elements PER * (lane % 16) + i of the half-width tables.
    float cosines[PER], sines[PER];
    if (rotary_dim) {
        const size_t table = static_cast<size_t>(position) * (head_dim / 2) + PER * (lane & 15);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            cosines[i] = cos_table[table + i];
            sines[i] = lane < 16 ? -sin_table[table + i] : sin_table[table + i];   // first half: x cos - partner sin; second half: x cos + partner sin
        }
    }
    // A warp takes the heads warp, warp + warps, ...; their vectors are asked for several at a time, so that the loads of
    // one token's heads travel together instead of one after another.
    constexpr int kBatch = 6;
    for (int first = warp; first < heads_total; first += warps * kBatch) {
        Vector loaded[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int head = first + b * warps;
            if (head < heads_total) loaded[b] = *reinterpret_cast<const Vector*>(row + static_cast<size_t>(head) * head_dim + PER * lane);
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int head = first + b * warps;
            if (head >= heads_total) break;
            T* target;
            const float* weight;
            if (head < n_heads) {
                target = queries + (static_cast<size_t>(token) * n_heads + head) * head_dim;
                weight = q_weight;
            } else {
                const bool is_key = head < n_heads + n_kv_heads;
                const int kv_head = head - n_heads - (is_key ? 0 : n_kv_heads);
                target = (is_key ? keys : values) + cache_base + static_cast<size_t>(kv_head) * page_tokens * head_dim;
                weight = k_weight;
                if (!is_key) {  // values are stored as projected
                    *reinterpret_cast<Vector*>(target + PER * lane) = loaded[b];
                    continue;
                }
            }
            float value[PER];
#pragma unroll
            for (int i = 0; i < PER; ++i) value[i] = to_float(loaded[b].v[i]);
            if (weight) {
                float squares = 0.0f;
#pragma unroll
                for (int i = 0; i < PER; ++i) squares += value[i] * value[i];
                const float inverse = rsqrtf(warp_sum(squares) / static_cast<float>(head_dim) + eps);
#pragma unroll
                for (int i = 0; i < PER; ++i) value[i] = round_through<T>(value[i] * inverse * weight[PER * lane + i]);
            }
            Vector result;
            if (rotary_dim) {
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const float partner = __shfl_xor_sync(0xffffffffu, value[i], 16);
                    result.v[i] = from_float<T>(value[i] * cosines[i] + partner * sines[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < PER; ++i) result.v[i] = from_float<T>(value[i]);
            }
            *reinterpret_cast<Vector*>(target + PER * lane) = result;
        }
    }
}

// One warp per (token, query head).  Keys are taken 32 at a time: lane `l` scores key `l` of the chunk
// with a full dot product, the chunk's maximum and sum are found by shuffles, and the values are
// accumulated with each lane owning elements `lane, lane + 32, ...` of the head.
template <typename T>
__global__ void attention_generic_kernel(
    const T* __restrict__ queries, const T* __restrict__ keys, const T* __restrict__ values, T* __restrict__ out,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows,
    int page_stride, int page_tokens, int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale, int window) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ float query_shared[];  // [warps][head_dim]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const long long pair = static_cast<long long>(blockIdx.x) * warps + warp;
    if (pair >= static_cast<long long>(n_tokens) * n_heads) return;  // whole warps leave; no block-wide sync follows
    const int token = static_cast<int>(pair / n_heads), head = static_cast<int>(pair % n_heads);
    const int kv_head = head / (n_heads / n_kv_heads);
    const int position = positions[token];
    const int* pages = page_rows + static_cast<size_t>(token_seq[token]) * page_stride;
    float* query = query_shared + warp * head_dim;
    const T* query_row = queries + (static_cast<size_t>(token) * n_heads + head) * head_dim;
    for (int e = lane; e < head_dim; e += 32) query[e] = to_float(query_row[e]);
    __syncwarp();

    const int first_key = (window > 0 && position - window + 1 > 0) ? position - window + 1 : 0;
    float running_max = -INFINITY, running_sum = 0.0f;
    float acc[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) acc[i] = 0.0f;
    const size_t head_stride = static_cast<size_t>(page_tokens) * head_dim;

    for (int chunk = first_key; chunk <= position; chunk += 32) {
        const int key = chunk + lane;
        const bool live = key <= position;
        float score = -INFINITY;
        size_t offset = 0;
        if (live) {
            const int page = pages[key / page_tokens];
            offset = (static_cast<size_t>(page) * n_kv_heads + kv_head) * head_stride +
                     static_cast<size_t>(key % page_tokens) * head_dim;
            const T* key_row = keys + offset;
            float dot = 0.0f;
            for (int e = 0; e < head_dim; ++e) dot = fmaf(query[e], to_float(key_row[e]), dot);
            score = dot * scale;
        }
        const float chunk_max = warp_max(score);
        const float new_max = fmaxf(running_max, chunk_max);  // finite: lane 0 of every chunk is live
        const float correction = expf(running_max - new_max);
        const float weight = live ? expf(score - new_max) : 0.0f;
        running_sum = running_sum * correction + warp_sum(weight);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) acc[i] *= correction;
        const int in_chunk = min(32, position - chunk + 1);
        for (int j = 0; j < in_chunk; ++j) {
            const float w = __shfl_sync(0xffffffffu, weight, j);
            const size_t value_offset = __shfl_sync(0xffffffffu, static_cast<unsigned long long>(offset), j);
            const T* value_row = values + value_offset;
#pragma unroll
            for (int i = 0; i < kMaxPerLane; ++i) {
                const int e = lane + 32 * i;
                if (e < head_dim) acc[i] = fmaf(w, to_float(value_row[e]), acc[i]);
            }
        }
    }
    T* target = out + (static_cast<size_t>(token) * n_heads + head) * head_dim;
    const float inverse = 1.0f / running_sum;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        if (e < head_dim) target[e] = from_float<T>(acc[i] * inverse);
    }
}

}  // namespace

TAU_EXPORT int tau_attention_prepare(
    int dtype, const void* projected, long long projected_stride, void* queries, void* keys, void* values,
    const float* q_weight, const float* k_weight, float eps, const float* cos_table, const float* sin_table,
    int rotary_dim, const int* positions, const int* token_seq, const int* page_rows, int page_stride, int page_tokens,
    int n_tokens, int n_heads, int n_kv_heads, int head_dim, int write_cache, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!projected || !queries || !positions || head_dim <= 0 || head_dim > 32 * kMaxPerLane || n_heads <= 0 ||
        n_kv_heads <= 0 || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) ||
        (rotary_dim > 0 && (!cos_table || !sin_table)) ||
        (write_cache && (!keys || !values || !token_seq || !page_rows || page_tokens <= 0)))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int heads_total = write_cache ? n_heads + 2 * n_kv_heads : n_heads;
    const int threads = 32 * (heads_total < 8 ? heads_total : 8);
    // The vector form: heads of 64, 128 or 256 elements rotated whole or not at all, rows aligned to a vector.
    const bool whole = (rotary_dim == 0 || rotary_dim == head_dim) && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
                       projected_stride % (head_dim / 32) == 0;
#define TAU_PREPARE_VEC(T, PER)                                                                                                     \
    tau_launch(attention_prepare_vec_kernel<T, PER>, dim3(n_tokens), dim3(threads), 0, s, static_cast<const T*>(projected),          \
               projected_stride, static_cast<T*>(queries), static_cast<T*>(keys), static_cast<T*>(values), q_weight, k_weight, eps,  \
               cos_table, sin_table, rotary_dim, positions, token_seq, page_rows, page_stride, page_tokens, n_heads, n_kv_heads,     \
               write_cache)
    if (whole && dtype == TAU_BF16) {
        if (head_dim == 64) TAU_PREPARE_VEC(bf16, 2);
        else if (head_dim == 128) TAU_PREPARE_VEC(bf16, 4);
        else TAU_PREPARE_VEC(bf16, 8);
        return tau_launch_status();
    }
    if (whole && dtype == TAU_F32) {
        if (head_dim == 64) TAU_PREPARE_VEC(float, 2);
        else if (head_dim == 128) TAU_PREPARE_VEC(float, 4);
        else TAU_PREPARE_VEC(float, 8);
        return tau_launch_status();
    }
#undef TAU_PREPARE_VEC
    if (dtype == TAU_F32)
        tau_launch(attention_prepare_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, 
            static_cast<const float*>(projected), projected_stride, static_cast<float*>(queries), static_cast<float*>(keys),
            static_cast<float*>(values), q_weight, k_weight, eps, cos_table, sin_table, rotary_dim, positions, token_seq,
            page_rows, page_stride, page_tokens, n_heads, n_kv_heads, head_dim, write_cache);
    else if (dtype == TAU_BF16)
        tau_launch(attention_prepare_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, 
            static_cast<const bf16*>(projected), projected_stride, static_cast<bf16*>(queries), static_cast<bf16*>(keys),
            static_cast<bf16*>(values), q_weight, k_weight, eps, cos_table, sin_table, rotary_dim, positions, token_seq,
            page_rows, page_stride, page_tokens, n_heads, n_kv_heads, head_dim, write_cache);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_attention_generic(
    int dtype, const void* queries, const void* keys, const void* values, void* out, const int* positions,
    const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int n_tokens, int n_heads,
    int n_kv_heads, int head_dim, float scale, int window, void* stream) {
    if (n_tokens <= 0) return 0;
    if (!queries || !keys || !values || !out || !positions || !token_seq || !page_rows || head_dim <= 0 ||
        head_dim > 32 * kMaxPerLane || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_tokens <= 0 ||
        window < 0)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    constexpr int warps = 4;
    const long long pairs = static_cast<long long>(n_tokens) * n_heads;
    const unsigned blocks = static_cast<unsigned>((pairs + warps - 1) / warps);
    const size_t shared = warps * head_dim * sizeof(float);
    if (dtype == TAU_F32)
        tau_launch(attention_generic_kernel<float>, dim3(blocks), dim3(warps * 32), shared, s, 
            static_cast<const float*>(queries), static_cast<const float*>(keys), static_cast<const float*>(values),
            static_cast<float*>(out), positions, token_seq, page_rows, page_stride, page_tokens, n_tokens, n_heads,
            n_kv_heads, head_dim, scale, window);
    else if (dtype == TAU_BF16)
        tau_launch(attention_generic_kernel<bf16>, dim3(blocks), dim3(warps * 32), shared, s, 
            static_cast<const bf16*>(queries), static_cast<const bf16*>(keys), static_cast<const bf16*>(values),
            static_cast<bf16*>(out), positions, token_seq, page_rows, page_stride, page_tokens, n_tokens, n_heads,
            n_kv_heads, head_dim, scale, window);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}
