// Token selection from 32-bit logits `[rows, vocab]`: greedy argmax and Gumbel-max temperature sampling.
//
// Greedy follows crates/cuda-kernels/src/kernels/greedy_argmax.cu:19-31,65-94,101-117: every logit becomes an
// integer key that orders like the 32-bit float total order, NaN never takes part, the higher token id wins
// among equal keys, and a row of NaN only is reported as invalid.  Two launches: blocks over vocabulary chunks
// write one candidate each to scratch memory, then one block per row merges them.  Rows are independent.
//
// Temperature sampling picks argmax(logit / T + g) with g = -log(-log u), u from Philox4x32-10 with counter
// (token id, index of the token within its request, request number, 0) and the seed as key.
#include "common.cuh"

namespace {

constexpr unsigned kThreads = 256;
constexpr unsigned kItemsPerBlock = 2048;

struct Candidate {
    unsigned key, token, valid;
};

__device__ __forceinline__ Candidate candidate_of(float value, unsigned token) {
    const unsigned bits = __float_as_uint(value);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return {0u, 0u, 0u};
    return {bits ^ ((bits & 0x80000000u) ? 0xffffffffu : 0x80000000u), token, 1u};
}

__device__ __forceinline__ Candidate better(Candidate a, Candidate b) {
    if (!b.valid) return a;
    if (!a.valid || b.key > a.key || (b.key == a.key && b.token > a.token)) return b;
    return a;
}

__device__ Candidate block_best(Candidate value, Candidate* partial) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        Candidate other = {__shfl_xor_sync(0xffffffffu, value.key, offset), __shfl_xor_sync(0xffffffffu, value.token, offset),
                           __shfl_xor_sync(0xffffffffu, value.valid, offset)};
        value = better(value, other);
    }
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = value;
    __syncthreads();
    if (threadIdx.x < 32) {
        value = threadIdx.x < kThreads / 32 ? partial[threadIdx.x] : Candidate{0u, 0u, 0u};
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            Candidate other = {__shfl_xor_sync(0xffffffffu, value.key, offset), __shfl_xor_sync(0xffffffffu, value.token, offset),
                               __shfl_xor_sync(0xffffffffu, value.valid, offset)};
            value = better(value, other);
        }
    }
    return value;  // meaningful in thread 0
}

__device__ __forceinline__ unsigned philox_first_word(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0, unsigned k1) {
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const unsigned long long p0 = 0xD2511F53ull * c0, p1 = 0xCD9E8D57ull * c2;
        const unsigned hi0 = static_cast<unsigned>(p0 >> 32), lo0 = static_cast<unsigned>(p0);
        const unsigned hi1 = static_cast<unsigned>(p1 >> 32), lo1 = static_cast<unsigned>(p1);
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c0;
}

// Score whose maximum is the chosen token.  NaN logits stay NaN and are left out by candidate_of.
__device__ __forceinline__ float gumbel_score(float logit, float inverse_temperature, unsigned token, unsigned token_index,
                                              unsigned request, unsigned seed_lo, unsigned seed_hi) {
    const unsigned word = philox_first_word(token, token_index, request, 0u, seed_lo, seed_hi);
    const float u = (static_cast<float>(word >> 8) + 0.5f) * (1.0f / 16777216.0f);  // in (0, 1), 24 bits
    return logit * inverse_temperature - logf(-logf(u));
}

template <bool Gumbel>
__global__ void chunk_best_kernel(const float* __restrict__ logits, unsigned vocab, unsigned* __restrict__ scratch,
                                  float inverse_temperature, unsigned seed_lo, unsigned seed_hi,
                                  const int* __restrict__ request_ids, const int* __restrict__ token_indices) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ Candidate partial[kThreads / 32];
    const unsigned row = blockIdx.y;
    const float* row_logits = logits + static_cast<size_t>(row) * vocab;
    Candidate best{0u, 0u, 0u};
    const unsigned first = blockIdx.x * kItemsPerBlock;
    const unsigned last = min(vocab, first + kItemsPerBlock);
    unsigned request = 0, token_index = 0;
    if (Gumbel) {
        request = static_cast<unsigned>(request_ids[row]);
        token_index = static_cast<unsigned>(token_indices[row]);
    }
    for (unsigned index = first + threadIdx.x; index < last; index += kThreads) {
        float value = row_logits[index];
        if (Gumbel) value = gumbel_score(value, inverse_temperature, index, token_index, request, seed_lo, seed_hi);
        best = better(best, candidate_of(value, index));
    }
    best = block_best(best, partial);
    if (threadIdx.x == 0) {
        unsigned* slot = scratch + (static_cast<size_t>(row) * gridDim.x + blockIdx.x) * 3;
        slot[0] = best.key;
        slot[1] = best.token;
        slot[2] = best.valid;
    }
}

__global__ void merge_best_kernel(const unsigned* __restrict__ scratch, unsigned chunks, int* __restrict__ tokens,
                                  int* __restrict__ valid) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ Candidate partial[kThreads / 32];
    const unsigned row = blockIdx.x;
    const unsigned* row_scratch = scratch + static_cast<size_t>(row) * chunks * 3;
    Candidate best{0u, 0u, 0u};
    for (unsigned index = threadIdx.x; index < chunks; index += kThreads)
        best = better(best, {row_scratch[index * 3], row_scratch[index * 3 + 1], row_scratch[index * 3 + 2]});
    best = block_best(best, partial);
    if (threadIdx.x == 0) {  // both words are always written, also when every logit was NaN
        tokens[row] = static_cast<int>(best.token);
        valid[row] = static_cast<int>(best.valid);
    }
}

unsigned chunk_count(unsigned vocab) { return (vocab + kItemsPerBlock - 1) / kItemsPerBlock; }

}  // namespace

// Scratch words (uint32) that a selection over `rows` x `vocab` needs.
TAU_EXPORT long long tau_select_scratch_words(int rows, int vocab) {
    if (rows <= 0 || vocab <= 0) return 0;
    return static_cast<long long>(rows) * chunk_count(static_cast<unsigned>(vocab)) * 3;
}

TAU_EXPORT int tau_argmax(const float* logits, int rows, int vocab, unsigned* scratch, long long scratch_words, int* tokens,
                          int* valid, void* stream) {
    if (rows <= 0) return 0;
    if (!logits || !scratch || !tokens || !valid || vocab <= 0 || scratch_words < tau_select_scratch_words(rows, vocab))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned chunks = chunk_count(static_cast<unsigned>(vocab));
    tau_launch(chunk_best_kernel<false>, dim3(dim3(chunks, rows)), dim3(kThreads), 0, s, logits, vocab, scratch, 0.0f, 0u, 0u, nullptr, nullptr);
    int status = tau_launch_status();
    if (status) return status;
    tau_launch(merge_best_kernel, dim3(rows), dim3(kThreads), 0, s, scratch, chunks, tokens, valid);
    return tau_launch_status();
}

TAU_EXPORT int tau_sample_gumbel(const float* logits, int rows, int vocab, unsigned* scratch, long long scratch_words,
                                 int* tokens, int* valid, float inverse_temperature, unsigned long long seed,
                                 const int* request_ids, const int* token_indices, void* stream) {
    if (rows <= 0) return 0;
    if (!logits || !scratch || !tokens || !valid || !request_ids || !token_indices || vocab <= 0 ||
        !(inverse_temperature > 0.0f) || scratch_words < tau_select_scratch_words(rows, vocab))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned chunks = chunk_count(static_cast<unsigned>(vocab));
    tau_launch(chunk_best_kernel<true>, dim3(dim3(chunks, rows)), dim3(kThreads), 0, s, logits, vocab, scratch, inverse_temperature,
                                                                   static_cast<unsigned>(seed), static_cast<unsigned>(seed >> 32),
                                                                   request_ids, token_indices);
    int status = tau_launch_status();
    if (status) return status;
    tau_launch(merge_best_kernel, dim3(rows), dim3(kThreads), 0, s, scratch, chunks, tokens, valid);
    return tau_launch_status();
}

// ---------------------------------------------------------------------------------------------------
// The variant that allocates nothing (declared and described in sampling_static.h).
#include "sampling_static.h"

namespace {

// Scratch of the static variant.  In host code this name is only a stand-in for the symbol: the device
// address comes from cudaGetSymbolAddress, once per device, and that address is what the kernels get.
static __device__ __align__(256) unsigned static_scratch[TAU_ARGMAX_STATIC_WORDS];

constexpr int kMaxDevices = 64;
unsigned* static_scratch_address[kMaxDevices] = {};

}  // namespace

namespace {
// A few words from device memory into pinned host memory, stored by the kernel itself: a copy by the copy engine in the
// same stream held the next kernel up by about 80 us, these stores do not.
__global__ void store_words_kernel(const int* __restrict__ source, volatile int* target, int count) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (int i = threadIdx.x; i < count; i += blockDim.x) target[i] = source[i];
    __threadfence_system();
}
}  // namespace

// `pinned_target` is page-locked host memory; the words are there when the stream has passed this launch.
TAU_EXPORT int tau_store_words_host(const int* source, int* pinned_target, int count, void* stream) {
    if (count <= 0) return 0;
    if (!source || !pinned_target || count > 1 << 20) return cudaErrorInvalidValue;
    cudaPointerAttributes attributes;
    if (cudaPointerGetAttributes(&attributes, pinned_target) != cudaSuccess || attributes.type != cudaMemoryTypeHost || !attributes.devicePointer) {
        cudaGetLastError();
        return cudaErrorInvalidValue;   // not page-locked, or not addressable from the device
    }
    tau_launch(store_words_kernel, dim3(1), dim3(128), 0, static_cast<cudaStream_t>(stream), source, static_cast<volatile int*>(attributes.devicePointer), count);
    return tau_launch_status();
}

TAU_EXPORT long long tau_argmax_static_words_needed(int rows, int vocab) { return tau_select_scratch_words(rows, vocab); }

TAU_EXPORT const char* tau_argmax_static_error(int code) {
    switch (code) {
        case 0: return "no error";
        case TAU_ARGMAX_STATIC_TOO_LARGE: return "rows * ceil(vocab / 2048) * 3 exceeds the static scratch of 24576 words";
        case TAU_ARGMAX_STATIC_BAD_ARGUMENT: return "null pointer, or rows or vocab not positive";
        case TAU_ARGMAX_STATIC_BAD_DEVICE: return "the current device number is 64 or more";
        default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown code";
    }
}

TAU_EXPORT int tau_argmax_static(const float* logits, int rows, int vocab, int* tokens, int* valid, void* stream) {
    if (!logits || !tokens || !valid || rows <= 0 || vocab <= 0) return TAU_ARGMAX_STATIC_BAD_ARGUMENT;
    if (tau_select_scratch_words(rows, vocab) > TAU_ARGMAX_STATIC_WORDS) return TAU_ARGMAX_STATIC_TOO_LARGE;
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return static_cast<int>(status);
    if (device < 0 || device >= kMaxDevices) return TAU_ARGMAX_STATIC_BAD_DEVICE;
    if (!static_scratch_address[device]) {  // set-up: first call on this device, with this device current
        unsigned* address = nullptr;
        status = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), static_scratch);
        if (status != cudaSuccess) return static_cast<int>(status);
        static_scratch_address[device] = address;
    }
    unsigned* scratch = static_scratch_address[device];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned chunks = chunk_count(static_cast<unsigned>(vocab));
    // Writes scratch[0 .. rows * chunks * 3): every word that the merge below reads.
    tau_launch(chunk_best_kernel<false>, dim3(dim3(chunks, rows)), dim3(kThreads), 0, s, logits, vocab, scratch, 0.0f, 0u, 0u, nullptr, nullptr);
    int launched = tau_launch_status();
    if (launched) return launched;
    tau_launch(merge_best_kernel, dim3(rows), dim3(kThreads), 0, s, scratch, chunks, tokens, valid);
    return tau_launch_status();
}
