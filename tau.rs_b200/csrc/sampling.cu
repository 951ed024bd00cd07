// Token selection from 32-bit logits `[rows, vocab]` in one launch: greedy argmax and Gumbel-max temperature sampling.
//
// What is chosen is the reference's (crates/engine/src/generation.rs:81-95; crates/cuda-kernels/src/kernels/
// greedy_argmax.cu:19-31): the greatest logit by the total order of 32-bit floats, NaN never chosen, the highest
// token id among equal logits, and a row of NaN only reported as invalid.  How it is done is this library's own: a
// logit and its token id are packed into one 64-bit word, `ordered(logit) << 32 | token id`, so that the greatest
// word is the choice and the tie rule costs nothing; zero stands for "nothing to choose from" (a NaN).  The grid is
// (vocabulary slices, rows).  A block reduces its slice to one word, stores it, and takes a ticket of its row; the
// block that takes the last ticket of a row reduces the row's words and writes the token.  No block waits for another,
// and one launch serves any number of rows.  The tickets start at zero and each row's last block puts its ticket back.
//
// Temperature sampling picks argmax(logit / T + g) with g = -log(-log u), u from Philox4x32-10 with counter
// (token id, index of the token within its request, request number, 0) and the seed as key.
#include "common.cuh"
#include "sampling_static.h"

namespace {

constexpr unsigned kThreads = 256;
constexpr unsigned kSliceItems = 2048;        // logits per block
constexpr unsigned kTicketWords = 8192;       // the scratch begins with one ticket per row; a launch serves at most this many rows
typedef unsigned long long Packed;

// Monotone map of the float total order onto unsigned integers: negative values have all bits flipped, others the sign bit.
__device__ __forceinline__ Packed pack(float value, unsigned token) {
    if (value != value) return 0ull;
    const unsigned bits = __float_as_uint(value);
    const unsigned ordered = bits ^ (static_cast<unsigned>(static_cast<int>(bits) >> 31) | 0x80000000u);   // >= 0x007fffff for -inf
    return (static_cast<Packed>(ordered) << 32) | token;
}

__device__ __forceinline__ Packed greater_of(Packed a, Packed b) { return a > b ? a : b; }

__device__ __forceinline__ Packed warp_greatest(Packed value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value = greater_of(value, __shfl_xor_sync(0xffffffffu, value, offset));
    return value;
}

// The block's greatest word, in every thread of warp 0.  `shared` holds one word per warp.
__device__ __forceinline__ Packed block_greatest(Packed value, Packed* shared) {
    value = warp_greatest(value);
    __syncthreads();   // `shared` may still be read from an earlier call
    if ((threadIdx.x & 31) == 0) shared[threadIdx.x >> 5] = value;
    __syncthreads();
    value = (threadIdx.x < kThreads / 32) ? shared[threadIdx.x] : 0ull;
    return threadIdx.x < 32 ? warp_greatest(value) : 0ull;
}

__device__ __forceinline__ unsigned philox_first_word(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0, unsigned k1) {
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c0;
}

struct Noise {
    float inverse_temperature;
    unsigned seed_lo, seed_hi, request, token_index;
};

// Score whose maximum is the chosen token.  A NaN logit stays NaN and packs to zero.
template <bool Gumbel> __device__ __forceinline__ float score(float logit, unsigned token, const Noise& noise) {
    if (!Gumbel) return logit;
    const unsigned word = philox_first_word(token, noise.token_index, noise.request, 0u, noise.seed_lo, noise.seed_hi);
    const float u = (static_cast<float>(word >> 8) + 0.5f) * (1.0f / 16777216.0f);  // in (0, 1), 24 bits
    return logit * noise.inverse_temperature - logf(-logf(u));
}

template <bool Gumbel>
__global__ void __launch_bounds__(kThreads) select_kernel(const float* __restrict__ logits, unsigned vocab, Packed* slices, unsigned* tickets,
                                                          int* __restrict__ tokens, int* __restrict__ valid, float inverse_temperature,
                                                          unsigned seed_lo, unsigned seed_hi, const int* __restrict__ request_ids,
                                                          const int* __restrict__ token_indices) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ Packed shared[kThreads / 32];
    __shared__ unsigned is_last;
    const unsigned row = blockIdx.y, n_slices = gridDim.x;
    const float* row_logits = logits + static_cast<size_t>(row) * vocab;
    Noise noise = {inverse_temperature, seed_lo, seed_hi, 0u, 0u};
    if (Gumbel) {
        noise.request = static_cast<unsigned>(request_ids[row]);
        noise.token_index = static_cast<unsigned>(token_indices[row]);
    }
    const unsigned first = blockIdx.x * kSliceItems, last = min(vocab, first + kSliceItems);
    Packed best = 0ull;
    if ((reinterpret_cast<uintptr_t>(row_logits) & 15u) == 0) {   // rows that start on 16 bytes are read four logits at a time
        const unsigned whole = first + ((last - first) & ~3u);
        for (unsigned index = first + threadIdx.x * 4; index < whole; index += kThreads * 4) {
            const float4 four = *reinterpret_cast<const float4*>(row_logits + index);
            best = greater_of(best, pack(score<Gumbel>(four.x, index, noise), index));
            best = greater_of(best, pack(score<Gumbel>(four.y, index + 1, noise), index + 1));
            best = greater_of(best, pack(score<Gumbel>(four.z, index + 2, noise), index + 2));
            best = greater_of(best, pack(score<Gumbel>(four.w, index + 3, noise), index + 3));
        }
        for (unsigned index = whole + threadIdx.x; index < last; index += kThreads)
            best = greater_of(best, pack(score<Gumbel>(row_logits[index], index, noise), index));
    } else {
        for (unsigned index = first + threadIdx.x; index < last; index += kThreads)
            best = greater_of(best, pack(score<Gumbel>(row_logits[index], index, noise), index));
    }
    best = block_greatest(best, shared);
    if (threadIdx.x == 0) {
        slices[static_cast<size_t>(row) * n_slices + blockIdx.x] = best;
        __threadfence();                                            // the word is visible before the ticket is
        is_last = atomicAdd(&tickets[row], 1u) == n_slices - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const volatile Packed* row_slices = slices + static_cast<size_t>(row) * n_slices;
    best = 0ull;
    for (unsigned index = threadIdx.x; index < n_slices; index += kThreads) best = greater_of(best, row_slices[index]);
    best = block_greatest(best, shared);
    if (threadIdx.x == 0) {   // both are always written, so that a row of NaN does not keep an earlier call's token
        tokens[row] = static_cast<int>(static_cast<unsigned>(best));
        valid[row] = best != 0ull;
        tickets[row] = 0u;    // as the next call expects it
    }
}

unsigned slice_count(unsigned vocab) { return (vocab + kSliceItems - 1) / kSliceItems; }

template <bool Gumbel>
int launch_select(const float* logits, int rows, int vocab, Packed* slices, unsigned* tickets, int* tokens, int* valid, float inverse_temperature,
                  unsigned long long seed, const int* request_ids, const int* token_indices, cudaStream_t stream) {
    const unsigned n_slices = slice_count(static_cast<unsigned>(vocab));
    for (int begin = 0; begin < rows; begin += kTicketWords) {      // one launch unless there are more rows than tickets
        const int count = rows - begin < static_cast<int>(kTicketWords) ? rows - begin : static_cast<int>(kTicketWords);
        tau_launch(select_kernel<Gumbel>, dim3(n_slices, count), dim3(kThreads), 0, stream, logits + static_cast<size_t>(begin) * vocab,
                   static_cast<unsigned>(vocab), slices, tickets, tokens + begin, valid + begin, inverse_temperature,
                   static_cast<unsigned>(seed), static_cast<unsigned>(seed >> 32), Gumbel ? request_ids + begin : nullptr,
                   Gumbel ? token_indices + begin : nullptr);
        const int status = tau_launch_status();
        if (status) return status;
    }
    return 0;
}

}  // namespace

// Scratch words (uint32) that a selection over `rows` x `vocab` needs: the tickets, then one 64-bit word per row and
// slice.  The first 8,192 words (the tickets) must be zero before the first call and are zero again after every call;
// the rest may hold anything.
TAU_EXPORT long long tau_select_scratch_words(int rows, int vocab) {
    if (rows <= 0 || vocab <= 0) return 0;
    const long long live_rows = rows < static_cast<int>(kTicketWords) ? rows : kTicketWords;
    return kTicketWords + live_rows * slice_count(static_cast<unsigned>(vocab)) * 2;
}

TAU_EXPORT int tau_argmax(const float* logits, int rows, int vocab, unsigned* scratch, long long scratch_words, int* tokens,
                          int* valid, void* stream) {
    if (rows <= 0) return 0;
    if (!logits || !scratch || !tokens || !valid || vocab <= 0 || scratch_words < tau_select_scratch_words(rows, vocab) ||
        (reinterpret_cast<uintptr_t>(scratch) & 7u))
        return cudaErrorInvalidValue;
    return launch_select<false>(logits, rows, vocab, reinterpret_cast<Packed*>(scratch + kTicketWords), scratch, tokens, valid, 0.0f, 0ull,
                                nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

TAU_EXPORT int tau_sample_gumbel(const float* logits, int rows, int vocab, unsigned* scratch, long long scratch_words,
                                 int* tokens, int* valid, float inverse_temperature, unsigned long long seed,
                                 const int* request_ids, const int* token_indices, void* stream) {
    if (rows <= 0) return 0;
    if (!logits || !scratch || !tokens || !valid || !request_ids || !token_indices || vocab <= 0 ||
        !(inverse_temperature > 0.0f) || scratch_words < tau_select_scratch_words(rows, vocab) || (reinterpret_cast<uintptr_t>(scratch) & 7u))
        return cudaErrorInvalidValue;
    return launch_select<true>(logits, rows, vocab, reinterpret_cast<Packed*>(scratch + kTicketWords), scratch, tokens, valid,
                               inverse_temperature, seed, request_ids, token_indices, static_cast<cudaStream_t>(stream));
}

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

// ---------------------------------------------------------------------------------------------------
// The variant that allocates nothing (declared and described in sampling_static.h).
namespace {

// Scratch of the static variant: 8,192 tickets, then 8,192 64-bit words.  A call that passes the size rule below has at
// most 8,192 rows and at most 8,192 (row, slice) pairs, so both halves are large enough.  The array is zero when the
// library is loaded, which is what the tickets need; the kernel puts every ticket back to zero.
// In host code this name is only a stand-in for the symbol: the device address comes from cudaGetSymbolAddress,
// once per device, and that address is what the kernel gets.
static __device__ __align__(256) unsigned static_scratch[TAU_ARGMAX_STATIC_WORDS];
static_assert(TAU_ARGMAX_STATIC_WORDS == kTicketWords * 3, "tickets and 64-bit words share the array as 1 : 2");

constexpr int kMaxDevices = 64;
unsigned* static_scratch_address[kMaxDevices] = {};

long long static_words_needed(int rows, int vocab) {
    if (rows <= 0 || vocab <= 0) return 0;
    return static_cast<long long>(rows) * slice_count(static_cast<unsigned>(vocab)) * 3;
}

}  // namespace

TAU_EXPORT long long tau_argmax_static_words_needed(int rows, int vocab) { return static_words_needed(rows, vocab); }

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
    if (static_words_needed(rows, vocab) > TAU_ARGMAX_STATIC_WORDS) return TAU_ARGMAX_STATIC_TOO_LARGE;
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
    status = cudaMemsetAsync(scratch, 0, sizeof(unsigned) * rows, s);   // the tickets of this call's rows; no allocation
    if (status != cudaSuccess) return static_cast<int>(status);
    // One launch.  Every 64-bit word that a row's last block reads has been written by a block of this call.
    return launch_select<false>(logits, rows, vocab, reinterpret_cast<Packed*>(scratch + kTicketWords), scratch, tokens, valid, 0.0f, 0ull,
                                nullptr, nullptr, static_cast<cudaStream_t>(stream));
}
