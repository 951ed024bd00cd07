// Random weights drawn on the device: `out[i] = shift + scale * n_i`, n ~ N(0, 1), from a counter-based stream.
//
// The stream is the one of weights/random_init.py, bit for bit: Philox4x32-10 with a 64-bit key per tensor and the
// counter (block, 0, 0, 0); block b gives elements 4 b .. 4 b + 3 by two Box-Muller pairs.  Every operation between the
// words and the value is a single IEEE operation with one rounding (`__fmul_rn`, `__fadd_rn`, `__fdiv_rn`,
// `__fsqrt_rn`, which the compiler neither fuses nor replaces by approximations), and logarithm, sine and cosine are
// the same short polynomials as on the host, so both sides give the same bits.  The reference has no random-weights
// mode (its tests use zeros and patterned tensors, crates/models/src/qwen3_5_common/model.rs:65).
#include "common.cuh"

namespace {

// Constants go from decimal to double to float, as numpy's do.
constexpr float kLn2 = static_cast<float>(0.6931471805599453);
constexpr float kSqrt2 = static_cast<float>(1.4142135623730951);
constexpr float kQuarterPi = static_cast<float>(0.7853981633974483);

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

__device__ __forceinline__ void philox4x32(unsigned c0, unsigned k0, unsigned k1, unsigned (&out)[4]) {
    unsigned c1 = 0u, c2 = 0u, c3 = 0u;
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
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// -2 ln u for u = ((word >> 9) + 1/2) 2^-23.
__device__ __forceinline__ float minus_two_log(unsigned word) {
    const float u = mul(add(static_cast<float>(word >> 9), 0.5f), 1.1920928955078125e-07f);   // 2^-23
    const unsigned bits = __float_as_uint(u);
    int exponent = static_cast<int>(bits >> 23) - 127;
    float mantissa = __uint_as_float((bits & 0x7FFFFFu) | 0x3F800000u);
    if (mantissa > kSqrt2) {
        mantissa = mul(mantissa, 0.5f);
        exponent += 1;
    }
    const float s = __fdiv_rn(add(mantissa, -1.0f), add(mantissa, 1.0f));
    const float z = mul(s, s);
    float p = static_cast<float>(1.0 / 11);
    p = add(mul(p, z), static_cast<float>(1.0 / 9));
    p = add(mul(p, z), static_cast<float>(1.0 / 7));
    p = add(mul(p, z), static_cast<float>(1.0 / 5));
    p = add(mul(p, z), static_cast<float>(1.0 / 3));
    p = mul(p, z);
    const float log_m = mul(add(s, mul(s, p)), 2.0f);
    const float log_u = add(mul(static_cast<float>(exponent), kLn2), log_m);
    return mul(log_u, -2.0f);
}

__device__ __forceinline__ void cos_sin(unsigned word, float& cos_full, float& sin_full) {
    const unsigned k = word >> 9, octant = k >> 20;
    unsigned fraction = k & 0xFFFFFu;
    const bool odd = octant & 1u;
    if (odd) fraction = 0xFFFFFu - fraction;
    const float theta = mul(mul(add(static_cast<float>(fraction), 0.5f), 9.5367431640625e-07f), kQuarterPi);   // 2^-20
    const float t = mul(theta, theta);
    float s = static_cast<float>(1.0 / 362880);
    s = add(mul(s, t), static_cast<float>(-1.0 / 5040));
    s = add(mul(s, t), static_cast<float>(1.0 / 120));
    s = add(mul(s, t), static_cast<float>(-1.0 / 6));
    const float sine = add(theta, mul(theta, mul(s, t)));
    float c = static_cast<float>(-1.0 / 3628800);
    c = add(mul(c, t), static_cast<float>(1.0 / 40320));
    c = add(mul(c, t), static_cast<float>(-1.0 / 720));
    c = add(mul(c, t), static_cast<float>(1.0 / 24));
    c = add(mul(c, t), static_cast<float>(-1.0 / 2));
    const float cosine = add(1.0f, mul(c, t));
    const float first = odd ? sine : cosine, second = odd ? cosine : sine;
    switch (octant >> 1) {
        case 0: cos_full = first; sin_full = second; break;
        case 1: cos_full = -second; sin_full = first; break;
        case 2: cos_full = -first; sin_full = -second; break;
        default: cos_full = second; sin_full = -first; break;
    }
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long count, unsigned key0, unsigned key1, float scale, float shift) {
    const long long blocks = (count + 3) / 4;
    for (long long block = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; block < blocks;
         block += static_cast<long long>(gridDim.x) * blockDim.x) {
        unsigned words[4];
        philox4x32(static_cast<unsigned>(block), key0, key1, words);
        float values[4];
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
            const float radius = __fsqrt_rn(minus_two_log(words[2 * pair]));
            float cosine, sine;
            cos_sin(words[2 * pair + 1], cosine, sine);
            values[2 * pair] = add(mul(mul(radius, cosine), scale), shift);
            values[2 * pair + 1] = add(mul(mul(radius, sine), scale), shift);
        }
        const long long first = block * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (first + i < count) out[first + i] = from_float<T>(values[i]);
    }
}

}  // namespace

// `count` may not exceed 2^34 (the counter's first word numbers the blocks of four).
TAU_EXPORT int tau_random_normal(int dtype, void* out, long long count, unsigned key0, unsigned key1, float scale, float shift, void* stream) {
    if (count <= 0) return 0;
    if (!out || count > (1ll << 34)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long blocks = (count + 3) / 4;
    const unsigned grid = static_cast<unsigned>(blocks / 256 + 1 < 4096 ? blocks / 256 + 1 : 4096);
    if (dtype == TAU_BF16)
        random_normal_kernel<bf16><<<grid, 256, 0, s>>>(static_cast<bf16*>(out), count, key0, key1, scale, shift);
    else if (dtype == TAU_F32)
        random_normal_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(out), count, key0, key1, scale, shift);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}
