// Weight-streaming product for a few rows of activations (decode): out[M, N] = x[M, K] * w[N, K]^T + bias, M <= 32.
//
// The reference runs these products through cuBLAS as m x 1 x k problems (crates/models/src/components/cuda/
// decode/operation.rs:150-193).  Here the step is bound by reading `w` once from HBM, so the kernel is shaped
// around that stream: a block owns 16 consecutive output features, its warps (16, or 12 where that lets every block
// be resident at once) split K in interleaved chunks of 64 elements, cp.async keeps two chunks per warp in flight in
// lane-private shared-memory slots, and the few activation rows are re-read from L1/L2.  (Measured on the Qwen3-8B
// layer shapes at 8 rows: 16 warps with two chunks in flight stream 5.4 TB/s; 8 warps, deeper rings or an L2 prefetch
// of the block's rows are all slower; the 6144 x 4096 product, whose 384 blocks of 16 warps need a second, thin wave,
// takes 10.0 us with 12 warps against 12.9 us.)  The arithmetic is mma.sync m16n8k16 (bfloat16 in, float accumulate) with the weight
// rows as the A operand and the activations as B; a thread's 16-byte load is used as the fragments of two
// consecutive MMAs, which permutes K inside a chunk identically for both operands and so leaves every dot
// product unchanged.  Partial sums of the warps meet in shared memory.
//
// Needs K % 8 == 0, 16-byte aligned rows of x and w (row strides multiples of 8 elements); other shapes go
// to the plain tiled kernel.
#include "common.cuh"

namespace {

#ifndef TAU_SKINNY_PREFETCH
#define TAU_SKINNY_PREFETCH 0
#endif
#ifndef TAU_SKINNY_MIN_BLOCKS
#define TAU_SKINNY_MIN_BLOCKS 1
#endif
constexpr int kRows = 16;       // output features per block
constexpr int kChunk = 64;      // K elements per warp iteration

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#ifndef TAU_SKINNY_DEPTH
#define TAU_SKINNY_DEPTH 2
#endif
constexpr int kDepth = TAU_SKINNY_DEPTH;                          // chunks in flight per warp
// Shared memory of a block of `warps` warps: the ring, [warp][depth][piece][lane] of 16 bytes, later reused for the
// partial sums, at most [warp][4 * 8 tokens][17] floats.
constexpr int ring_bytes(int warps) {
    return warps * kDepth * 4 * 32 * 16 > warps * 32 * (kRows + 1) * 4 ? warps * kDepth * 4 * 32 * 16 : warps * 32 * (kRows + 1) * 4;
}

__device__ __forceinline__ void copy_async_16(void* destination, const void* source, bool real) {
    const unsigned address = static_cast<unsigned>(__cvta_generic_to_shared(destination));
    const int bytes = real ? 16 : 0;   // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(address), "l"(source), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// `Gated`: a block's 16 rows are 8 gate rows followed by their 8 up rows; it writes silu(gate) * up to `out[M, N / 2]`.
template <int NB, typename TOut, bool Gated, int kWarps>
__global__ void __launch_bounds__(kWarps * 32, TAU_SKINNY_MIN_BLOCKS)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias, TOut* __restrict__ out,
                   int M, int N, int K, long long x_stride, long long w_stride, long long out_stride) {
    grid_dependents_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * kRows;
    // The weights do not depend on the previous kernel: ask L2 for this block's rows, then wait for the activations.
    if (TAU_SKINNY_PREFETCH && threadIdx.x < kRows && row0 + threadIdx.x < N) {
        const bf16* row = w + static_cast<size_t>(row0 + threadIdx.x) * w_stride;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row), "r"(static_cast<unsigned>(K) * 2u) : "memory");
    }
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
    // The weight stream goes through a ring in shared memory that is private to each lane: cp.async puts the four
    // 16-byte pieces of a chunk into the lane's own slots `kDepth` chunks ahead, and the lane reads them back when
    // their turn comes.  Nothing is shared between lanes, so no barrier is needed, and no register waits for data.
    extern __shared__ __align__(16) uint8_t ring_raw[];
    uint4* ring = reinterpret_cast<uint4*>(ring_raw) + (static_cast<size_t>(warp) * kDepth * 4) * 32 + lane;   // [depth][piece][lane]
    const int n_chunks = K > warp * kChunk ? (K - warp * kChunk + kWarps * kChunk - 1) / (kWarps * kChunk) : 0;
    auto issue_chunk = [&](int index) {
        if (index < n_chunks) {
            const int chunk = (warp + index * kWarps) * kChunk;
            const int k_first = chunk + t * 8, k_second = chunk + 32 + t * 8;
            uint4* slot = ring + (index % kDepth) * 4 * 32;
            // K % 8 == 0: a group of 8 elements is whole or absent; an absent group is filled with zeros.
            copy_async_16(slot, w_lo + (k_first < K ? k_first : 0), k_first < K);
            copy_async_16(slot + 32, w_hi + (k_first < K ? k_first : 0), k_first < K);
            copy_async_16(slot + 64, w_lo + (k_second < K ? k_second : 0), k_second < K);
            copy_async_16(slot + 96, w_hi + (k_second < K ? k_second : 0), k_second < K);
        }
        copy_async_commit();
    };
#pragma unroll
    for (int index = 0; index < kDepth - 1; ++index) issue_chunk(index);
    grid_dependency_wait();   // the weights do not depend on the previous kernel; the activations do
    for (int index = 0; index < n_chunks; ++index) {
        issue_chunk(index + kDepth - 1);
        const int chunk = (warp + index * kWarps) * kChunk;
        const int k_first = chunk + t * 8, k_second = chunk + 32 + t * 8;
        const bool first_live = k_first < K, second_live = k_second < K;
        uint4 x1[NB], x2[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            x1[j] = (x_live[j] && first_live) ? __ldg(reinterpret_cast<const uint4*>(x_row[j] + k_first)) : zero;
            x2[j] = (x_live[j] && second_live) ? __ldg(reinterpret_cast<const uint4*>(x_row[j] + k_second)) : zero;
        }
        copy_async_wait<kDepth - 1>();   // this lane's pieces of chunk `index` have landed
        const uint4* slot = ring + (index % kDepth) * 4 * 32;
        const uint4 lo1 = slot[0], hi1 = slot[32], lo2 = slot[64], hi2 = slot[96];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            mma_bf16(acc[j], lo1.x, hi1.x, lo1.y, hi1.y, x1[j].x, x1[j].y);
            mma_bf16(acc[j], lo1.z, hi1.z, lo1.w, hi1.w, x1[j].z, x1[j].w);
            mma_bf16(acc[j], lo2.x, hi2.x, lo2.y, hi2.y, x2[j].x, x2[j].y);
            mma_bf16(acc[j], lo2.z, hi2.z, lo2.w, hi2.w, x2[j].z, x2[j].w);
        }
    }
    copy_async_wait<0>();
    __syncthreads();   // the ring is done with; its memory now holds the warps' partial sums
    float (*partial)[NB * 8][kRows + 1] = reinterpret_cast<float (*)[NB * 8][kRows + 1]>(ring_raw);
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
        float sum = 0.0f;
#pragma unroll
        for (int wi = 0; wi < kWarps; ++wi) sum += partial[wi][token][r];
        if (bias && feature < N) sum += bias[feature];
        if (Gated) {
            // Threads r and r ^ 8 of the same 16 hold a gate and its up value; both are rounded as the unfused product would store them.
            const float mine = round_through<bf16>(sum);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
            if (r < 8 && token < M && feature < N)
                out[static_cast<size_t>(token) * out_stride + (row0 >> 1) + r] = from_float<TOut>(mine / (1.0f + expf(-mine)) * other);
        } else if (token < M && feature < N) {
            out[static_cast<size_t>(token) * out_stride + feature] = from_float<TOut>(sum);
        }
    }
}

template <int NB, typename TOut, bool Gated, int kWarps>
int launch_with(const void* x, const void* w, const float* bias, void* out, int M, int N, int K, long long x_stride, long long w_stride,
                long long out_stride, cudaStream_t stream, int* resident_blocks) {
    constexpr int bytes = ring_bytes(kWarps);
    static int resident = 0;   // blocks of this kernel that the device holds at once
    if (!resident) {
        cudaError_t status = cudaFuncSetAttribute(gemm_skinny_kernel<NB, TOut, Gated, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        int device = 0, sms = 0, per_sm = 0;
        if (status == cudaSuccess) status = cudaGetDevice(&device);
        if (status == cudaSuccess) status = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (status == cudaSuccess)
            status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_skinny_kernel<NB, TOut, Gated, kWarps>, kWarps * 32, bytes);
        if (status != cudaSuccess) return static_cast<int>(status);
        resident = per_sm * sms > 0 ? per_sm * sms : 1;
    }
    if (resident_blocks) {   // a query: nothing is launched
        *resident_blocks = resident;
        return 0;
    }
    const unsigned blocks = (N + kRows - 1) / kRows;
    tau_launch(gemm_skinny_kernel<NB, TOut, Gated, kWarps>, dim3(blocks), dim3(kWarps * 32), bytes, stream, static_cast<const bf16*>(x),
               static_cast<const bf16*>(w), bias, static_cast<TOut*>(out), M, N, K, x_stride, w_stride, out_stride);
    return tau_launch_status();
}

// 16 warps keep the most bytes in flight; where their blocks need a second wave that 12-warp blocks (more of which are
// resident) do not, the 12-warp form runs instead.
template <int NB, typename TOut, bool Gated>
int launch_typed(const void* x, const void* w, const float* bias, void* out, int M, int N, int K, long long x_stride, long long w_stride,
                 long long out_stride, cudaStream_t stream) {
    int wide = 0, narrow = 0;
    int status = launch_with<NB, TOut, Gated, 16>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, stream, &wide);
    if (status == 0) status = launch_with<NB, TOut, Gated, 12>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, stream, &narrow);
    if (status != 0) return status;
    const int blocks = (N + kRows - 1) / kRows;
    if (blocks > wide && blocks <= narrow)
        return launch_with<NB, TOut, Gated, 12>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, stream, nullptr);
    return launch_with<NB, TOut, Gated, 16>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, stream, nullptr);
}

template <int NB, bool Gated>
int launch(int out_dtype, const void* x, const void* w, const float* bias, void* out, int M, int N, int K, long long x_stride,
           long long w_stride, long long out_stride, cudaStream_t stream) {
    if (out_dtype == TAU_BF16) return launch_typed<NB, bf16, Gated>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, stream);
    return launch_typed<NB, float, Gated>(x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, stream);
}

}  // namespace

TAU_EXPORT int tau_gemm_skinny_max_rows() { return 32; }

// bfloat16 inputs; `out_dtype` bfloat16 or float32.  Strides in elements.
TAU_EXPORT int tau_gemm_skinny(int out_dtype, const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                               long long x_stride, long long w_stride, long long out_stride, int gated, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!x || !w || !out || K <= 0 || M > 32 || (K & 7) || (x_stride & 7) || (w_stride & 7) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (out_dtype != TAU_BF16 && out_dtype != TAU_F32) || (gated && (N & 15)))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gated) {
        if (M <= 8) return launch<1, true>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
        if (M <= 16) return launch<2, true>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
        return launch<4, true>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    }
    if (M <= 8) return launch<1, false>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    if (M <= 16) return launch<2, false>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
    return launch<4, false>(out_dtype, x, w, bias, out, M, N, K, x_stride, w_stride, out_stride, s);
}
