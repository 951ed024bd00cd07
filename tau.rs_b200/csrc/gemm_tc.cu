// Tensor-core product for sm_100a: out[M, N] = x[M, K] * w[N, K]^T + bias, bfloat16 in, float accumulate.
//
// The reference hands its dense projections to cuBLAS (crates/models/src/components/cuda/decode/
// operation.rs:150-193, crates/models/src/components/cuda/decode/blas.rs:17-53).  This kernel is written for
// the fifth-generation tensor cores instead: operands are brought into shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast), one thread issues tcgen05.mma, the accumulator
// lives in tensor memory and is read back with tcgen05.ld for the epilogue.
//
// The weight is the stationary operand: a tile is 128 output features (the MMA's M) by BN tokens (its N,
// 16 to 256), so the same kernel serves a 2,048-token prefill (BN = 256) and a decode batch of 64 (BN = 64).
// Both operands are K-major as they lie in memory (`w` is `[out, in]`, `x` is `[tokens, in]`).  In tensor
// memory lane = feature and column = token; an epilogue thread owns one feature and walks the tokens.
//
// A block is persistent over tiles and has six warps: one TMA producer, one MMA issuer, four epilogue
// warps (one per 32-lane quarter of tensor memory).  Shared-memory stages are handed over with
// full/empty mbarriers; two accumulators in tensor memory let the epilogue of one tile overlap the
// products of the next.  Every wait on an mbarrier is bounded: after about two seconds the waiter raises
// an error flag, every role leaves its loop, tensor memory is freed and the kernel returns.
//
// Needs K % 8 == 0 and 16-byte aligned rows (TMA strides); other shapes go to the plain tiled kernel.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;        // features per tile
constexpr int BK = 64;         // K elements per stage: 128 bytes, one swizzle row
constexpr int kMmaK = 16;      // K of one tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

__device__ int gemm_tc_error = 0;   // raised when a wait ran out; read by tau_gemm_tc_status

__device__ __forceinline__ uint32_t smem_address(const void* pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    return now;
}

__device__ __forceinline__ void barrier_init(uint64_t* barrier, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(barrier)), "r"(count));
}

__device__ __forceinline__ void barrier_expect_bytes(uint64_t* barrier, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(barrier)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void barrier_arrive(uint64_t* barrier) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(barrier)) : "memory");
}

__device__ __forceinline__ bool barrier_try_wait(uint64_t* barrier, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_address(barrier)), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with the given parity to complete.  Returns false if the block is giving up.
__device__ __forceinline__ bool barrier_wait(uint64_t* barrier, uint32_t parity, volatile int* abort_flag) {
    if (barrier_try_wait(barrier, parity)) return true;
    const unsigned long long started = global_timer();
    for (uint32_t spin = 1;; ++spin) {
        if (barrier_try_wait(barrier, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer() - started > kWaitLimitNs) {
                *abort_flag = 1;
                atomicExch(&gemm_tc_error, 1);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* destination, const CUtensorMap* map, int inner, int outer, uint64_t* barrier) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_address(destination)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(inner), "r"(outer), "r"(smem_address(barrier))
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes with the 128-byte swizzle:
// groups of 8 rows are 1024 bytes apart; version 1; the leading offset is not used by swizzled K-major tiles.
__device__ __forceinline__ uint64_t tile_descriptor(uint32_t address) {
    return static_cast<uint64_t>((address >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: float accumulate, bfloat16 A and B, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instruction_descriptor(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void mma_issue(uint32_t accumulator, uint64_t a, uint64_t b, uint32_t descriptor, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(accumulator), "l"(a), "l"(b), "r"(descriptor), "r"(accumulate)
        : "memory");
}

// Makes the barrier complete when every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t* barrier) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_address(barrier)) : "memory");
}

__device__ __forceinline__ void tensor_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tensor_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tensor_load_16(uint32_t address, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(address));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct Shared {
    // Barriers and bookkeeping; the operand stages follow at the next 1024-byte boundary.
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t accumulator_full[2];
    uint64_t accumulator_empty[2];
    uint32_t tensor_memory_base;
    int abort_flag;
};

// `Gated`: the weight's rows come in groups of 16, 8 gate rows followed by their 8 up rows; the epilogue writes
// silu(gate) * up, so `out` has N / 2 columns (crates/cuda-kernels/src/kernels/silu_and_mul.cu:51-76 as an epilogue).
template <int BN, typename TOut, bool Gated>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap input_map,
               const float* __restrict__ bias, TOut* __restrict__ out, int M, int N, int K, long long out_stride, int stages) {
    grid_dependents_launch();
    extern __shared__ uint8_t shared_raw[];
    Shared* shared = reinterpret_cast<Shared*>(shared_raw);
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(shared_raw) + sizeof(Shared) + 1023) & ~uintptr_t(1023));
    constexpr uint32_t kWeightBytes = BM * BK * 2, kInputBytes = BN * BK * 2, kStageBytes = kWeightBytes + kInputBytes;
    constexpr uint32_t kColumns = 2 * BN < 32 ? 32 : 2 * BN;   // two accumulators; a power of two of at least 32

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feature_tiles = (N + BM - 1) / BM, token_tiles = (M + BN - 1) / BN;
    const int n_tiles = feature_tiles * token_tiles;
    const int k_blocks = (K + BK - 1) / BK;
    volatile int* abort_flag = &shared->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            barrier_init(&shared->full[s], 1);
            barrier_init(&shared->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            barrier_init(&shared->accumulator_full[a], 1);
            barrier_init(&shared->accumulator_empty[a], 4);   // one arrival per epilogue warp
        }
        shared->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // one warp allocates tensor memory for the block
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(&shared->tensor_memory_base)),
                     "r"(kColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tensor_fence_before_sync();
    __syncthreads();
    tensor_fence_after_sync();
    const uint32_t tensor_base = shared->tensor_memory_base;
    grid_dependency_wait();   // barriers and tensor memory were set up while the previous kernel was finishing

    if (warp == 0) {
        // ---- producer: TMA loads of the weight and input tiles of each stage --------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
                const int feature0 = (tile / token_tiles) * BM, token0 = (tile % token_tiles) * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!barrier_wait(&shared->empty[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
                    uint8_t* weight_tile = tiles + stage * kStageBytes;
                    barrier_expect_bytes(&shared->full[stage], kStageBytes);
                    tma_load_2d(weight_tile, &weight_map, kb * BK, feature0, &shared->full[stage]);
                    tma_load_2d(weight_tile + kWeightBytes, &input_map, kb * BK, token0, &shared->full[stage]);
                    if (++stage == static_cast<uint32_t>(stages)) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ---------------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t descriptor = instruction_descriptor(BN);
            uint32_t stage = 0, phase = 0, local = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++local) {
                const uint32_t slot = local & 1u, use = local >> 1;
                // The epilogue must have drained this accumulator (its first use needs no wait).
                if (use > 0 && !barrier_wait(&shared->accumulator_empty[slot], (use - 1) & 1u, abort_flag)) { alive = false; break; }
                tensor_fence_after_sync();
                const uint32_t accumulator = tensor_base + slot * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!barrier_wait(&shared->full[stage], phase, abort_flag)) { alive = false; break; }
                    tensor_fence_after_sync();
                    const uint32_t weight_address = smem_address(tiles + stage * kStageBytes);
                    const uint32_t input_address = weight_address + kWeightBytes;
#pragma unroll
                    for (int k = 0; k < BK / kMmaK; ++k) {
                        mma_issue(accumulator, tile_descriptor(weight_address + k * kMmaK * 2), tile_descriptor(input_address + k * kMmaK * 2),
                                  descriptor, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    mma_commit(&shared->empty[stage]);   // the stage is free once these products have read it
                    if (++stage == static_cast<uint32_t>(stages)) { stage = 0; phase ^= 1u; }
                }
                if (alive) mma_commit(&shared->accumulator_full[slot]);
            }
        }
    } else {
        // ---- epilogue: four warps, each owns the 32 lanes of tensor memory that its number allows ----
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++local) {
            const uint32_t slot = local & 1u, use = local >> 1;
            const int feature = (tile / token_tiles) * BM + quarter * 32 + lane;
            const int token0 = (tile % token_tiles) * BN;
            if (!barrier_wait(&shared->accumulator_full[slot], use & 1u, abort_flag)) { alive = false; break; }
            tensor_fence_after_sync();
            const float offset = (bias != nullptr && feature < N) ? bias[feature] : 0.0f;
            const uint32_t lane_base = tensor_base + (static_cast<uint32_t>(quarter * 32) << 16) + slot * BN;
#pragma unroll 1
            for (int chunk = 0; chunk < BN; chunk += 16) {
                uint32_t v[16];
                tensor_load_16(lane_base + chunk, v);
                if (Gated) {
                    // Lanes 0-7 of each 16 hold gate rows, lanes 8-15 the matching up rows: bring them together.
                    const int out_feature = (feature >> 4) * 8 + (feature & 7);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        // Both are rounded to the storage type first, as the unfused product would have stored them.
                        const float mine = round_through<bf16>(__uint_as_float(v[j]) + offset);
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
                        const int token = token0 + chunk + j;
                        if ((lane & 8) == 0 && feature < N && token < M)
                            out[static_cast<size_t>(token) * out_stride + out_feature] = from_float<TOut>(__fdividef(mine, 1.0f + __expf(-mine)) * other);   // the result is rounded to bfloat16: the fast forms lose nothing
                    }
                } else if (feature < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int token = token0 + chunk + j;
                        if (token < M) out[static_cast<size_t>(token) * out_stride + feature] = from_float<TOut>(__uint_as_float(v[j]) + offset);
                    }
                }
            }
            tensor_fence_before_sync();
            __syncwarp();
            if (lane == 0) barrier_arrive(&shared->accumulator_empty[slot]);
        }
    }

    // ---- teardown: everyone meets, then the allocating warp frees tensor memory -----------------------
    tensor_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tensor_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tensor_base), "r"(kColumns) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled function = nullptr;
    if (!function) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            function = reinterpret_cast<EncodeTiled>(entry);
    }
    return function;
}

// A map over a row-major bfloat16 matrix `[rows, K]` with row stride `stride` elements; boxes of `box_rows` x 64.
bool make_map(CUtensorMap* map, const void* base, int rows, int K, long long stride, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(stride) * 2};
    const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
    static int count = 0;
    if (!count) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    }
    return count;
}

template <int BN, typename TOut, bool Gated>
int launch(const CUtensorMap& weight_map, const CUtensorMap& input_map, const float* bias, void* out, int M, int N, int K,
           long long out_stride, cudaStream_t stream) {
    constexpr int stage_bytes = (BM + BN) * BK * 2;
    int stages = (200 * 1024) / stage_bytes;
    if (stages > 8) stages = 8;
    const int shared_bytes = sizeof(Shared) + 1024 + stages * stage_bytes;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(gemm_tc_kernel<BN, TOut, Gated>, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_bytes);
        if (status != cudaSuccess) return static_cast<int>(status);
        configured = true;
    }
    const int tiles = ((N + BM - 1) / BM) * ((M + BN - 1) / BN);
    const int blocks = tiles < sm_count() ? tiles : sm_count();
    tau_launch(gemm_tc_kernel<BN, TOut, Gated>, dim3(blocks), dim3(kThreads), shared_bytes, stream, weight_map, input_map, bias, static_cast<TOut*>(out), M, N, K,
                                                                         out_stride, stages);
    return tau_launch_status();
}

template <typename TOut, bool Gated>
int dispatch(const CUtensorMap& weight_map, const CUtensorMap& input_map, int box, const float* bias, void* out, int M, int N, int K,
             long long out_stride, cudaStream_t stream) {
    switch (box) {
        case 16: return launch<16, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, stream);
        case 32: return launch<32, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, stream);
        case 64: return launch<64, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, stream);
        case 128: return launch<128, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, stream);
        default: return launch<256, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, stream);
    }
}

}  // namespace

// 0 if no wait has run out since the library was loaded (synchronises the device).
TAU_EXPORT int tau_gemm_tc_status() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, gemm_tc_error, sizeof(int)) != cudaSuccess) return -1;
    return flag;
}

// bfloat16 inputs; `out_dtype` bfloat16 or float32.  Strides in elements.  `token_box` = 0 picks the token tile from M.
// `gated`: rows of `w` are groups of 8 gate rows and their 8 up rows; `out` is `[M, N / 2]` = silu(gate) * up.
TAU_EXPORT int tau_gemm_tc(int out_dtype, const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                           long long x_stride, long long w_stride, long long out_stride, int token_box, int gated, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!x || !w || !out || K <= 0 || (K & 7) || (x_stride & 7) || (w_stride & 7) || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (reinterpret_cast<uintptr_t>(w) & 15) || (out_dtype != TAU_BF16 && out_dtype != TAU_F32))
        return cudaErrorInvalidValue;
    int box = token_box;
    if (box == 0) box = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if (box != 16 && box != 32 && box != 64 && box != 128 && box != 256) return cudaErrorInvalidValue;
    CUtensorMap weight_map, input_map;
    if (!make_map(&weight_map, w, N, K, w_stride, BM) || !make_map(&input_map, x, M, K, x_stride, box)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gated) return dispatch<bf16, true>(weight_map, input_map, box, bias, out, M, N, K, out_stride, s);
    if (out_dtype == TAU_BF16) return dispatch<bf16, false>(weight_map, input_map, box, bias, out, M, N, K, out_stride, s);
    return dispatch<float, false>(weight_map, input_map, box, bias, out, M, N, K, out_stride, s);
}
