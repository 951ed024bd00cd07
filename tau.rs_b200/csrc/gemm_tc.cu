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
// With few tiles (a decode batch of 64 has 32 tiles of the output projection for 148 SMs) the work is also cut
// along K: a work item is (tile, K range), each item leaves its float partial tile in a workspace, and the
// epilogue warp that arrives last at a (tile, quarter) ticket adds the partials in the order of the ranges, so
// the sum does not depend on who finishes last, and stores the result.  No block waits for another.
// Where all items are resident at once, the blocks of a tile are launched as one thread-block cluster instead: the
// partials stay in shared memory, the blocks meet at the cluster's barrier, and each adds and stores a slice of
// the tile's tokens, reading the others' partials through distributed shared memory (again in the order of the ranges).
//
// Needs K % 8 == 0 and 16-byte aligned rows (TMA strides); other shapes go to the plain tiled kernel.
#include <cuda.h>
#include <cstdio>

#include "common.cuh"

namespace {

constexpr int BM = 128;        // features per tile
constexpr int BK = 64;         // K elements per stage: 128 bytes, one swizzle row
constexpr int kMmaK = 16;      // K of one tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;        // producer, issuer, four epilogue warps
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

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

// The address, in the cluster's shared window, of `pointer`'s twin in the block of rank `rank`.
__device__ __forceinline__ uint32_t cluster_address(const void* pointer, uint32_t rank) {
    uint32_t address;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(address) : "r"(smem_address(pointer)), "r"(rank));
    return address;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_address_of(uint32_t shared_address, int rank) {
    uint32_t address;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(address) : "r"(shared_address), "r"(rank));
    return address;
}

// Four floats from the shared memory of a block of the cluster (an address from `cluster_address`).
__device__ __forceinline__ float4 cluster_load_4(uint32_t address) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(address) : "memory");
    return v;
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
__global__ void __launch_bounds__(kThreads, BN <= 128 ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap input_map,
               const float* __restrict__ bias, TOut* __restrict__ out, int M, int N, int K, long long out_stride, int stages,
               int splits, float* __restrict__ workspace, int* __restrict__ tickets, int clustered) {
    extern __shared__ uint8_t shared_raw[];
    Shared* shared = reinterpret_cast<Shared*>(shared_raw);
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(shared_raw) + sizeof(Shared) + 1023) & ~uintptr_t(1023));
    constexpr uint32_t kWeightBytes = BM * BK * 2, kInputBytes = BN * BK * 2, kStageBytes = kWeightBytes + kInputBytes;
    constexpr uint32_t kColumns = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;   // two accumulators; a power of two of at least 32
    float* const own_partial = reinterpret_cast<float*>(tiles);   // clustered: [token][BM] floats over the stages, once they are done with

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feature_tiles = (N + BM - 1) / BM, token_tiles = (M + BN - 1) / BN;
    const int n_items = feature_tiles * token_tiles * splits;   // item = tile * splits + K range
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
    // Only now may the next kernel's blocks start beside this one: a block of it that took tensor memory before this block
    // had its own would make this block's allocation wait for a kernel that in turn waits for this one.
    grid_dependents_launch();
    // Barriers and tensor memory were set up while the previous kernel was finishing.  Each role waits for that kernel
    // only before it touches what that kernel may write or read: the inputs (producer) and the output (epilogue).

    if (warp == 0) {
        // ---- producer: TMA loads of the weight and input tiles of each stage --------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            // The weight never depends on the previous kernel: until every stage is in use, only weight tiles are asked
            // for; then the producer waits for the previous kernel and sends the input tiles of those stages after them.
            bool waited = false;
            int held = 0, held_k[8], held_token[8];
            auto release = [&]() {
                grid_dependency_wait();
                waited = true;
                for (int h = 0; h < held; ++h)
                    tma_load_2d(tiles + h * kStageBytes + kWeightBytes, &input_map, held_k[h], held_token[h], &shared->full[h]);
            };
            for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
                const int tile = item / splits, split = item - tile * splits;
                const int feature0 = (tile / token_tiles) * BM, token0 = (tile % token_tiles) * BN;
                const int kb_begin = k_blocks * split / splits, count = k_blocks * (split + 1) / splits - kb_begin;
                for (int i = 0; i < count; ++i) {
                    const int kb = kb_begin + i;
                    if (!waited && held == stages) release();
                    if (!barrier_wait(&shared->empty[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
                    uint8_t* weight_tile = tiles + stage * kStageBytes;
                    barrier_expect_bytes(&shared->full[stage], kStageBytes);
                    tma_load_2d(weight_tile, &weight_map, kb * BK, feature0, &shared->full[stage]);
                    if (waited) {
                        tma_load_2d(weight_tile + kWeightBytes, &input_map, kb * BK, token0, &shared->full[stage]);
                    } else {   // the first `stages` loads: stage == held
                        held_k[held] = kb * BK;
                        held_token[held] = token0;
                        ++held;
                    }
                    if (++stage == static_cast<uint32_t>(stages)) { stage = 0; phase ^= 1u; }
                }
            }
            if (!waited) release();
        }
    } else if (warp == 1) {
        // ---- MMA issuer ---------------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t descriptor = instruction_descriptor(BN);
            uint32_t stage = 0, phase = 0, local = 0;
            bool alive = true;
            for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x, ++local) {
                const uint32_t slot = local & 1u, use = local >> 1;
                const int split = item % splits;
                const int kb_begin = k_blocks * split / splits, kb_end = k_blocks * (split + 1) / splits;
                // The epilogue must have drained this accumulator (its first use needs no wait).
                if (use > 0 && !barrier_wait(&shared->accumulator_empty[slot], (use - 1) & 1u, abort_flag)) { alive = false; break; }
                tensor_fence_after_sync();
                const uint32_t accumulator = tensor_base + slot * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {   // the producer decides which K block a stage holds
                    if (!barrier_wait(&shared->full[stage], phase, abort_flag)) { alive = false; break; }
                    tensor_fence_after_sync();
                    const uint32_t weight_address = smem_address(tiles + stage * kStageBytes);
                    const uint32_t input_address = weight_address + kWeightBytes;
#pragma unroll
                    for (int k = 0; k < BK / kMmaK; ++k) {
                        mma_issue(accumulator, tile_descriptor(weight_address + k * kMmaK * 2), tile_descriptor(input_address + k * kMmaK * 2),
                                  descriptor, (kb > kb_begin || k > 0) ? 1u : 0u);
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
        grid_dependency_wait();   // the output, the workspace and the tickets may still be in use by the previous kernel
        for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x, ++local) {
            const uint32_t slot = local & 1u, use = local >> 1;
            const int tile = item / splits;
            const int feature = (tile / token_tiles) * BM + quarter * 32 + lane;
            const int token0 = (tile % token_tiles) * BN;
            if (!barrier_wait(&shared->accumulator_full[slot], use & 1u, abort_flag)) { alive = false; break; }
            tensor_fence_after_sync();
            const float offset = (bias != nullptr && feature < N) ? bias[feature] : 0.0f;
            const uint32_t lane_base = tensor_base + (static_cast<uint32_t>(quarter * 32) << 16) + slot * BN;
            // Finishes one value of this thread's feature; every lane of the warp calls it together.
            auto finish = [&](float value, int token) {
                if (Gated) {
                    // Lanes 0-7 of each 16 hold gate rows, lanes 8-15 the matching up rows: bring them together.
                    // Both are rounded to the storage type first, as the unfused product would have stored them.
                    const float mine = round_through<bf16>(value + offset);
                    const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
                    if ((lane & 8) == 0 && feature < N && token < M)
                        out[static_cast<size_t>(token) * out_stride + (feature >> 4) * 8 + (feature & 7)] =
                            from_float<TOut>(__fdividef(mine, 1.0f + __expf(-mine)) * other);   // the result is rounded to bfloat16: the fast forms lose nothing
                } else if (feature < N && token < M) {
                    out[static_cast<size_t>(token) * out_stride + feature] = from_float<TOut>(value + offset);
                }
            };
            if (splits == 1) {
#pragma unroll 1
                for (int chunk = 0; chunk < BN; chunk += 16) {
                    uint32_t v[16];
                    tensor_load_16(lane_base + chunk, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) finish(__uint_as_float(v[j]), token0 + chunk + j);
                }
                tensor_fence_before_sync();
                __syncwarp();
                if (lane == 0) barrier_arrive(&shared->accumulator_empty[slot]);
                continue;
            }
            const int live = min(BN, M - token0);
            if (clustered) {
                // A K range of the tile, one of a cluster's: the partial stays here, in the memory of the stages (every
                // product has read them: the accumulator is complete), as [token][feature of the tile].
#pragma unroll 1
                for (int chunk = 0; chunk < live; chunk += 16) {
                    uint32_t v[16];
                    tensor_load_16(lane_base + chunk, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (chunk + j < live) own_partial[(chunk + j) * BM + quarter * 32 + lane] = __uint_as_float(v[j]);
                }
                tensor_fence_before_sync();
                __syncwarp();
                if (lane == 0) barrier_arrive(&shared->accumulator_empty[slot]);
                continue;
            }
            // A K range of the tile: the partial goes to the workspace as [token][feature of the tile].
            float* mine = workspace + static_cast<size_t>(item) * (BN * BM) + quarter * 32 + lane;
#pragma unroll 1
            for (int chunk = 0; chunk < live; chunk += 16) {
                uint32_t v[16];
                tensor_load_16(lane_base + chunk, v);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (chunk + j < live) __stcg(mine + (chunk + j) * BM, __uint_as_float(v[j]));
            }
            tensor_fence_before_sync();
            __syncwarp();
            if (lane == 0) barrier_arrive(&shared->accumulator_empty[slot]);
            // The warp that takes the last ticket of this quarter of the tile adds the partials and stores.
            __threadfence();
            __syncwarp();
            int ticket = 0;
            if (lane == 0) ticket = atomicAdd(&tickets[tile * 4 + quarter], 1);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            if (ticket != splits - 1) continue;
            __threadfence();
            if (lane == 0) tickets[tile * 4 + quarter] = 0;   // left at zero for the next launch
            // Here a lane owns four neighbouring features of four tokens apart: 16-byte loads, many of them in flight,
            // since this warp alone reads what `splits` blocks wrote.  The ranges are added in their order, whoever is last.
            const int sub = lane >> 3, group = lane & 7;
            const int feature4 = (tile / token_tiles) * BM + quarter * 32 + group * 4;
            float offset4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) offset4[i] = (bias != nullptr && feature4 + i < N) ? bias[feature4 + i] : 0.0f;
            const float4* first = reinterpret_cast<const float4*>(workspace + static_cast<size_t>(tile) * splits * (BN * BM) + quarter * 32 + group * 4);
            constexpr int kSteps = BN / 4 < 16 ? BN / 4 : 16;
#pragma unroll 1
            for (int block = 0; block < live; block += 4 * kSteps) {
                float4 sum[kSteps];
#pragma unroll
                for (int u = 0; u < kSteps; ++u) sum[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 1
                for (int s = 0; s < splits; ++s) {
                    float4 part[kSteps];
#pragma unroll
                    for (int u = 0; u < kSteps; ++u) {
                        const int token = block + 4 * u + sub;
                        part[u] = token < live ? __ldcg(first + (static_cast<size_t>(s) * BN + token) * (BM / 4)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
#pragma unroll
                    for (int u = 0; u < kSteps; ++u) {
                        sum[u].x += part[u].x; sum[u].y += part[u].y; sum[u].z += part[u].z; sum[u].w += part[u].w;
                    }
                }
#pragma unroll
                for (int u = 0; u < kSteps; ++u) {
                    const int token = token0 + block + 4 * u + sub;
                    const float value[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
                    if (Gated) {
                        // Groups 0-1 of each four hold gate rows, groups 2-3 the matching up rows (two lanes further).
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float mine = round_through<bf16>(value[i] + offset4[i]);
                            const float other = __shfl_xor_sync(0xffffffffu, mine, 2);
                            const int feature = feature4 + i;
                            if ((group & 2) == 0 && feature < N && token < M)
                                out[static_cast<size_t>(token) * out_stride + (feature >> 4) * 8 + (feature & 7)] =
                                    from_float<TOut>(__fdividef(mine, 1.0f + __expf(-mine)) * other);
                        }
                    } else if (token < M) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (feature4 + i < N) out[static_cast<size_t>(token) * out_stride + feature4 + i] = from_float<TOut>(value[i] + offset4[i]);
                    }
                }
            }
        }
    }

    // ---- teardown: everyone meets, then the allocating warp frees tensor memory -----------------------
    tensor_fence_before_sync();
    __syncthreads();
    if (clustered) {
        // The cluster's blocks hold the K ranges of one tile.  Every thread of every block comes here, also after a wait
        // that ran out, so the two meetings below cannot be missed.  Between them each block adds, for its slice of the
        // tile's tokens, the partials of all ranges in their order (its own among them) and stores the result.
        cluster_sync_all();
        if (*abort_flag == 0) {
            grid_dependency_wait();
            const int tile = blockIdx.x / splits;
            const int rank = static_cast<int>(cluster_rank());
            const int feature0 = (tile / token_tiles) * BM, token0 = (tile % token_tiles) * BN;
            const int live = min(BN, M - token0);
            const int per = (live + splits - 1) / splits;
            const int first = rank * per, count = max(0, min(per, live - first));
            const int group = threadIdx.x & 31;                 // four neighbouring features of the tile; a warp spans its 128
            const int feature4 = feature0 + group * 4;
            float offset4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) offset4[i] = (bias != nullptr && feature4 + i < N) ? bias[feature4 + i] : 0.0f;
            const uint32_t own = smem_address(own_partial);
            for (int row = warp; row < count; row += kThreads / 32) {
                const int token_in_tile = first + row;
                const uint32_t address = own + static_cast<uint32_t>((token_in_tile * BM + group * 4) * 4);
                float4 part[8];
#pragma unroll
                for (int r = 0; r < 8; ++r)   // all ranges' loads leave together
                    part[r] = r < splits ? cluster_load_4(cluster_address_of(address, r)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                float value[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r < splits) { value[0] += part[r].x; value[1] += part[r].y; value[2] += part[r].z; value[3] += part[r].w; }
                const int token = token0 + token_in_tile;
                if (Gated) {
                    // Groups 0-1 of each four hold gate rows, groups 2-3 the matching up rows (two lanes further).
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float mine = round_through<bf16>(value[i] + offset4[i]);
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 2);
                        const int feature = feature4 + i;
                        if ((group & 2) == 0 && feature < N)
                            out[static_cast<size_t>(token) * out_stride + (feature >> 4) * 8 + (feature & 7)] =
                                from_float<TOut>(__fdividef(mine, 1.0f + __expf(-mine)) * other);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (feature4 + i < N) out[static_cast<size_t>(token) * out_stride + feature4 + i] = from_float<TOut>(value[i] + offset4[i]);
                }
            }
        }
        cluster_sync_all();   // nobody leaves while another still reads its partial
    }
    if (warp == 1) {
        tensor_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tensor_base), "r"(kColumns) : "memory");
    }
}

// ---- pairs of SMs on one tile ------------------------------------------------------------------------------
// For many tokens the product is bound by the tensor cores, and a 128 x 256 tile per SM spends as much shared-memory
// bandwidth on filling and reading its operands as the products can use.  Two blocks of a cluster therefore share a
// 256 (tokens) x 256 (features) tile: each brings 128 of the tokens and half of the weight rows, one thread of the first
// block issues tcgen05.mma.cta_group::2, which reads the weight halves of both blocks, and each block's tensor memory
// receives its 128 tokens x 256 features.  Per product a block fills 32 KB of shared memory, not 48 KB.
//
// Here the tokens are the rows of the product (lanes of tensor memory) and the features its columns, so an epilogue
// thread owns one token and reads runs of neighbouring features: it stores 16 bytes at a time where the output's rows
// allow it, and the gate and up values of a gated product (groups of 8 and 8 features) meet inside one thread.
//
// Pair `p` takes the tiles `p, p + pairs, ...`: at any time the pairs work on neighbouring tiles at the same depth of
// K, so a block of the weight or of the input is fetched from memory once and hit in L2 by the others within
// microseconds.  (Sharing out the last, partly filled wave in quarter tiles of 64 features was measured and is not
// done: copies of 32 weight rows and products of 64 to 192 features ran so much slower that the products of a
// 2,048-token prefill layer took 655 us against 551 us.)
//
// The first block's `full` barriers count the bytes of both blocks' copies (the peer's TMA copies signal them across
// the cluster); tcgen05.commit signals `empty` and `accumulator_full` in both blocks; the epilogue warps of both
// blocks release an accumulator at the first block's barrier.  All waits are bounded as above.  No copy is multicast.
constexpr int kPairTokens = 256, kPairHalf = 128, kPairFeatures = 256;

__device__ __forceinline__ void barrier_arrive_cluster(uint32_t cluster_barrier) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_barrier) : "memory");
}

// A TMA copy into this block's shared memory whose bytes are counted by a barrier given as a cluster address.
__device__ __forceinline__ void tma_load_2d_pair(void* destination, const CUtensorMap* map, int inner, int outer, uint32_t cluster_barrier) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_address(destination)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(inner), "r"(outer), "r"(cluster_barrier)
                 : "memory");
}

__device__ __forceinline__ void mma_issue_pair(uint32_t accumulator, uint64_t a, uint64_t b, uint32_t descriptor, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(accumulator), "l"(a), "l"(b), "r"(descriptor), "r"(accumulate)
        : "memory");
}

// Arrives, in both blocks of the pair, at the barrier that lies where `barrier` lies, once the products issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint64_t* barrier) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_address(barrier)),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}

// 32 consecutive columns of this thread's lane; the caller waits (`tensor_load_wait`) before it uses them.
__device__ __forceinline__ void tensor_load_32(uint32_t address, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(address));
}

__device__ __forceinline__ void tensor_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_pair(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

// `vector_stores`: the output's rows start on 16 bytes and N is a multiple of 8 (16 where gated), so 16-byte stores of
// whole groups of features are safe; otherwise every value is stored on its own.
template <typename TOut, bool Gated>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap input_map,
                    const float* __restrict__ bias, TOut* __restrict__ out, int M, int N, int K, long long out_stride, int stages,
                    int vector_stores) {
    extern __shared__ uint8_t shared_raw[];
    Shared* shared = reinterpret_cast<Shared*>(shared_raw);
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(shared_raw) + sizeof(Shared) + 1023) & ~uintptr_t(1023));
    constexpr uint32_t kInputBytes = kPairHalf * BK * 2, kWeightBytes = BM * BK * 2, kStageBytes = kInputBytes + kWeightBytes;
    constexpr uint32_t kColumns = 2 * kPairFeatures;   // two accumulators of 256 columns: all of tensor memory

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int feature_tiles = (N + kPairFeatures - 1) / kPairFeatures, token_tiles = (M + kPairTokens - 1) / kPairTokens;
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
            barrier_init(&shared->accumulator_empty[a], 8);   // one arrival per epilogue warp of both blocks (used in the first block)
        }
        shared->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both blocks allocates tensor memory for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(&shared->tensor_memory_base)),
                     "r"(kColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tensor_fence_before_sync();
    cluster_sync_all();   // both blocks' barriers exist before either signals the other's
    tensor_fence_after_sync();
    const uint32_t tensor_base = shared->tensor_memory_base;
    grid_dependents_launch();   // after this pair holds its tensor memory (see gemm_tc_kernel)

    if (warp == 0) {
        // ---- producer (both blocks): this block's 128 tokens and its 128 weight rows -----------------------------
        if (lane == 0) {
            grid_dependency_wait();
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            for (int tile = pair; tile < n_tiles && alive; tile += n_pairs) {
                const int token0 = (tile % token_tiles) * kPairTokens + static_cast<int>(rank) * kPairHalf;
                const int feature0 = (tile / token_tiles) * kPairFeatures + static_cast<int>(rank) * BM;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!barrier_wait(&shared->empty[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
                    uint8_t* input_tile = tiles + stage * kStageBytes;
                    const uint32_t first_full = cluster_address(&shared->full[stage], 0);
                    if (rank == 0) barrier_expect_bytes(&shared->full[stage], 2 * kStageBytes);   // the bytes of both blocks
                    tma_load_2d_pair(input_tile, &input_map, kb * BK, token0, first_full);
                    tma_load_2d_pair(input_tile + kInputBytes, &weight_map, kb * BK, feature0, first_full);
                    if (++stage == static_cast<uint32_t>(stages)) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: one thread of the first block, for both --------------------------------------------------
        if (lane == 0 && rank == 0) {
            // M = 256 tokens over the pair, N = 256 features.
            const uint32_t descriptor = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kPairFeatures >> 3) << 17) |
                                        (static_cast<uint32_t>(kPairTokens >> 4) << 24);
            uint32_t stage = 0, phase = 0, local = 0;
            bool alive = true;
            for (int tile = pair; tile < n_tiles && alive; tile += n_pairs, ++local) {
                const uint32_t slot = local & 1u, use = local >> 1;
                if (use > 0 && !barrier_wait(&shared->accumulator_empty[slot], (use - 1) & 1u, abort_flag)) { alive = false; break; }
                tensor_fence_after_sync();
                const uint32_t accumulator = tensor_base + slot * kPairFeatures;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!barrier_wait(&shared->full[stage], phase, abort_flag)) { alive = false; break; }
                    tensor_fence_after_sync();
                    const uint32_t input_address = smem_address(tiles + stage * kStageBytes);
                    const uint32_t weight_address = input_address + kInputBytes;
#pragma unroll
                    for (int k = 0; k < BK / kMmaK; ++k) {
                        mma_issue_pair(accumulator, tile_descriptor(input_address + k * kMmaK * 2), tile_descriptor(weight_address + k * kMmaK * 2),
                                       descriptor, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    mma_commit_pair(&shared->empty[stage]);   // frees the stage in both blocks
                    if (++stage == static_cast<uint32_t>(stages)) { stage = 0; phase ^= 1u; }
                }
                if (alive) mma_commit_pair(&shared->accumulator_full[slot]);
            }
        }
    } else {
        // ---- epilogue (both blocks): this block's 128 tokens of the tile's 256 features; a thread owns a token -------
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool alive = true;
        grid_dependency_wait();
        for (int tile = pair; tile < n_tiles && alive; tile += n_pairs, ++local) {
            const uint32_t slot = local & 1u, use = local >> 1;
            const int tile_feature0 = (tile / token_tiles) * kPairFeatures;
            const int warp_token0 = (tile % token_tiles) * kPairTokens + static_cast<int>(rank) * kPairHalf + quarter * 32;
            const int token = warp_token0 + lane;
            if (!barrier_wait(&shared->accumulator_full[slot], use & 1u, abort_flag)) { alive = false; break; }
            tensor_fence_after_sync();
            const uint32_t lane_base = tensor_base + (static_cast<uint32_t>(quarter * 32) << 16) + slot * kPairFeatures;
            const bool row_live = token < M;
            // The values of `count` (a multiple of 32) features from `column` on, bias added: every lane of the warp calls it together.
            auto load_features = [&](int column, float (&value)[32]) {
                uint32_t v[32];
                tensor_load_32(lane_base + column, v);
                tensor_load_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) value[j] = __uint_as_float(v[j]);
                if (bias != nullptr) {
                    const int feature = tile_feature0 + column;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (feature + j < N) value[j] += __ldg(bias + feature + j);
                }
            };
            // silu(gate) * up of the 16 + 16 features in `value` (groups of 8 gate values followed by their 8 up values); both
            // are rounded to the storage type first, as the unfused product would have stored them.
            auto gated_pairs = [&](const float (&value)[32], uint32_t* packed) {
#pragma unroll
                for (int group = 0; group < 2; ++group) {
                    float result[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float gate = round_through<bf16>(value[16 * group + j]), up = round_through<bf16>(value[16 * group + 8 + j]);
                        result[j] = __fdividef(gate, 1.0f + __expf(-gate)) * up;   // the result is rounded to bfloat16: the fast forms lose nothing
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) packed[4 * group + j] = pack_pair(result[2 * j], result[2 * j + 1]);
                }
            };
            if (warp_token0 < M && vector_stores) {   // the same for the whole warp
                // A lane gathers 128 bytes of its token's output row at a time (64 bfloat16 features, 32 float ones, or the
                // 64 results of 128 gated ones), the warp turns its 32 x 128 bytes over in shared memory, and then eight lanes
                // store one row's 128 bytes side by side: a store touches 4 lines of memory and fills them, where the lanes'
                // own rows would be 32 lines, 16 bytes of each.
                constexpr int kFeaturesPerPass = Gated ? 128 : (sizeof(TOut) == 2 ? 64 : 32);
                constexpr int kOutputsPerPass = Gated ? 64 : kFeaturesPerPass;
                constexpr int kOutputsPerPiece = 16 / static_cast<int>(sizeof(TOut));
                const uint32_t staging = smem_address(tiles + stages * kStageBytes) + static_cast<uint32_t>(quarter) * 4096u;
                const int outputs = Gated ? N / 2 : N;
#pragma unroll 1
                for (int column = 0; column < kPairFeatures; column += kFeaturesPerPass) {
                    if (tile_feature0 + column >= N) break;
                    uint32_t packed[32];
                    if constexpr (Gated) {
#pragma unroll
                        for (int part = 0; part < 4; ++part) {
                            float value[32];
                            load_features(column + 32 * part, value);
                            gated_pairs(value, packed + 8 * part);
                        }
                    } else if constexpr (sizeof(TOut) == 2) {
#pragma unroll
                        for (int part = 0; part < 2; ++part) {
                            float value[32];
                            load_features(column + 32 * part, value);
#pragma unroll
                            for (int j = 0; j < 16; ++j) packed[16 * part + j] = pack_pair(value[2 * j], value[2 * j + 1]);
                        }
                    } else {
                        float value[32];
                        load_features(column, value);
#pragma unroll
                        for (int j = 0; j < 32; ++j) packed[j] = __float_as_uint(value[j]);
                    }
                    __syncwarp();   // the pass before has been read out of the staging rows
#pragma unroll
                    for (int piece = 0; piece < 8; ++piece)   // row `lane`; the pieces of a row change places so that eight lanes meet eight banks
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(staging + lane * 128u + ((piece ^ (lane & 7)) << 4)),
                                     "r"(packed[4 * piece]), "r"(packed[4 * piece + 1]), "r"(packed[4 * piece + 2]), "r"(packed[4 * piece + 3])
                                     : "memory");
                    __syncwarp();
                    const int output0 = (Gated ? (tile_feature0 + column) / 2 : tile_feature0 + column) + (lane & 7) * kOutputsPerPiece;
#pragma unroll
                    for (int step = 0; step < 8; ++step) {
                        const int row = 4 * step + (lane >> 3);
                        uint4 data;
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(data.x), "=r"(data.y), "=r"(data.z), "=r"(data.w)
                                     : "r"(staging + row * 128u + (((lane & 7) ^ (row & 7)) << 4)));
                        if (warp_token0 + row < M && output0 < outputs)
                            *reinterpret_cast<uint4*>(out + static_cast<size_t>(warp_token0 + row) * out_stride + output0) = data;
                    }
                }
                (void)kOutputsPerPass;
            } else if (warp_token0 < M) {
                // Rows of the output that do not start on 16 bytes, or a number of features that cuts a group: value by value.
#pragma unroll 1
                for (int column = 0; column < kPairFeatures; column += 32) {
                    const int feature = tile_feature0 + column;
                    if (feature >= N) break;
                    float value[32];
                    load_features(column, value);
                    if (!row_live) continue;
                    if (Gated) {
                        uint32_t packed[8];
                        gated_pairs(value, packed);
                        TOut* target = out + static_cast<size_t>(token) * out_stride + (feature >> 1);
                        const bf16* results = reinterpret_cast<const bf16*>(packed);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (feature + 16 * (j / 8) < N) target[j] = from_float<TOut>(__bfloat162float(results[j]));
                    } else {
                        TOut* target = out + static_cast<size_t>(token) * out_stride + feature;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (feature + j < N) target[j] = from_float<TOut>(value[j]);
                    }
                }
            }
            tensor_fence_before_sync();
            __syncwarp();
            if (lane == 0) barrier_arrive_cluster(cluster_address(&shared->accumulator_empty[slot], 0));
        }
    }

    // ---- teardown: both blocks meet (neither's shared or tensor memory is in use by the other), then free -------------
    tensor_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tensor_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tensor_base), "r"(kColumns) : "memory");
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

// Token tiles up to 128 belong to products that are bound by reading the weight (a decode batch): their blocks take
// half an SM's shared memory, so that two are resident and the next kernel's blocks can start beside this one's.
template <int BN> constexpr int stage_budget() { return BN <= 128 ? 100 * 1024 : 200 * 1024; }
template <int BN> constexpr int blocks_per_sm() { return BN <= 128 ? 2 : 1; }

// How many K ranges a product is cut into.  Products of few tokens are bound by reading the weight, which wants nearly
// every SM reading; they pay for each further range with the last block's sum over the ranges.  So: the fewest ranges that
// put an item on about seven SMs in eight, in one wave of resident blocks.  (Measured on 4096 x 4096, 6144 x 4096 and
// 4096 x 12288 weights at 16 to 512 tokens: within 5% of the best cut.)  Beyond 1,024 tokens there are tiles enough.
int choose_splits(int M, int tiles, int k_blocks, int slots, long long workspace_floats, int tile_floats) {
    if (M > 1024 || tiles * 4 > 4096) return 1;
    constexpr int kMinBlocks = 4;
    const int target = sm_count() * 7 / 8;
    int splits = (target + tiles - 1) / tiles;
    if (splits > 8) splits = 8;
    while (splits > 1 && (k_blocks / splits < kMinBlocks || tiles * splits > slots ||
                          static_cast<long long>(tiles) * splits * tile_floats > workspace_floats))
        --splits;
    return splits;
}

struct SplitPlan {
    int splits;              // 0: choose
    float* workspace;
    long long workspace_floats;
    int* tickets;            // 4096 ints, zero between launches
    int cluster;             // 0: the ranges of a tile meet in the workspace even where a cluster could be formed
};

template <int BN, typename TOut, bool Gated>
int launch(const CUtensorMap& weight_map, const CUtensorMap& input_map, const float* bias, void* out, int M, int N, int K,
           long long out_stride, const SplitPlan& plan, cudaStream_t stream) {
    constexpr int stage_bytes = (BM + BN) * BK * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(gemm_tc_kernel<BN, TOut, Gated>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  static_cast<int>(sizeof(Shared)) + 1024 + 200 * 1024);
        if (status != cudaSuccess) return static_cast<int>(status);
        configured = true;
    }
    const int tiles = ((N + BM - 1) / BM) * ((M + BN - 1) / BN);
    const int k_blocks = (K + BK - 1) / BK;
    const int slots = sm_count() * blocks_per_sm<BN>();
    int splits = 1;
    if (plan.workspace && plan.tickets) {
        if (plan.splits == 0) {
            splits = choose_splits(M, tiles, k_blocks, slots, plan.workspace_floats, BN * BM);
        } else {
            splits = plan.splits;
            if (splits > 1 && (splits > k_blocks || static_cast<long long>(tiles) * splits * (BN * BM) > plan.workspace_floats || tiles * 4 > 4096))
                return cudaErrorInvalidValue;
        }
    } else if (plan.splits > 1) {
        return cudaErrorInvalidValue;
    }
    const int items = tiles * splits;
    const int blocks = items < slots ? items : slots;
    // With at most one block per SM, a block takes the whole SM's shared memory for stages: more bytes on their way
    // (the 6144 x 4096 product at 128 tokens: 18.9 us against 23.5 us).
    bool roomy = blocks <= sm_count();
    auto shared_for = [&](bool whole_sm, int* stage_count) {
        int count = (whole_sm ? 200 * 1024 : stage_budget<BN>()) / stage_bytes;
        if (count > 8) count = 8;
        *stage_count = count;
        return static_cast<int>(sizeof(Shared)) + 1024 + count * stage_bytes;
    };
    int stages = 0;
    int shared_bytes = shared_for(roomy, &stages);
    // All items resident at once: the ranges of a tile form a cluster and meet in shared memory.  A cluster is placed
    // inside one GPC, so fewer clusters fit than blocks alone would: 48 clusters of 3 whole-SM blocks did not fit the
    // 148 SMs and took two waves.  For whole-SM blocks the driver says how many clusters fit; half-SM blocks (for which
    // its answer was the same, though twice as many ran at once) are clustered while they fill at most three quarters
    // of their places.
    if (splits > 1 && splits <= 8 && items == blocks && plan.cluster != 0) {
        bool whole = false;
        if (roomy || blocks_per_sm<BN>() == 1) {
            static int fits[9] = {};   // clusters of whole-SM blocks of this size that are resident at once: 0 unknown, -1 no answer
            int& known = fits[splits];
            if (known == 0) {
                int whole_stages = 0;
                cudaLaunchConfig_t config = {};
                config.gridDim = dim3(blocks);
                config.blockDim = dim3(kThreads);
                config.dynamicSmemBytes = shared_for(true, &whole_stages);
                cudaLaunchAttribute attribute[1];
                attribute[0].id = cudaLaunchAttributeClusterDimension;
                attribute[0].val.clusterDim.x = splits;
                attribute[0].val.clusterDim.y = 1;
                attribute[0].val.clusterDim.z = 1;
                config.attrs = attribute;
                config.numAttrs = 1;
                int clusters = 0;
                known = cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_kernel<BN, TOut, Gated>, &config) == cudaSuccess && clusters > 0 ? clusters : -1;
                if (known < 0) cudaGetLastError();
            }
            whole = known >= tiles;
        }
        const bool half = !whole && blocks_per_sm<BN>() == 2 && items <= sm_count() * 2 * 3 / 4;
        if (whole || half) {
            int cluster_stages = 0;
            const int cluster_bytes = shared_for(whole, &cluster_stages);
            if (cluster_stages * stage_bytes >= BN * BM * 4) {   // the partial tile lies over the stages
                tau_launch_clusters(splits, gemm_tc_kernel<BN, TOut, Gated>, dim3(blocks), dim3(kThreads), cluster_bytes, stream, weight_map, input_map,
                                    bias, static_cast<TOut*>(out), M, N, K, out_stride, cluster_stages, splits, plan.workspace, plan.tickets, 1);
                return tau_launch_status();
            }
        }
    }
    tau_launch(gemm_tc_kernel<BN, TOut, Gated>, dim3(blocks), dim3(kThreads), shared_bytes, stream, weight_map, input_map, bias, static_cast<TOut*>(out), M, N, K,
               out_stride, stages, splits, plan.workspace, plan.tickets, 0);
    return tau_launch_status();
}

template <typename TOut, bool Gated>
int launch_pair(const CUtensorMap& weight_map, const CUtensorMap& input_map, const float* bias, void* out, int M, int N, int K,
                long long out_stride, cudaStream_t stream) {
    constexpr int stage_bytes = (kPairHalf + BM) * BK * 2;
    int stages = (200 * 1024) / stage_bytes;
    if (stages > 8) stages = 8;
    const int shared_bytes = sizeof(Shared) + 1024 + stages * stage_bytes + 4 * 4096;   // and the epilogue warps' staging rows
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(gemm_tc_pair_kernel<TOut, Gated>, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_bytes);
        if (status != cudaSuccess) return static_cast<int>(status);
        configured = true;
    }
    const int tiles = ((N + kPairFeatures - 1) / kPairFeatures) * ((M + kPairTokens - 1) / kPairTokens);
    const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
    // 16-byte stores need rows of the output that start on 16 bytes and whole groups of features inside N.
    const int group = Gated ? 16 : (sizeof(TOut) == 2 ? 8 : 4);
    const int vector_stores = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (out_stride * sizeof(TOut)) % 16 == 0 && N % group == 0;
    tau_launch_clusters(2, gemm_tc_pair_kernel<TOut, Gated>, dim3(2 * pairs), dim3(kThreads), shared_bytes, stream, weight_map, input_map, bias,
                        static_cast<TOut*>(out), M, N, K, out_stride, stages, vector_stores);
    return tau_launch_status();
}

template <typename TOut, bool Gated>
int dispatch(const CUtensorMap& weight_map, const CUtensorMap& input_map, int box, const float* bias, void* out, int M, int N, int K,
             long long out_stride, const SplitPlan& plan, cudaStream_t stream) {
    if (box == kPairHalf + 1) return launch_pair<TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, stream);
    switch (box) {
        case 16: return launch<16, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, plan, stream);
        case 32: return launch<32, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, plan, stream);
        case 64: return launch<64, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, plan, stream);
        case 128: return launch<128, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, plan, stream);
        case 192: return launch<192, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, plan, stream);
        default: return launch<256, TOut, Gated>(weight_map, input_map, bias, out, M, N, K, out_stride, plan, stream);
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
// `workspace` (`workspace_floats` floats) and `tickets` (4096 ints, zero, left at zero) allow cutting along K; `splits` = 0
// lets the launcher choose, 1 forbids it, more asks for exactly that many ranges (refused if they do not fit).
// `cluster`: 0 keeps the ranges of a tile from meeting in a cluster's shared memory (they meet in the workspace).
// `pair`: 1 runs 256 x 256 tiles on pairs of SMs (only with the 256-token tile), 0 never, -1 where the 256-token tile is chosen.
TAU_EXPORT int tau_gemm_tc(int out_dtype, const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                           long long x_stride, long long w_stride, long long out_stride, int token_box, int gated, int splits,
                           void* workspace, long long workspace_floats, void* tickets, int pair, int cluster, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!x || !w || !out || K <= 0 || (K & 7) || (x_stride & 7) || (w_stride & 7) || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (reinterpret_cast<uintptr_t>(w) & 15) || (out_dtype != TAU_BF16 && out_dtype != TAU_F32) || splits < 0)
        return cudaErrorInvalidValue;
    const SplitPlan plan{splits, static_cast<float*>(workspace), workspace_floats, static_cast<int*>(tickets), cluster};
    int box = token_box;
    if (box == 0) box = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if (box != 16 && box != 32 && box != 64 && box != 128 && box != 192 && box != 256) return cudaErrorInvalidValue;
    if (pair > 0 && (box != 256 || splits > 1)) return cudaErrorInvalidValue;
    bool paired = box == 256 && pair != 0 && splits <= 1;   // a cut along K is run on single SMs, whether asked for or chosen
    if (paired && pair < 0 && splits == 0 && workspace && tickets) {
        const int feature_tiles = (N + BM - 1) / BM, tiles = feature_tiles * ((M + 255) / 256);
        if (choose_splits(M, tiles, (K + BK - 1) / BK, sm_count(), workspace_floats, 256 * BM) > 1) {
            paired = false;
        } else if (token_box == 0 && M <= 1024 && ((N + 255) / 256) * ((M + 255) / 256) * 100 >= 54 * (sm_count() / 2)) {
            // Pairs of SMs (256 x 256 tiles) as soon as their tiles fill a good half of the pairs: from there on they beat every
            // tile on single SMs (a gated 24576 x 4096 product at 256 tokens: 53.7 us against 69.2 us in tiles of 128 tokens;
            // 6144 x 4096 at 1,024 tokens: 44.9 us against 51.5 us in tiles of 192), below it they leave too many SMs idle
            // (4096 x 12288 at 512 tokens, 32 tiles for 74 pairs: 62.7 us against 49.1 us).
        } else if (token_box == 0 && M <= 1024) {
            // Between the batches that are cut along K and the prompts that fill every SM several times, the token tile
            // decides how many SMs have work: 512 tokens of a 6144-feature product are 96 tiles of 256 tokens, but 144
            // of 192.  An estimate of waves x (tokens of a tile + a fixed part) picks among 256, 192 and 128.  Beyond 1,024
            // tokens the pairs always win (6,328 tokens of a gated 6144 x 1024 product: 195 us in tiles of 192 on single SMs).
            int best = 256;
            long long best_cost = 0;
            for (int candidate : {256, 192, 128}) {
                const long long count = static_cast<long long>(feature_tiles) * ((M + candidate - 1) / candidate);
                const long long cost = ((count + sm_count() - 1) / sm_count()) * (candidate + 64);
                if (candidate == 256 || cost < best_cost) { best = candidate; best_cost = cost; }
            }
            if (best != 256) {
                box = best;
                paired = false;
            }
        }
    }
    CUtensorMap weight_map, input_map;
    if (!make_map(&weight_map, w, N, K, w_stride, BM) || !make_map(&input_map, x, M, K, x_stride, paired ? kPairHalf : box)) return cudaErrorInvalidValue;
    if (paired) box = kPairHalf + 1;   // the dispatcher's mark for the paired kernel
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gated) return dispatch<bf16, true>(weight_map, input_map, box, bias, out, M, N, K, out_stride, plan, s);
    if (out_dtype == TAU_BF16) return dispatch<bf16, false>(weight_map, input_map, box, bias, out, M, N, K, out_stride, plan, s);
    return dispatch<float, false>(weight_map, input_map, box, bias, out, M, N, K, out_stride, plan, s);
}
