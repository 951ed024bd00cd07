// Prefill attention on the fifth-generation tensor cores: bfloat16, causal, runs of new tokens over the paged cache.
//
// Compiled for one head size (-DTAU_HEAD_DIM=64 or 128).  The reference materialises the score matrix and an additive
// mask (crates/models/src/components/gated_attention.rs:449-473); here a block owns 128 query positions of one head,
// walks the keys in tiles of 64 (one cache page), and keeps both accumulators in tensor memory:
//
//   S = Q K^T     tcgen05.mma, A = Q tile and B = key tile from shared memory (both K-major, 128-byte swizzle, by TMA)
//   softmax       four warps, one query row per thread: tcgen05.ld of the row, mask (`key <= query position`,
//                 crates/models/src/qwen3_5_common/model.rs:154), running maximum and sum in 32-bit, probabilities
//                 rounded to bfloat16 and written to shared memory in the swizzled K-major layout
//   O += P V      tcgen05.mma, A = P from shared memory, B = value tile as it lies (`[key][d]`, MN-major)
//
// The accumulator O is rescaled only when a row's maximum has grown by more than 2^8 since the last rescale, so most
// tiles do not touch it; the final division by the row sum makes the result exact either way.  The score products run
// one tile ahead of the softmax (two score buffers in tensor memory), so the tensor cores work on tile i + 1 and on the
// second product of tile i - 1 while the four warps are busy with tile i; two blocks share an SM (96 KB of shared memory
// and 256 columns of tensor memory each) and fill each other's gaps.  Blocks are numbered with the heads fastest and the
// last query tiles first, so that the tiles with the most keys start first on every head.
// Six warps: four for the softmax (one per 32-lane quarter of tensor memory), one TMA producer, one MMA issuer.  Every
// mbarrier wait is bounded: after about two seconds the waiter raises an error flag, every role leaves its loop, tensor
// memory is freed and the kernel returns (`tau_attention_prefill_tc_status`).
#include <cuda.h>

#include "common.cuh"

#ifndef TAU_HEAD_DIM
#error "compile with -DTAU_HEAD_DIM=64 or 128"
#endif

namespace {

constexpr int D = TAU_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tensor-core prefill kernel serves head sizes 64 and 128");
constexpr int BM = 128;                 // query rows per block
constexpr int BN = 64;                  // keys per tile: one cache page
constexpr int kHalves = D / 64;         // 64-element (128-byte) slices of the head dimension
constexpr int kThreads = 192;
constexpr int kQBytes = BM * D * 2;
constexpr int kKeyBytes = BN * D * 2;   // a key tile, or a value tile
#ifndef TAU_ATTN_KEY_STAGES
#define TAU_ATTN_KEY_STAGES 2
#endif
constexpr int kKeyStages = TAU_ATTN_KEY_STAGES;   // key tiles in flight: a key tile is free as soon as its scores are done
constexpr int kValueStages = 2;                   // value tiles in flight: free when the second product of their tile is done
// Shared memory: Q, the key ring, the value ring, then the barriers; nothing is spent on aligning the tiles (dynamic
// shared memory starts at a multiple of 1,024 bytes, which the kernel checks before it does anything else), so that
// even three key stages at head size 128 (112 KB + 136 bytes) leave room for two blocks per SM.  A third key stage
// changed nothing (47.5 us against 47.4 us at 2,048 tokens, 514 against 509 us at 8,192): the keys are not what the
// tensor core waits for.
constexpr uint32_t kColumns = 256;      // two score buffers in columns [0, 64) and [64, 128), O in columns [128, 128 + D);
                                        // the probabilities of a tile (bfloat16 pairs, 32 columns) take the place of its scores
constexpr uint32_t kOColumn = 128;
constexpr float kRescaleThreshold = 8.0f;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

__device__ int attention_tc_error = 0;

__device__ __forceinline__ uint32_t smem_address(const void* pointer) { return static_cast<uint32_t>(__cvta_generic_to_shared(pointer)); }

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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"   // may sleep up to the hint before it answers
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_address(barrier)), "r"(parity), "r"(20000u)
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
                atomicExch(&attention_tc_error, 1);
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

// K-major tile, rows of 128 bytes, 128-byte swizzle: groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t k_major_descriptor(uint32_t address) {
    return static_cast<uint64_t>((address >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major tile (the value tile `[key][d]`): 128-byte rows hold 64 consecutive d of one key; groups of 8 keys are
// 1024 bytes apart (stride offset); the next 64 d lie `kKeyBytes / kHalves` bytes further (leading offset).
__device__ __forceinline__ uint64_t mn_major_descriptor(uint32_t address) {
    constexpr uint64_t leading = (kKeyBytes / kHalves) >> 4;
    return static_cast<uint64_t>((address >> 4) & 0x3fffu) | (leading << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// float accumulate, bfloat16 operands, M = 128, N = n; `b_mn_major` marks the B operand as MN-major.
__device__ __forceinline__ uint32_t instruction_descriptor(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(BM >> 4) << 24);
}
__device__ __forceinline__ void mma_issue(uint32_t accumulator, uint64_t a, uint64_t b, uint32_t descriptor, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(accumulator), "l"(a), "l"(b), "r"(descriptor), "r"(accumulate)
        : "memory");
}
// The same with the A operand in tensor memory (lane = row, a column holds two neighbouring bfloat16 of K).
__device__ __forceinline__ void mma_issue_from_tensor(uint32_t accumulator, uint32_t a, uint64_t b, uint32_t descriptor, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(accumulator), "r"(a), "l"(b), "r"(descriptor), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* barrier) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_address(barrier)) : "memory");
}
__device__ __forceinline__ void tensor_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tensor_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Starts a load of 32 columns of this thread's lane; see tensor_load_wait.
__device__ __forceinline__ void tensor_load_32(uint32_t address, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address));
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The values of earlier tensor_load_32 calls may be used only after this.
__device__ __forceinline__ void tensor_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tensor_store_32(uint32_t address, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(address), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tensor_store_words_32(uint32_t address, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
          "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
          "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 2^x on the special-function unit, one instruction (inputs here are <= 8 or -inf; tiny results may flush to zero).
__device__ __forceinline__ float fast_exp2(float value) {
    float result;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(result) : "f"(value));
    return result;
}

// Two 32-bit floats in one 64-bit register for the packed arithmetic of sm_100 (one instruction, two results): the softmax
// warps are bound by the instructions they issue, and half of a row's scalings and sums are instructions saved.
typedef unsigned long long Float2;
__device__ __forceinline__ Float2 pair_of(float low, float high) {
    Float2 pair;
    asm("mov.b64 %0, {%1, %2};" : "=l"(pair) : "f"(low), "f"(high));
    return pair;
}
__device__ __forceinline__ void unpair(Float2 pair, float& low, float& high) { asm("mov.b64 {%0, %1}, %2;" : "=f"(low), "=f"(high) : "l"(pair)); }
__device__ __forceinline__ Float2 fma_pair(Float2 a, Float2 b, Float2 c) {
    Float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ Float2 add_pair(Float2 a, Float2 b) {
    Float2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max_of_three(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ unsigned pack_bf16(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const unsigned*>(&pair);
}

struct Shared {
    uint64_t q_full;
    uint64_t k_full[kKeyStages];    // a key tile has landed
    uint64_t v_full[kValueStages];  // a value tile has landed
    uint64_t k_free[kKeyStages];    // the first product that read a key tile has finished
    uint64_t v_free[kValueStages];  // the second product that read a value tile has finished
    uint64_t s_full[2];             // scores of a tile are in their buffer of tensor memory
    uint64_t s_free[2];             // the softmax has read that buffer
    uint64_t p_ready[2];            // probabilities of a tile are in tensor memory (and O has been rescaled if need be)
    uint64_t pv_done;               // the second product of a tile has finished
    uint32_t tensor_memory_base;
    int abort_flag;
};

__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                            const __grid_constant__ CUtensorMap v_map, bf16* __restrict__ out, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_start, const int* __restrict__ page_rows, int page_stride, int n_seqs,
                            int n_heads, int n_kv_heads, float scale, int window) {
    extern __shared__ uint8_t shared_raw[];
    uint8_t* tiles = shared_raw;                                   // the swizzled tiles need 1,024-byte alignment
    uint8_t* q_tile = tiles;                                       // kHalves slices of [128 rows x 128 bytes]
    uint8_t* key_tiles = tiles + kQBytes;                          // kKeyStages key tiles
    uint8_t* value_tiles = key_tiles + kKeyStages * kKeyBytes;     // kValueStages value tiles
    Shared* shared = reinterpret_cast<Shared*>(value_tiles + kValueStages * kKeyBytes);
    if ((smem_address(shared_raw) & 1023u) != 0u) {   // never seen; the same for every thread, before anything is set up
        if (threadIdx.x == 0) atomicExch(&attention_tc_error, 2);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &shared->abort_flag;

    if (warp == 4 && lane == 0) {   // the descriptors of the three copies, on their way before the first copy asks for them
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&q_map)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&k_map)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&v_map)) : "memory");
    }
    if (threadIdx.x == 0) {
        barrier_init(&shared->q_full, 1);
        for (int s = 0; s < kKeyStages; ++s) {
            barrier_init(&shared->k_full[s], 1);
            barrier_init(&shared->k_free[s], 1);
        }
        for (int s = 0; s < kValueStages; ++s) {
            barrier_init(&shared->v_full[s], 1);
            barrier_init(&shared->v_free[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            barrier_init(&shared->s_full[b], 1);
            barrier_init(&shared->s_free[b], 4);     // one arrival per softmax warp
            barrier_init(&shared->p_ready[b], 4);
        }
        barrier_init(&shared->pv_done, 1);
        shared->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(&shared->tensor_memory_base)),
                     "r"(kColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tensor_fence_before_sync();
    __syncthreads();
    tensor_fence_after_sync();
    const uint32_t tensor_base = shared->tensor_memory_base;
    // The next kernel's blocks may start only now that this block holds its tensor memory: had one of them taken the
    // columns first, this block's allocation would wait for a kernel that waits for this one.
    grid_dependents_launch();
    grid_dependency_wait();

    // Which sequence and which 128-row tile of it?  Blocks are numbered sequence by sequence, last tiles first.
    int block = blockIdx.y, seq = 0, row0 = 0, n_new = 0;   // heads vary fastest, so the heaviest tiles of every head start first
    for (; seq < n_seqs; ++seq) {
        row0 = cu_seqlens[seq];
        n_new = cu_seqlens[seq + 1] - row0;
        const int blocks_here = (n_new + BM - 1) / BM;
        if (block < blocks_here) {
            block = blocks_here - 1 - block;
            break;
        }
        block -= blocks_here;
    }
    const bool has_work = seq < n_seqs;
    const int head = blockIdx.x, kv_head = head / (n_heads / n_kv_heads);
    const int start = has_work ? seq_start[seq] : 0;
    const int rows_here = has_work ? min(BM, n_new - block * BM) : 0;
    const int position0 = start + block * BM;                 // position of row 0
    const int last_position = position0 + rows_here - 1;      // of the last real row
    int first_key = 0;
    if (window > 0 && position0 - window + 1 > 0) first_key = position0 - window + 1;
    const int first_tile = first_key / BN;
    const int n_tiles = has_work ? last_position / BN - first_tile + 1 : 0;
    const int* pages = page_rows + static_cast<size_t>(has_work ? seq : 0) * page_stride;

    if (warp == 4) {
        // ---- producer -------------------------------------------------------------------------------------------
        if (lane == 0 && has_work) {
            barrier_expect_bytes(&shared->q_full, kQBytes);
            for (int half = 0; half < kHalves; ++half)
                tma_load_2d(q_tile + half * (BM * 128), &q_map, head * D + half * 64, row0 + block * BM, &shared->q_full);
            // The place of key tile i is free when the scores of tile i - kKeyStages are done, which is earlier than the place
            // of value tile i (free when the second product of tile i - kValueStages is done): keys are asked for ahead
            // of values, in the order in which their places come free.
            auto load_keys = [&](int i) {
                const int s = i % kKeyStages;
                const uint32_t use = i / kKeyStages;
                if (use > 0 && !barrier_wait(&shared->k_free[s], (use - 1) & 1u, abort_flag)) return false;
                const int row = (pages[first_tile + i] * n_kv_heads + kv_head) * BN;
                barrier_expect_bytes(&shared->k_full[s], kKeyBytes);
                for (int half = 0; half < kHalves; ++half)
                    tma_load_2d(key_tiles + s * kKeyBytes + half * (BN * 128), &k_map, half * 64, row, &shared->k_full[s]);
                return true;
            };
            auto load_values = [&](int i) {
                const int s = i % kValueStages;
                const uint32_t use = i / kValueStages;
                if (use > 0 && !barrier_wait(&shared->v_free[s], (use - 1) & 1u, abort_flag)) return false;
                const int row = (pages[first_tile + i] * n_kv_heads + kv_head) * BN;
                barrier_expect_bytes(&shared->v_full[s], kKeyBytes);
                for (int half = 0; half < kHalves; ++half)
                    tma_load_2d(value_tiles + s * kKeyBytes + half * (BN * 128), &v_map, half * 64, row, &shared->v_full[s]);
                return true;
            };
            // Completion order of the products: scores 0, scores 1, second product 0, scores 2, second product 1, ...; a
            // load is issued when the product that frees its place is the next to finish, so no wait blocks a later load
            // whose place is free already: keys run kAhead tiles ahead of values.
            constexpr int kAhead = kKeyStages - kValueStages + 1;
            bool alive = true;
            for (int i = 0; i < n_tiles + kAhead && alive; ++i) {
                if (i < n_tiles) alive = load_keys(i);
                if (alive && i >= kAhead) alive = load_values(i - kAhead);
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer -----------------------------------------------------------------------------------------
        if (lane == 0 && has_work) {
            const uint32_t score_descriptor = instruction_descriptor(BN, false), value_descriptor = instruction_descriptor(D, true);
            const uint32_t q_address = smem_address(q_tile);
            // Scores run one tile ahead of the softmax: while the four warps work on tile i, the products of tile i + 1
            // fill the other score buffer, and the second product of tile i follows as soon as its probabilities are there.
            auto issue_scores = [&](int i) {
                const int s = i % kKeyStages;
                const uint32_t key_address = smem_address(key_tiles + s * kKeyBytes);
                if (!barrier_wait(&shared->k_full[s], (i / kKeyStages) & 1u, abort_flag)) return false;
                // The buffer also held the probabilities of tile i - 2; their product was issued before this one and the
                // tensor core takes products in the order of issue, so only the softmax's read needs waiting for.
                if (i >= 2 && !barrier_wait(&shared->s_free[i & 1], ((i >> 1) - 1) & 1u, abort_flag)) return false;
                tensor_fence_after_sync();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t offset = (k / 4) * 128 * BM + (k % 4) * 32;          // slice of 64 d, then 16 d inside it
                    const uint32_t key_offset = (k / 4) * 128 * BN + (k % 4) * 32;
                    mma_issue(tensor_base + (i & 1) * BN, k_major_descriptor(q_address + offset),
                              k_major_descriptor(key_address + key_offset), score_descriptor, k > 0 ? 1u : 0u);
                }
                mma_commit(&shared->k_free[s]);
                mma_commit(&shared->s_full[i & 1]);
                return true;
            };
            bool alive = barrier_wait(&shared->q_full, 0, abort_flag) && issue_scores(0);
            for (int i = 0; i < n_tiles && alive; ++i) {
                if (i + 1 < n_tiles && !issue_scores(i + 1)) break;
                const int s = i % kValueStages;
                const uint32_t value_address = smem_address(value_tiles + s * kKeyBytes);
                if (!barrier_wait(&shared->v_full[s], (i / kValueStages) & 1u, abort_flag)) break;
                // Probabilities lie where the scores of the tile were: 16 keys are 8 columns.
                if (!barrier_wait(&shared->p_ready[i & 1], (i >> 1) & 1u, abort_flag)) break;
                tensor_fence_after_sync();
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {
                    mma_issue_from_tensor(tensor_base + kOColumn, tensor_base + (i & 1) * BN + k * 8, mn_major_descriptor(value_address + k * 2048),
                                          value_descriptor, (i > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(&shared->v_free[s]);
                mma_commit(&shared->pv_done);
            }
        }
    } else if (has_work) {
        // ---- softmax: thread = query row ----------------------------------------------------------------------------
        const int row = warp * 32 + lane;                         // warp w may touch lanes 32 w .. 32 w + 31 of tensor memory
        const uint32_t lane_base = tensor_base + (static_cast<uint32_t>(warp * 32) << 16);
        const int position = position0 + row;
        const float scale_log2 = scale * 1.4426950408889634f;
        float used_max = -INFINITY, sum = 0.0f;                   // the maximum that O and `sum` are scaled by
        bool alive = true;
        for (int i = 0; i < n_tiles && alive; ++i) {
            const int s = i % kValueStages;
            if (!barrier_wait(&shared->s_full[i & 1], (i >> 1) & 1u, abort_flag)) { alive = false; break; }
            tensor_fence_after_sync();
            float score[BN];
            {
                float low[32], high[32];
                tensor_load_32(lane_base + (i & 1) * BN, low);
                tensor_load_32(lane_base + (i & 1) * BN + 32, high);
                tensor_load_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    score[j] = low[j];
                    score[32 + j] = high[j];
                }
            }
            tensor_fence_before_sync();
            __syncwarp();
            if (lane == 0) barrier_arrive(&shared->s_free[i & 1]);
            const int key0 = (first_tile + i) * BN;
            if (key0 + BN - 1 > last_position) {
                // Rows of the page beyond the last position hold whatever an earlier sequence left there.  Their
                // probabilities are zero, but zero times a stale NaN is not: clear those value rows before the product.
                uint8_t* value_tile = value_tiles + s * kKeyBytes;
                const int first_stale = last_position - key0 + 1;
                if (!barrier_wait(&shared->v_full[s], (i / kValueStages) & 1u, abort_flag)) { alive = false; break; }   // the tile must have landed first
                for (int item = threadIdx.x; item < (BN - first_stale) * kHalves * 8; item += 128) {
                    const int chunk = item % 8, half = (item / 8) % kHalves, stale_row = first_stale + item / (8 * kHalves);
                    *reinterpret_cast<uint4*>(value_tile + half * (BN * 128) + stale_row * 128 + chunk * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            const bool needs_mask = key0 + BN - 1 > position0 || (window > 0 && key0 <= position0 + BM - 1 - window);
            if (needs_mask) {   // a diagonal tile (or a window's edge): keys [lowest, highest] of the tile are visible to this row
                const int highest = position - key0, lowest = window > 0 ? position - window + 1 - key0 : 0;
#pragma unroll
                for (int j = 0; j < BN; ++j) score[j] = (j <= highest && j >= lowest) ? score[j] : -INFINITY;
            }
            float partial_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < BN; j += 2) partial_max[(j >> 1) & 3] = max_of_three(partial_max[(j >> 1) & 3], score[j], score[j + 1]);
            // Of the raw scores; the scale is positive and is applied afterwards.
            float tile_max = fmaxf(fmaxf(partial_max[0], partial_max[1]), fmaxf(partial_max[2], partial_max[3]));
            tile_max *= scale_log2;
            // Rescale O and the sum only when the maximum has grown by more than the threshold (or nothing was kept yet).
            float shift = used_max;
            const bool grow = tile_max > used_max + kRescaleThreshold;     // true for the first key a row sees
            // The loads and stores of tensor memory are warp-wide, so the whole warp takes part if any of its rows grows.
            const bool rescale = grow && i > 0 && used_max != -INFINITY;
            // A wait on an mbarrier names a phase by its parity alone, so it tells apart only the phase in progress and the one
            // before it.  While this warp works on tile i the second products of the tiles up to i - 2 are done (the scores of
            // tile i were issued behind them) and that of tile i cannot have begun (it needs this warp's probabilities): the
            // barrier is in phase i - 1 or i, and a wait for phase i - 1 is safe.  After the last tile's probabilities are
            // handed over it may be in phase n - 2, n - 1 or n, which a wait for phase n - 1 cannot tell apart (in phase
            // n - 2 it would pass at once, before the last two products): so the last tile always waits for phase n - 2
            // first, which leaves n - 1 or n for the wait behind the loop.
            const bool last_tile = i == n_tiles - 1 && i > 0;
            if (__any_sync(0xffffffffu, rescale) || last_tile) {
                // O must not be touched while the second product of the tile before is still writing it.  Only here (and
                // at the last tile): a warp whose maxima have settled never waits for that product, and its exponentials
                // run beside it.
                if (!barrier_wait(&shared->pv_done, (i - 1) & 1u, abort_flag)) { alive = false; break; }
                tensor_fence_after_sync();
            }
            if (__any_sync(0xffffffffu, rescale)) {
                const float factor = rescale ? exp2f(used_max - tile_max) : 1.0f;
                sum *= factor;
                float part[32];
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    tensor_load_32(lane_base + kOColumn + c * 32, part);
                    tensor_load_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) part[j] *= factor;
                    tensor_store_32(lane_base + kOColumn + c * 32, part);
                }
            }
            if (grow) {
                used_max = tile_max;
                shift = tile_max;
            }
            const float subtract = shift == -INFINITY ? 0.0f : shift;   // a row that has seen no key yet
            // Probabilities: this row's 64 values as 32 pairs of bfloat16, written over the row's scores in tensor memory,
            // where the second product takes them as its A operand.
            uint32_t packed[BN / 2];
            Float2 partial_sum[4] = {pair_of(0.0f, 0.0f), pair_of(0.0f, 0.0f), pair_of(0.0f, 0.0f), pair_of(0.0f, 0.0f)};
            const Float2 scale_pair = pair_of(scale_log2, scale_log2), shift_pair = pair_of(-subtract, -subtract);
#pragma unroll
            for (int j = 0; j < BN; j += 2) {
                float x0, x1;
                unpair(fma_pair(pair_of(score[j], score[j + 1]), scale_pair, shift_pair), x0, x1);
                const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                partial_sum[(j >> 1) & 3] = add_pair(partial_sum[(j >> 1) & 3], pair_of(p0, p1));
                packed[j / 2] = pack_bf16(p0, p1);
            }
            {
                float low, high;
                unpair(add_pair(add_pair(partial_sum[0], partial_sum[1]), add_pair(partial_sum[2], partial_sum[3])), low, high);
                sum += low + high;
            }
            tensor_store_words_32(lane_base + (i & 1) * BN, packed);
            if (key0 + BN - 1 > last_position) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the cleared value rows, for the tensor core's reads
            tensor_fence_before_sync();
            __syncwarp();
            if (lane == 0) barrier_arrive(&shared->p_ready[i & 1]);
        }
        if (alive && n_tiles > 0 && barrier_wait(&shared->pv_done, (n_tiles - 1) & 1u, abort_flag)) {
            tensor_fence_after_sync();
            const float inverse = 1.0f / sum;
            // Every product is done, so the place of the Q tile is free: the rows go there as bfloat16 (16-byte pieces,
            // exchanged among a row's first eight by the row's number so that neighbouring rows fall into different
            // banks), and each warp then writes its own 32 rows with whole lines, 32 / (D / 8) rows to an instruction.  A
            // thread that wrote its row straight from its registers would touch 32 lines with every instruction.
            uint8_t* staging = q_tile + row * (D * 2);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                float part[32];
                tensor_load_32(lane_base + kOColumn + c * 32, part);   // every thread of the warp takes part in the load
                tensor_load_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const uint4 packed = make_uint4(pack_bf16(part[j] * inverse, part[j + 1] * inverse), pack_bf16(part[j + 2] * inverse, part[j + 3] * inverse),
                                                    pack_bf16(part[j + 4] * inverse, part[j + 5] * inverse), pack_bf16(part[j + 6] * inverse, part[j + 7] * inverse));
                    const int piece = c * 4 + j / 8;
                    *reinterpret_cast<uint4*>(staging + ((piece ^ (row & 7)) << 4)) = packed;
                }
            }
            __syncwarp();
            constexpr int kPieces = D / 8, kRowsAtOnce = 32 / kPieces;
            const int piece = lane % kPieces;
            uint4 line[32 / kRowsAtOnce];
#pragma unroll
            for (int step = 0; step < 32 / kRowsAtOnce; ++step) {
                const int r = warp * 32 + step * kRowsAtOnce + lane / kPieces;
                line[step] = *reinterpret_cast<const uint4*>(q_tile + r * (D * 2) + ((piece ^ (r & 7)) << 4));
            }
#pragma unroll
            for (int step = 0; step < 32 / kRowsAtOnce; ++step) {
                const int r = warp * 32 + step * kRowsAtOnce + lane / kPieces;
                if (r < rows_here)
                    *reinterpret_cast<uint4*>(out + (static_cast<size_t>(row0 + block * BM + r) * n_heads + head) * D + piece * 8) = line[step];
            }
        }
    }

    tensor_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tensor_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tensor_base), "r"(kColumns) : "memory");
    }
}

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

// A map over a row-major bfloat16 matrix `[rows, columns]`; boxes of `box_rows` rows by 64 columns (128 bytes), swizzled.
bool make_map(CUtensorMap* map, const void* base, long long rows, long long columns, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(columns), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(columns) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

TAU_EXPORT int tau_attention_prefill_tc_head_dim() { return D; }

// 0 if no wait has run out since the library was loaded (synchronises the device).
TAU_EXPORT int tau_attention_prefill_tc_status() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, attention_tc_error, sizeof(int)) != cudaSuccess) return -1;
    return flag;
}

// `n_pages`: pages of the cache layer (keys and values are `[n_pages, n_kv_heads, 64, D]`).
TAU_EXPORT int tau_attention_prefill_tc(const void* queries, const void* keys, const void* values, void* out, const int* cu_seqlens,
                                        const int* seq_start, const int* page_rows, int page_stride, int page_tokens, long long n_pages,
                                        int n_seqs, int n_tokens, int n_heads, int n_kv_heads, float scale, int window, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (!queries || !keys || !values || !out || !cu_seqlens || !seq_start || !page_rows || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads != 0 || page_tokens != BN || window < 0 || n_pages <= 0)
        return cudaErrorInvalidValue;
    CUtensorMap q_map, k_map, v_map;
    const long long cache_rows = n_pages * n_kv_heads * BN;
    if (cache_rows > 0x7fffffffLL) return cudaErrorInvalidValue;   // a tile's row is a 32-bit coordinate of the copy
    if (!make_map(&q_map, queries, n_tokens, static_cast<long long>(n_heads) * D, BM) || !make_map(&k_map, keys, cache_rows, D, BN) ||
        !make_map(&v_map, values, cache_rows, D, BN))
        return cudaErrorInvalidValue;
    const int shared_bytes = kQBytes + (kKeyStages + kValueStages) * kKeyBytes + static_cast<int>(sizeof(Shared));
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_bytes);
        if (status != cudaSuccess) return static_cast<int>(status);
        configured = true;
    }
    const int blocks = (n_tokens + BM - 1) / BM + n_seqs;   // every sequence may leave a ragged block
    tau_launch(attention_prefill_tc_kernel, dim3(n_heads, blocks), dim3(kThreads), shared_bytes, static_cast<cudaStream_t>(stream), q_map,
               k_map, v_map, static_cast<bf16*>(out), cu_seqlens, seq_start, page_rows, page_stride, n_seqs, n_heads, n_kv_heads, scale, window);
    return tau_launch_status();
}
