// Prefill attention on the fifth-generation tensor cores: bfloat16, causal, runs of new tokens over the paged cache.
//
// Compiled for one head size (-DTAU_HEAD_DIM=64 or 128).  The reference materialises the score matrix and an additive
// mask (crates/models/src/components/gated_attention.rs:449-473); here an item of work is 128 query positions of one
// head, whose keys are walked in tiles of 64 (one cache page), with both accumulators in tensor memory:
//
//   S = Q K^T     tcgen05.mma, A = Q tile and B = key tile from shared memory (both K-major, 128-byte swizzle, by TMA)
//   softmax       four warps, one query row per thread: tcgen05.ld of the row, mask (`key <= query position`,
//                 crates/models/src/qwen3_5_common/model.rs:154; a warp whose rows see all of a tile's keys skips it, one
//                 whose rows see none writes zeros), running maximum and sum in 32-bit, probabilities rounded to
//                 bfloat16 and written over the row's scores in tensor memory
//   O += P V      tcgen05.mma, A = P from tensor memory, B = value tile as it lies (`[key][d]`, MN-major)
//
// The accumulator O is rescaled only when a row's maximum has grown by more than 2^8 since the last rescale, so most
// tiles do not touch it; the final division by the row sum makes the result exact either way.  The score products run
// one tile ahead of the softmax (two score buffers in tensor memory), so the tensor cores work on tile i + 1 and on the
// second product of tile i - 1 while the four warps are busy with tile i; two blocks share an SM (96 KB of shared memory
// and 256 columns of tensor memory each) and fill each other's gaps.
// The blocks stay: as many as the device holds at once (two to an SM), each taking item after item off a counter in
// global memory.  Items are numbered with the heads fastest and, sequence by sequence, the last query tiles first, so the
// tiles with the most keys are begun first and the short ones fill the end, whichever block is free.  The tile, the
// barriers and tensor memory are set up once in a block's life; the next item's Q tile and first keys arrive while the
// last tile of the item before is still at work, and an item's output rows leave through the place of the value tiles:
// a whole tile as one bulk tensor store that the producer thread issues, a ragged one by the warps themselves.
// Six warps: four for the softmax (one per 32-lane quarter of tensor memory), one TMA producer, one MMA issuer.  Every
// mbarrier wait is bounded: after about two seconds the waiter raises an error flag, every role leaves its loops, tensor
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

// Writes a swizzled tile of shared memory to its place in global memory; the thread that issues it joins it to a group and
// may wait until the group's reads of shared memory are over.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int inner, int outer, const void* source) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(inner),
                 "r"(outer), "r"(smem_address(source))
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

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
__device__ __forceinline__ void tensor_load_words_16(uint32_t address, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(address));
}
// Sixteen columns of this thread's lane; `tensor_store_wait` before anyone else may read them.
__device__ __forceinline__ void tensor_store_words_16(uint32_t address, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(address),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
                 "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}
__device__ __forceinline__ void tensor_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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

// What a block works on next: 128 query rows of one head of one sequence.  The producer thread takes items off a counter in
// global memory and tells the other warps through two places in shared memory.
struct Item {
    int seq;          // -1: no items are left
    int row;          // the tile's first row among the step's tokens
    int rows_here;    // real rows of the tile (0: a place in the grid that holds no tile)
    int position0;    // position of its first row in the sequence
    int head;
};

struct Shared {
    uint64_t q_full;                // the Q tile of an item has landed
    uint64_t q_free;                // the last scores of an item are done: the place of its Q tile may be written
    uint64_t k_full[kKeyStages];    // a key tile has landed
    uint64_t v_full[kValueStages];  // a value tile has landed
    uint64_t k_free[kKeyStages];    // the first product that read a key tile has finished
    uint64_t v_free[kValueStages];  // the second product that read a value tile has finished
    uint64_t s_full[2];             // scores of a tile are in their buffer of tensor memory
    uint64_t s_free[2];             // the softmax has read that buffer
    uint64_t p_ready[2];            // probabilities of a tile are in tensor memory (and O has been rescaled if need be)
    uint64_t pv_done;               // the second product of a tile has finished
    uint64_t staged;                // the four softmax warps are done with the place of the value tiles: an item's output rows lie
                                    // there for the producer to send off (a whole tile), or have been written by the warps (a ragged one)
    uint64_t item_full[2];          // an item has been written to its place
    uint64_t item_free[2];          // the issuer and the four softmax warps have read it
    Item item[2];
    uint32_t tensor_memory_base;
    int abort_flag;
};

// The tiles of an item: which keys its rows see.
struct Span {
    int last_position, first_tile, n_tiles;
};
__device__ __forceinline__ Span span_of(const Item& item, int window) {
    Span span;
    span.last_position = item.position0 + item.rows_here - 1;   // of the last real row
    int first_key = 0;
    if (window > 0 && item.position0 - window + 1 > 0) first_key = item.position0 - window + 1;
    span.first_tile = first_key / BN;
    span.n_tiles = item.rows_here > 0 ? span.last_position / BN - span.first_tile + 1 : 0;
    return span;
}

__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                            const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap out_map, bf16* __restrict__ out,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start, const int* __restrict__ page_rows,
                            int page_stride, int n_seqs, int n_tokens, int n_heads, int n_kv_heads, float scale, int window, int n_items,
                            int* __restrict__ schedule) {
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
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&out_map)) : "memory");
    }
    if (threadIdx.x == 0) {
        barrier_init(&shared->q_full, 1);
        barrier_init(&shared->q_free, 1);
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
            barrier_init(&shared->item_full[b], 1);
            barrier_init(&shared->item_free[b], 5);  // the issuer and the four softmax warps
        }
        barrier_init(&shared->pv_done, 1);
        barrier_init(&shared->staged, 4);
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

    // Items are numbered with the heads fastest and, sequence by sequence, the last query tiles first: the tiles with the
    // most keys are taken first, and the short ones fill the end.
    // Every role walks the same list of items; `n` counts the items with work, `t` their tiles (for the barriers' phases).
    if (warp == 4) {
        // ---- producer -------------------------------------------------------------------------------------------
        if (lane == 0) {
            auto take = [&]() { return static_cast<int>(atomicAdd(schedule, 1)); };
            int scan_seq = 0, scan_tiles = 0;   // the sequence of the last item, and the tiles of the sequences before it
            // Writes item `number` (-1: the end) to its place, once those who read the item two before it are done with it.
            auto publish = [&](uint32_t k, int& number) {
                if (k >= 2 && !barrier_wait(&shared->item_free[k & 1], ((k >> 1) - 1) & 1u, abort_flag)) return false;
                Item item = {-1, 0, 0, 0, 0};
                if (number >= 0) {
                    // A block's items come in rising order, so the search for an item's sequence goes on where the last ended.
                    const int tile = number / n_heads;
                    int row0 = 0, n_new = 0;
                    for (; scan_seq < n_seqs; ++scan_seq) {
                        row0 = cu_seqlens[scan_seq];
                        n_new = cu_seqlens[scan_seq + 1] - row0;
                        const int tiles_here = (n_new + BM - 1) / BM;
                        if (tile - scan_tiles < tiles_here) break;
                        scan_tiles += tiles_here;
                    }
                    if (scan_seq < n_seqs) {
                        const int block = (n_new + BM - 1) / BM - 1 - (tile - scan_tiles);   // the last tiles of a sequence first
                        item.head = number % n_heads;
                        item.seq = scan_seq;
                        item.row = row0 + block * BM;
                        item.rows_here = min(BM, n_new - block * BM);
                        item.position0 = seq_start[scan_seq] + block * BM;
                    } else {
                        number = -1;   // behind the last tile (the launch counts a ragged tile for every sequence): so are all that follow
                    }
                }
                shared->item[k & 1] = item;
                barrier_arrive(&shared->item_full[k & 1]);   // a release: the item is written before the arrival shows
                return true;
            };
            uint32_t kt = 0, vt = 0, n = 0;   // key tiles, value tiles and items with work so far
            // The output rows of an item leave through the place of the value tiles when all its products are done.  A whole
            // tile (or one that ends with the step's last token, where the copy engine cuts it off) is sent by this thread
            // as soon as the four warps have put it there; the warps write a ragged tile themselves.  Either way the place
            // is free for value tiles afterwards.
            int sent_row = 0, sent_head = 0;
            bool sent_whole = false;
            auto send_rows = [&]() {   // of item n - 1
                if (!barrier_wait(&shared->staged, (n - 1) & 1u, abort_flag)) return false;
                if (sent_whole) {
                    for (int half = 0; half < kHalves; ++half)
                        tma_store_2d(&out_map, sent_head * D + half * 64, sent_row, value_tiles + half * (BM * 128));
                    tma_store_commit();
                    tma_store_wait_read();
                }
                return true;
            };
            int number = take();
            if (number >= n_items) number = -1;
            bool alive = publish(0, number);
            for (uint32_t k = 0; alive && number >= 0; ++k) {
                const Item item = shared->item[k & 1];
                const Span span = span_of(item, window);
                int next = -1;
                if (span.n_tiles > 0) {
                    const int kv_head = item.head / (n_heads / n_kv_heads);
                    const int* pages = page_rows + static_cast<size_t>(item.seq) * page_stride;
                    if (n > 0 && !barrier_wait(&shared->q_free, (n - 1) & 1u, abort_flag)) break;
                    barrier_expect_bytes(&shared->q_full, kQBytes);
                    for (int half = 0; half < kHalves; ++half)
                        tma_load_2d(q_tile + half * (BM * 128), &q_map, item.head * D + half * 64, item.row, &shared->q_full);
                    // The place of key tile i is free when the scores of the tile kKeyStages before it are done, which is
                    // earlier than the place of value tile i (free when the second product of the tile kValueStages
                    // before it is done): keys are asked for ahead of values, in the order in which their places come free.
                    auto load_keys = [&](int i) {
                        const int s = kt % kKeyStages;
                        const uint32_t use = kt / kKeyStages;
                        if (use > 0 && !barrier_wait(&shared->k_free[s], (use - 1) & 1u, abort_flag)) return false;
                        const int row = (pages[span.first_tile + i] * n_kv_heads + kv_head) * BN;
                        barrier_expect_bytes(&shared->k_full[s], kKeyBytes);
                        for (int half = 0; half < kHalves; ++half)
                            tma_load_2d(key_tiles + s * kKeyBytes + half * (BN * 128), &k_map, half * 64, row, &shared->k_full[s]);
                        ++kt;
                        return true;
                    };
                    auto load_values = [&](int i) {
                        const int s = vt % kValueStages;
                        const uint32_t use = vt / kValueStages;
                        if (use > 0 && !barrier_wait(&shared->v_free[s], (use - 1) & 1u, abort_flag)) return false;
                        if (i == 0 && n > 0 && !send_rows()) return false;   // the item before this one leaves first
                        const int row = (pages[span.first_tile + i] * n_kv_heads + kv_head) * BN;
                        barrier_expect_bytes(&shared->v_full[s], kKeyBytes);
                        for (int half = 0; half < kHalves; ++half)
                            tma_load_2d(value_tiles + s * kKeyBytes + half * (BN * 128), &v_map, half * 64, row, &shared->v_full[s]);
                        ++vt;
                        return true;
                    };
                    // Completion order of the products: scores 0, scores 1, second product 0, scores 2, second product 1, ...; a
                    // load is issued when the product that frees its place is the next to finish, so no wait blocks a later load
                    // whose place is free already: keys run kAhead tiles ahead of values.
                    constexpr int kAhead = kKeyStages - kValueStages + 1;
                    for (int i = 0; i < span.n_tiles + kAhead && alive; ++i) {
                        // The next item is taken when this one has a few tiles left: late, so that blocks which are done
                        // early find the items that remain, but early enough for the answer to be here at this item's end.
                        if (i == max(0, span.n_tiles - 4)) next = take();
                        if (i < span.n_tiles) alive = load_keys(i);
                        if (alive && i >= kAhead) alive = load_values(i - kAhead);
                    }
                    ++n;
                    sent_row = item.row, sent_head = item.head;
                    sent_whole = item.rows_here == BM || item.row + item.rows_here == n_tokens;
                }
                if (span.n_tiles == 0) next = take();
                if (next >= n_items) next = -1;
                alive = alive && publish(k + 1, next);
                number = next;
            }
            if (alive && n > 0) send_rows();   // the last item's
        }
    } else if (warp == 5) {
        // ---- MMA issuer -----------------------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t score_descriptor = instruction_descriptor(BN, false), value_descriptor = instruction_descriptor(D, true);
            const uint32_t q_address = smem_address(q_tile);
            uint32_t t = 0, n = 0;   // tiles and items with work so far
            // Scores run one tile ahead of the softmax: while the four warps work on tile i, the products of tile i + 1
            // fill the other score buffer, and the second product of tile i follows as soon as its probabilities are there.
            auto issue_scores = [&](uint32_t tile, bool last_of_item) {
                const int s = tile % kKeyStages;
                const uint32_t key_address = smem_address(key_tiles + s * kKeyBytes);
                if (!barrier_wait(&shared->k_full[s], (tile / kKeyStages) & 1u, abort_flag)) return false;
                // The buffer also held the probabilities of the tile two before; their product was issued before this one and
                // the tensor core takes products in the order of issue, so only the softmax's read needs waiting for.
                if (tile >= 2 && !barrier_wait(&shared->s_free[tile & 1], ((tile >> 1) - 1) & 1u, abort_flag)) return false;
                tensor_fence_after_sync();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t offset = (k / 4) * 128 * BM + (k % 4) * 32;          // slice of 64 d, then 16 d inside it
                    const uint32_t key_offset = (k / 4) * 128 * BN + (k % 4) * 32;
                    mma_issue(tensor_base + (tile & 1) * BN, k_major_descriptor(q_address + offset),
                              k_major_descriptor(key_address + key_offset), score_descriptor, k > 0 ? 1u : 0u);
                }
                mma_commit(&shared->k_free[s]);
                mma_commit(&shared->s_full[tile & 1]);
                if (last_of_item) mma_commit(&shared->q_free);
                return true;
            };
            bool alive = true;
            for (uint32_t k = 0; alive; ++k) {
                if (!barrier_wait(&shared->item_full[k & 1], (k >> 1) & 1u, abort_flag)) break;
                const Item item = shared->item[k & 1];
                barrier_arrive(&shared->item_free[k & 1]);
                if (item.seq < 0) break;
                const int n_tiles = span_of(item, window).n_tiles;
                if (n_tiles == 0) continue;
                alive = barrier_wait(&shared->q_full, n & 1u, abort_flag) && issue_scores(t, n_tiles == 1);
                for (int i = 0; i < n_tiles && alive; ++i) {
                    if (i + 1 < n_tiles && !issue_scores(t + i + 1, i + 2 == n_tiles)) { alive = false; break; }
                    const uint32_t tile = t + i;
                    const int s = tile % kValueStages;
                    const uint32_t value_address = smem_address(value_tiles + s * kKeyBytes);
                    if (!barrier_wait(&shared->v_full[s], (tile / kValueStages) & 1u, abort_flag)) { alive = false; break; }
                    // Probabilities lie where the scores of the tile were: 16 keys are 8 columns.  The first tile of an item
                    // overwrites O: its probabilities come from the warps that have read the item before's O by then.
                    if (!barrier_wait(&shared->p_ready[tile & 1], (tile >> 1) & 1u, abort_flag)) { alive = false; break; }
                    tensor_fence_after_sync();
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk) {
                        mma_issue_from_tensor(tensor_base + kOColumn, tensor_base + (tile & 1) * BN + kk * 8,
                                              mn_major_descriptor(value_address + kk * 2048), value_descriptor, (i > 0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(&shared->v_free[s]);
                    mma_commit(&shared->pv_done);
                }
                t += n_tiles;
                ++n;
            }
        }
    } else {
        // ---- softmax: thread = query row ----------------------------------------------------------------------------
        const int row = warp * 32 + lane;                         // warp w may touch lanes 32 w .. 32 w + 31 of tensor memory
        const uint32_t lane_base = tensor_base + (static_cast<uint32_t>(warp * 32) << 16);
        const float scale_log2 = scale * 1.4426950408889634f;
        uint32_t t = 0;                                           // tiles so far
        bool alive = true;
        for (uint32_t k = 0; alive; ++k) {
            if (!barrier_wait(&shared->item_full[k & 1], (k >> 1) & 1u, abort_flag)) break;
            // The item stays in its place until this warp is done with it (the producer writes the item after the next
            // there, when its own work on the next is over), so the epilogue reads it again and the loop carries less.
            const volatile Item* item_place = &shared->item[k & 1];
            int n_tiles, first_tile, last_position, position0;
            {
                Item item;
                item.seq = item_place->seq, item.rows_here = item_place->rows_here, item.position0 = item_place->position0;
                if (item.seq < 0 || item.rows_here == 0) {
                    __syncwarp();
                    if (lane == 0) barrier_arrive(&shared->item_free[k & 1]);
                    if (item.seq < 0) break;
                    continue;
                }
                const Span span = span_of(item, window);
                n_tiles = span.n_tiles, first_tile = span.first_tile, last_position = span.last_position, position0 = item.position0;
            }
            const int position = position0 + row;
            float used_max = -INFINITY, sum = 0.0f;                   // the maximum that O and `sum` are scaled by
            for (int i = 0; i < n_tiles && alive; ++i) {
                const uint32_t tile = t + i;
                const int s = tile % kValueStages;
                if (!barrier_wait(&shared->s_full[tile & 1], (tile >> 1) & 1u, abort_flag)) { alive = false; break; }
                tensor_fence_after_sync();
                float score[BN];
                {
                    float low[32], high[32];
                    tensor_load_32(lane_base + (tile & 1) * BN, low);
                    tensor_load_32(lane_base + (tile & 1) * BN + 32, high);
                    tensor_load_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        score[j] = low[j];
                        score[32 + j] = high[j];
                    }
                }
                tensor_fence_before_sync();
                __syncwarp();
                if (lane == 0) barrier_arrive(&shared->s_free[tile & 1]);
                const int key0 = (first_tile + i) * BN;
                if (key0 + BN - 1 > last_position) {
                    // Rows of the page beyond the last position hold whatever an earlier sequence left there.  Their
                    // probabilities are zero, but zero times a stale NaN is not: clear those value rows before the product.
                    uint8_t* value_tile = value_tiles + s * kKeyBytes;
                    const int first_stale = last_position - key0 + 1;
                    if (!barrier_wait(&shared->v_full[s], (tile / kValueStages) & 1u, abort_flag)) { alive = false; break; }   // the tile must have landed first
                    for (int entry = threadIdx.x; entry < (BN - first_stale) * kHalves * 8; entry += 128) {
                        const int chunk = entry % 8, half = (entry / 8) % kHalves, stale_row = first_stale + entry / (8 * kHalves);
                        *reinterpret_cast<uint4*>(value_tile + half * (BN * 128) + stale_row * 128 + chunk * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                // Which of the tile's keys do this warp's 32 rows see?  All of them (no mask), some (a diagonal tile or a
                // window's edge: keys [lowest, highest] of the tile are visible to a row), or none.
                const int warp_first = position0 + warp * 32, warp_last = warp_first + 31;    // positions of the warp's rows
                const bool all_seen = key0 + BN - 1 <= warp_first && (window == 0 || key0 >= warp_last - window + 1);
                const bool none_seen = key0 > warp_last || (window > 0 && key0 + BN - 1 < warp_first - window + 1);
                if (!all_seen && !none_seen) {
                    const int highest = position - key0;
                    if (window > 0) {
                        const int lowest = position - window + 1 - key0;
#pragma unroll
                        for (int j = 0; j < BN; ++j) score[j] = (j <= highest && j >= lowest) ? score[j] : -INFINITY;
                    } else {
#pragma unroll
                        for (int j = 0; j < BN; ++j) score[j] = j <= highest ? score[j] : -INFINITY;
                    }
                }
                float tile_max = -INFINITY;
                if (!none_seen) {
                    float partial_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int j = 0; j < BN; j += 2) partial_max[(j >> 1) & 3] = max_of_three(partial_max[(j >> 1) & 3], score[j], score[j + 1]);
                    // Of the raw scores; the scale is positive and is applied afterwards.
                    tile_max = fmaxf(fmaxf(partial_max[0], partial_max[1]), fmaxf(partial_max[2], partial_max[3])) * scale_log2;
                }
                // Rescale O and the sum only when the maximum has grown by more than the threshold (or nothing was kept yet).
                float shift = used_max;
                const bool grow = tile_max > used_max + kRescaleThreshold;     // true for the first key a row sees
                // The loads and stores of tensor memory are warp-wide, so the whole warp takes part if any of its rows grows.
                const bool rescale = grow && i > 0 && used_max != -INFINITY;
                // A wait on an mbarrier names a phase by its parity alone, so it tells apart only the phase in progress and the one
                // before it.  While this warp works on tile t the second products of the tiles up to t - 2 are done (the scores of
                // tile t were issued behind them, or an earlier item's end waited for them) and that of tile t cannot have begun (it
                // needs this warp's probabilities): the barrier is in phase t - 1 or t, and a wait for phase t - 1 is safe.  After
                // an item's last probabilities are handed over it may be in phase t - 1, t or t + 1, which a wait for phase t
                // cannot tell apart (in phase t - 1 it would pass at once, before the last two products): so the last tile
                // always waits for phase t - 1 first, which leaves t or t + 1 for the wait behind the loop.
                const bool last_tile = i == n_tiles - 1 && i > 0;
                if (__any_sync(0xffffffffu, rescale) || last_tile) {
                    // O must not be touched while the second product of the tile before is still writing it.  Only here (and
                    // at the last tile): a warp whose maxima have settled never waits for that product, and its exponentials
                    // run beside it.
                    if (!barrier_wait(&shared->pv_done, (tile - 1) & 1u, abort_flag)) { alive = false; break; }
                    tensor_fence_after_sync();
                }
                if (__any_sync(0xffffffffu, rescale)) {
                    const float factor = rescale ? exp2f(used_max - tile_max) : 1.0f;
                    sum *= factor;
                    // Sixteen columns at a time: this happens in a row's first few tiles only, and the scores of the tile at
                    // hand wait in the registers meanwhile.
#pragma unroll 1
                    for (int c = 0; c < D / 16; ++c) {
                        uint32_t part[16];
                        tensor_load_words_16(lane_base + kOColumn + c * 16, part);
                        tensor_load_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) part[j] = __float_as_uint(__uint_as_float(part[j]) * factor);
                        tensor_store_words_16(lane_base + kOColumn + c * 16, part);
                        tensor_store_wait();
                    }
                }
                if (grow) {
                    used_max = tile_max;
                    shift = tile_max;
                }
                const float subtract = shift == -INFINITY ? 0.0f : shift;   // a row that has seen no key yet
                // Probabilities: this row's 64 values as 32 pairs of bfloat16, written over the row's scores in tensor memory,
                // where the second product takes them as its A operand.
                if (none_seen) {   // the rows of this warp lie before every key of the tile: nothing to add, zeros for the product
                    uint32_t zeros[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) zeros[j] = 0u;
                    tensor_store_words_16(lane_base + (tile & 1) * BN, zeros);
                    tensor_store_words_16(lane_base + (tile & 1) * BN + 16, zeros);
                } else {
                    Float2 partial_sum[4] = {pair_of(0.0f, 0.0f), pair_of(0.0f, 0.0f), pair_of(0.0f, 0.0f), pair_of(0.0f, 0.0f)};
                    const Float2 scale_pair = pair_of(scale_log2, scale_log2), shift_pair = pair_of(-subtract, -subtract);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {   // 32 keys are 16 columns
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            float x0, x1;
                            unpair(fma_pair(pair_of(score[half * 32 + j], score[half * 32 + j + 1]), scale_pair, shift_pair), x0, x1);
                            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                            partial_sum[(j >> 1) & 3] = add_pair(partial_sum[(j >> 1) & 3], pair_of(p0, p1));
                            packed[j / 2] = pack_bf16(p0, p1);
                        }
                        tensor_store_words_16(lane_base + (tile & 1) * BN + half * 16, packed);
                    }
                    float low, high;
                    unpair(add_pair(add_pair(partial_sum[0], partial_sum[1]), add_pair(partial_sum[2], partial_sum[3])), low, high);
                    sum += low + high;
                }
                tensor_store_wait();
                if (key0 + BN - 1 > last_position) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the cleared value rows, for the tensor core's reads
                tensor_fence_before_sync();
                __syncwarp();
                if (lane == 0) barrier_arrive(&shared->p_ready[tile & 1]);
            }
            t += n_tiles;
            if (!alive || !barrier_wait(&shared->pv_done, (t - 1) & 1u, abort_flag)) { alive = false; break; }
            tensor_fence_after_sync();
            const float inverse = 1.0f / sum;
            // Every product of the item is done, so the place of the value tiles is free (the next item's first value tile
            // waits for `staged`): the rows go there as bfloat16 in the layout of the copy engine's swizzled tiles (slices of
            // 64 elements, rows of 128 bytes, the 16-byte pieces of a row exchanged by the row's number, which also keeps
            // neighbouring rows out of each other's banks).  The producer thread sends a whole tile off; the warps write a
            // ragged one themselves, 32 / (D / 8) rows of whole lines to an instruction.
            {
                float part[2][32];
                tensor_load_32(lane_base + kOColumn, part[0]);
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    tensor_load_wait();
                    if (c + 1 < D / 32) tensor_load_32(lane_base + kOColumn + (c + 1) * 32, part[(c + 1) & 1]);   // on its way meanwhile
                    const float (&values)[32] = part[c & 1];
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        const uint4 packed = make_uint4(pack_bf16(values[j] * inverse, values[j + 1] * inverse), pack_bf16(values[j + 2] * inverse, values[j + 3] * inverse),
                                                        pack_bf16(values[j + 4] * inverse, values[j + 5] * inverse), pack_bf16(values[j + 6] * inverse, values[j + 7] * inverse));
                        const int piece = c * 4 + j / 8;
                        *reinterpret_cast<uint4*>(value_tiles + (piece >> 3) * (BM * 128) + row * 128 + (((piece & 7) ^ (row & 7)) << 4)) = packed;
                    }
                }
            }
            tensor_fence_before_sync();   // O has been read: the next item's first second product may overwrite it
            const int rows_here = item_place->rows_here, first_row = item_place->row, head = item_place->head;
            if (rows_here == BM || first_row + rows_here == n_tokens) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the rows, for the copy engine's reads
                __syncwarp();
                if (lane == 0) {
                    barrier_arrive(&shared->staged);
                    barrier_arrive(&shared->item_free[k & 1]);
                }
            } else {
                __syncwarp();
                constexpr int kPieces = D / 8, kRowsAtOnce = 32 / kPieces;
                const int piece = lane % kPieces;
                uint4 line[32 / kRowsAtOnce];
#pragma unroll
                for (int step = 0; step < 32 / kRowsAtOnce; ++step) {
                    const int r = warp * 32 + step * kRowsAtOnce + lane / kPieces;
                    line[step] = *reinterpret_cast<const uint4*>(value_tiles + (piece >> 3) * (BM * 128) + r * 128 + (((piece & 7) ^ (r & 7)) << 4));
                }
                // The next value tiles are written by the copy engine: this warp's reads come before its arrival.
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    barrier_arrive(&shared->staged);
                    barrier_arrive(&shared->item_free[k & 1]);
                }
                bf16* target = out + (static_cast<size_t>(first_row) * n_heads + head) * D + piece * 8;
#pragma unroll
                for (int step = 0; step < 32 / kRowsAtOnce; ++step) {
                    const int r = warp * 32 + step * kRowsAtOnce + lane / kPieces;
                    if (r < rows_here) *reinterpret_cast<uint4*>(target + static_cast<size_t>(r) * n_heads * D) = line[step];
                }
            }
        }
    }

    tensor_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tensor_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tensor_base), "r"(kColumns) : "memory");
    }
    // The block that leaves last puts the counters back to zero for the next launch.
    if (threadIdx.x == 0 && atomicAdd(schedule + 1, 1) == static_cast<int>(gridDim.x) - 1) {
        schedule[0] = 0;
        schedule[1] = 0;
        __threadfence();
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

// `n_pages`: pages of the cache layer (keys and values are `[n_pages, n_kv_heads, 64, D]`).  `schedule`: two integers at
// zero, which the kernel uses and puts back to zero; launches that share them must follow one another on one stream.
TAU_EXPORT int tau_attention_prefill_tc(const void* queries, const void* keys, const void* values, void* out, const int* cu_seqlens,
                                        const int* seq_start, const int* page_rows, int page_stride, int page_tokens, long long n_pages,
                                        int n_seqs, int n_tokens, int n_heads, int n_kv_heads, float scale, int window, int* schedule,
                                        void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (!queries || !keys || !values || !out || !cu_seqlens || !seq_start || !page_rows || !schedule || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads != 0 || page_tokens != BN || window < 0 || n_pages <= 0)
        return cudaErrorInvalidValue;
    CUtensorMap q_map, k_map, v_map, out_map;
    const long long cache_rows = n_pages * n_kv_heads * BN;
    if (cache_rows > 0x7fffffffLL) return cudaErrorInvalidValue;   // a tile's row is a 32-bit coordinate of the copy
    if (!make_map(&q_map, queries, n_tokens, static_cast<long long>(n_heads) * D, BM) || !make_map(&k_map, keys, cache_rows, D, BN) ||
        !make_map(&v_map, values, cache_rows, D, BN) || !make_map(&out_map, out, n_tokens, static_cast<long long>(n_heads) * D, BM))
        return cudaErrorInvalidValue;
    const int shared_bytes = kQBytes + (kKeyStages + kValueStages) * kKeyBytes + static_cast<int>(sizeof(Shared));
    static int places = 0;   // blocks that the device holds at once
    if (!places) {
        cudaError_t status = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_bytes);
        if (status != cudaSuccess) return static_cast<int>(status);
        // Two blocks to an SM: the kernel is compiled for that many (registers), tensor memory holds the columns of two,
        // and a block's shared memory (plus the kilobyte that the system keeps for each) fits twice.
        int device = 0, sms = 0, shared_per_sm = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            cudaDeviceGetAttribute(&shared_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, device) != cudaSuccess || sms <= 0)
            return cudaErrorInvalidValue;
        const int per_sm = shared_per_sm / (shared_bytes + 1024);
        if (per_sm < 1) return cudaErrorInvalidValue;
        places = sms * (per_sm < 2 ? per_sm : 2);   // tensor memory holds two blocks' columns
    }
    const long long items = (static_cast<long long>((n_tokens + BM - 1) / BM) + n_seqs) * n_heads;   // every sequence may leave a ragged tile
    if (items > 0x7fffffffLL) return cudaErrorInvalidValue;
    const int blocks = static_cast<int>(items < places ? items : places);
    tau_launch(attention_prefill_tc_kernel, dim3(blocks), dim3(kThreads), shared_bytes, static_cast<cudaStream_t>(stream), q_map, k_map, v_map,
               out_map, static_cast<bf16*>(out), cu_seqlens, seq_start, page_rows, page_stride, n_seqs, n_tokens, n_heads, n_kv_heads, scale,
               window, static_cast<int>(items), schedule);
    return tau_launch_status();
}
