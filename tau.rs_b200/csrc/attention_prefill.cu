// Prefill attention in bfloat16: runs of new tokens of many sequences, causal, over the paged cache.
//
// Compiled for one head size (-DTAU_HEAD_DIM=...).  The reference materialises `repeat_kv`, the score matrix
// `[B, nq, T, S]` and an additive mask (crates/models/src/components/gated_attention.rs:449-473); this kernel
// keeps scores in registers with an online softmax (32-bit statistics, `key <= query position`,
// crates/models/src/qwen3_5_common/model.rs:154) and never writes them.
//
// A warp owns 16 consecutive query positions of one head; the 4 warps of a block take the query heads of one
// KV group (or neighbouring query tiles when the group is small) and share the key and value tiles, which
// cp.async brings into shared memory a few tiles ahead.  Products are mma.sync m16n8k16 with fragments read
// as 16-byte vectors: a thread's 16 bytes of a key row feed two score products (the head dimension is permuted
// inside chunks of 32, identically for queries and keys), probabilities go from the score fragments into the
// A operand of the second product, and value fragments are assembled from 16-byte row reads with byte
// permutes (output column `64 r + 8 n + j` is column slot `n` of tile `j` in round `r`).
//
// The keys of the step's own tokens are in the cache already (the prepare kernel wrote them), so a run that
// continues a cached prefix, a whole prompt and a single token are the same case.
#include "common.cuh"

#ifndef TAU_HEAD_DIM
#error "compile with -DTAU_HEAD_DIM=<multiple of 16 up to 256>"
#endif

namespace {

constexpr int D = TAU_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head_dim must be a multiple of 16 between 16 and 256");
constexpr int kWarps = 4;
constexpr int kTile = 16;                  // query positions per warp
constexpr int kQkChunks = (D + 31) / 32;
constexpr int kRounds = (D + 63) / 64;

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_bf16(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const unsigned*>(&pair);
}

constexpr int kKeyTile = 64;                       // keys per shared-memory tile: one cache page
constexpr int kChunksPerRow = D / 8;               // 16-byte chunks in a row of D bfloat16
constexpr bool kSwizzle = (kChunksPerRow % 8) == 0;
constexpr int kTileBytes = kKeyTile * D * 2;       // one tile of keys, or of values
constexpr int kStages = D <= 128 ? 3 : 2;
constexpr int kSharedBytes = kStages * 2 * kTileBytes;

// Chunk `chunk` of row `row` lies at this byte offset of a tile.  Rows are 2 D bytes apart; the chunk number is
// XORed with the row's low bits so that 8 rows read at the same chunk fall into 8 different bank groups.
__device__ __forceinline__ int tile_offset(int row, int chunk) {
    return row * (D * 2) + ((kSwizzle ? (chunk ^ (row & 7)) : chunk) << 4);
}

__device__ __forceinline__ void copy_async_16(void* destination, const void* source, bool real) {
    const unsigned address = static_cast<unsigned>(__cvta_generic_to_shared(destination));
    const int bytes = real ? 16 : 0;   // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(address), "l"(source), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Block `blockIdx.x` serves `tiles_per_block` neighbouring query tiles of one sequence and `heads_per_block`
// heads of KV head `blockIdx.y / passes`; warp w takes tile w / heads_per_block and head w % heads_per_block.
// Keys and values pass through shared memory in tiles of 64 (one cache page), `kStages` deep, copied with
// cp.async by all threads and read by every warp of the block.
__global__ void __launch_bounds__(kWarps * 32)
attention_prefill_kernel(const bf16* __restrict__ queries, const bf16* __restrict__ keys, const bf16* __restrict__ values,
                         bf16* __restrict__ out, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                         const int* __restrict__ page_rows, int page_stride, int page_tokens, int n_seqs, int n_heads, int n_kv_heads,
                         int heads_per_block, int passes, float scale, int window) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ __align__(128) uint8_t tiles[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tiles_per_block = kWarps / heads_per_block;
    const int group = n_heads / n_kv_heads;
    // Which sequence does this block belong to?  Blocks are numbered sequence by sequence; a block index beyond
    // the last sequence has nothing to do.
    int block = blockIdx.x, seq = 0, row0 = 0, n_new = 0;
    for (; seq < n_seqs; ++seq) {
        row0 = cu_seqlens[seq];
        n_new = cu_seqlens[seq + 1] - row0;
        const int blocks_here = (n_new + kTile * tiles_per_block - 1) / (kTile * tiles_per_block);
        if (block < blocks_here) {
            block = blocks_here - 1 - block;   // the last tiles have the most keys: they start first
            break;
        }
        block -= blocks_here;
    }
    if (seq >= n_seqs) return;   // the whole block leaves
    const int kv_head = blockIdx.y / passes, pass = blockIdx.y % passes;
    const int start = seq_start[seq];                                   // positions cached before this step
    const int tile = block * tiles_per_block + warp / heads_per_block;  // this warp's query tile within the sequence
    const int head_in_group = pass * heads_per_block + warp % heads_per_block;
    const bool active = tile * kTile < n_new && head_in_group < group;   // an idle warp still copies and synchronises
    const int head = kv_head * group + (active ? head_in_group : 0);
    const int position0 = start + tile * kTile;
    const int rows_here = active ? min(kTile, n_new - tile * kTile) : 0;
    const int last_position = position0 + rows_here - 1;               // of this warp
    // The block's range of keys: from the first key that its first tile may see to the last position of its last tile.
    const int block_position0 = start + block * tiles_per_block * kTile;
    const int block_last = start + min(n_new, (block + 1) * tiles_per_block * kTile) - 1;
    int block_first_key = 0;
    if (window > 0 && block_position0 - window + 1 > 0) block_first_key = block_position0 - window + 1;
    const int first_tile = block_first_key / kKeyTile, last_tile = block_last / kKeyTile;
    const int n_key_tiles = last_tile - first_tile + 1;
    const int* pages = page_rows + static_cast<size_t>(seq) * page_stride;
    const size_t head_stride = static_cast<size_t>(page_tokens) * D;

    auto issue_tile = [&](int index) {   // copies key tile `first_tile + index` into stage `index % kStages`
        if (index < n_key_tiles) {
            const int key_tile = first_tile + index;
            const size_t base = (static_cast<size_t>(pages[key_tile * kKeyTile / page_tokens]) * n_kv_heads + kv_head) * head_stride +
                                static_cast<size_t>((key_tile * kKeyTile) % page_tokens) * D;
            uint8_t* stage = tiles + (index % kStages) * 2 * kTileBytes;
            for (int item = threadIdx.x; item < kKeyTile * kChunksPerRow; item += kWarps * 32) {
                const int row = item / kChunksPerRow, chunk = item % kChunksPerRow;
                const bool real = key_tile * kKeyTile + row <= block_last;   // rows beyond the block's last position become zero
                const size_t source = base + static_cast<size_t>(row) * D + chunk * 8;
                copy_async_16(stage + tile_offset(row, chunk), keys + (real ? source : base), real);
                copy_async_16(stage + kTileBytes + tile_offset(row, chunk), values + (real ? source : base), real);
            }
        }
        copy_async_commit();   // an empty group keeps the count of groups in step with the tiles
    };

    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    uint4 q_lo[kQkChunks], q_hi[kQkChunks];
    {
        const bool lo_live = g < rows_here, hi_live = g + 8 < rows_here;
        const bf16* base = queries + (static_cast<size_t>(row0 + (active ? tile * kTile : 0)) * n_heads + head) * D;
        const size_t row_stride = static_cast<size_t>(n_heads) * D;
#pragma unroll
        for (int c = 0; c < kQkChunks; ++c) {
            const int e = 32 * c + 8 * t;
            const bool inside = e + 8 <= D;
            q_lo[c] = (lo_live && inside) ? *reinterpret_cast<const uint4*>(base + g * row_stride + e) : zero4;
            q_hi[c] = (hi_live && inside) ? *reinterpret_cast<const uint4*>(base + (g + 8) * row_stride + e) : zero4;
        }
    }
    const float scale_log2 = scale * 1.4426950408889634f;
    const int position_lo = position0 + g, position_hi = position0 + g + 8;
    float max_lo = -INFINITY, max_hi = -INFINITY, sum_lo = 0.0f, sum_hi = 0.0f;
    float acc[kRounds][8][4];
#pragma unroll
    for (int r = 0; r < kRounds; ++r)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[r][j][i] = 0.0f;
    int warp_first_key = 0;
    if (window > 0 && position0 - window + 1 > 0) warp_first_key = position0 - window + 1;

#pragma unroll
    for (int index = 0; index < kStages - 1; ++index) issue_tile(index);

    for (int index = 0; index < n_key_tiles; ++index) {
        copy_async_wait<kStages - 2>();   // this thread's copies of tile `index` have landed
        __syncthreads();                  // ... and everyone's; and everyone is done with the stage refilled next
        issue_tile(index + kStages - 1);
        const uint8_t* key_tile = tiles + (index % kStages) * 2 * kTileBytes;
        const uint8_t* value_tile = key_tile + kTileBytes;
        const int tile_key0 = (first_tile + index) * kKeyTile;
        if (!active || tile_key0 > last_position || tile_key0 + kKeyTile <= warp_first_key) continue;   // nothing for this warp here
#pragma unroll 1
        for (int block16 = 0; block16 < kKeyTile / 16; ++block16) {
            const int base = tile_key0 + block16 * 16;
            if (base > last_position) break;
            if (base + 16 <= warp_first_key) continue;
            float score[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) score[nt][i] = 0.0f;
                const int row = block16 * 16 + 8 * nt + g;
#pragma unroll
                for (int c = 0; c < kQkChunks; ++c) {
                    // Every thread takes part in every product; a chunk beyond the head contributes zeros.
                    const uint4 k = (32 * c + 8 * t + 8 <= D) ? *reinterpret_cast<const uint4*>(key_tile + tile_offset(row, 4 * c + t)) : zero4;
                    mma_bf16(score[nt], q_lo[c].x, q_hi[c].x, q_lo[c].y, q_hi[c].y, k.x, k.y);
                    mma_bf16(score[nt], q_lo[c].z, q_hi[c].z, q_lo[c].w, q_hi[c].w, k.z, k.w);
                }
            }
            // score[nt][0..1]: row g, keys base + 8 nt + 2t + {0, 1}; score[nt][2..3]: row g + 8, the same keys.
            float block_lo = -INFINITY, block_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = base + 8 * nt + 2 * t + e;
                    const bool lo_ok = key <= position_lo && (window == 0 || key > position_lo - window);
                    const bool hi_ok = key <= position_hi && (window == 0 || key > position_hi - window);
                    score[nt][e] = lo_ok ? score[nt][e] * scale_log2 : -INFINITY;
                    score[nt][2 + e] = hi_ok ? score[nt][2 + e] * scale_log2 : -INFINITY;
                    block_lo = fmaxf(block_lo, score[nt][e]);
                    block_hi = fmaxf(block_hi, score[nt][2 + e]);
                }
            block_lo = fmaxf(block_lo, __shfl_xor_sync(0xffffffffu, block_lo, 1));
            block_lo = fmaxf(block_lo, __shfl_xor_sync(0xffffffffu, block_lo, 2));
            block_hi = fmaxf(block_hi, __shfl_xor_sync(0xffffffffu, block_hi, 1));
            block_hi = fmaxf(block_hi, __shfl_xor_sync(0xffffffffu, block_hi, 2));
            // A row that has seen no key yet keeps its maximum at -inf; subtract 0 then, so that nothing becomes NaN.
            const float new_lo = fmaxf(max_lo, block_lo), new_hi = fmaxf(max_hi, block_hi);
            const float shift_lo = new_lo == -INFINITY ? 0.0f : new_lo, shift_hi = new_hi == -INFINITY ? 0.0f : new_hi;
            const float correction_lo = exp2f(max_lo - shift_lo), correction_hi = exp2f(max_hi - shift_hi);
            max_lo = new_lo;
            max_hi = new_hi;
            float p[2][4];
            float share_lo = 0.0f, share_hi = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    p[nt][e] = exp2f(score[nt][e] - shift_lo);
                    p[nt][2 + e] = exp2f(score[nt][2 + e] - shift_hi);
                    share_lo += p[nt][e];
                    share_hi += p[nt][2 + e];
                }
            sum_lo = sum_lo * correction_lo + share_lo;
            sum_hi = sum_hi * correction_hi + share_hi;
            const unsigned pa0 = pack_bf16(p[0][0], p[0][1]), pa1 = pack_bf16(p[0][2], p[0][3]);
            const unsigned pa2 = pack_bf16(p[1][0], p[1][1]), pa3 = pack_bf16(p[1][2], p[1][3]);
            const int value_row = block16 * 16 + 2 * t;   // keys 2t, 2t+1, 2t+8, 2t+9 of the block
#pragma unroll
            for (int r = 0; r < kRounds; ++r) {
                {
                    const bool inside = 64 * r + 8 * g + 8 <= D;   // columns beyond the head are zeros; the products still run
                    const uint4 v0 = inside ? *reinterpret_cast<const uint4*>(value_tile + tile_offset(value_row, 8 * r + g)) : zero4;
                    const uint4 v1 = inside ? *reinterpret_cast<const uint4*>(value_tile + tile_offset(value_row + 1, 8 * r + g)) : zero4;
                    const uint4 v8 = inside ? *reinterpret_cast<const uint4*>(value_tile + tile_offset(value_row + 8, 8 * r + g)) : zero4;
                    const uint4 v9 = inside ? *reinterpret_cast<const uint4*>(value_tile + tile_offset(value_row + 9, 8 * r + g)) : zero4;
                    const unsigned* k0 = reinterpret_cast<const unsigned*>(&v0);
                    const unsigned* k1 = reinterpret_cast<const unsigned*>(&v1);
                    const unsigned* k8 = reinterpret_cast<const unsigned*>(&v8);
                    const unsigned* k9 = reinterpret_cast<const unsigned*>(&v9);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const unsigned selector = (j & 1) ? 0x7632u : 0x5410u;
                        const unsigned b0 = __byte_perm(k0[j >> 1], k1[j >> 1], selector);
                        const unsigned b1 = __byte_perm(k8[j >> 1], k9[j >> 1], selector);
                        acc[r][j][0] *= correction_lo;
                        acc[r][j][1] *= correction_lo;
                        acc[r][j][2] *= correction_hi;
                        acc[r][j][3] *= correction_hi;
                        mma_bf16(acc[r][j], pa0, pa1, pa2, pa3, b0, b1);
                    }
                }
            }
        }
    }
    copy_async_wait<0>();
    if (!active) return;
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    const float inverse_lo = 1.0f / sum_lo, inverse_hi = 1.0f / sum_hi;
    bf16* out_base = out + (static_cast<size_t>(row0 + tile * kTile) * n_heads + head) * D;
    const size_t row_stride = static_cast<size_t>(n_heads) * D;
    // acc[r][j][0], [1]: row g, columns 64 r + 16 t + j and + 8; [2], [3]: row g + 8, the same columns.
#pragma unroll
    for (int r = 0; r < kRounds; ++r)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c0 = 64 * r + 16 * t + j, c1 = c0 + 8;
            if (g < rows_here) {
                if (c0 < D) out_base[g * row_stride + c0] = __float2bfloat16_rn(acc[r][j][0] * inverse_lo);
                if (c1 < D) out_base[g * row_stride + c1] = __float2bfloat16_rn(acc[r][j][1] * inverse_lo);
            }
            if (g + 8 < rows_here) {
                if (c0 < D) out_base[(g + 8) * row_stride + c0] = __float2bfloat16_rn(acc[r][j][2] * inverse_hi);
                if (c1 < D) out_base[(g + 8) * row_stride + c1] = __float2bfloat16_rn(acc[r][j][3] * inverse_hi);
            }
        }
}

}  // namespace

TAU_EXPORT int tau_attention_prefill_head_dim() { return D; }

// `max_blocks`: an upper bound of sum over sequences of ceil(new tokens / (16 * tiles per block)), from the host.
TAU_EXPORT int tau_attention_prefill(const void* queries, const void* keys, const void* values, void* out, const int* cu_seqlens,
                                     const int* seq_start, const int* page_rows, int page_stride, int page_tokens, int n_seqs,
                                     int n_tokens, int n_heads, int n_kv_heads, float scale, int window, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (!queries || !keys || !values || !out || !cu_seqlens || !seq_start || !page_rows || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads != 0 || page_tokens <= 0 || window < 0)
        return cudaErrorInvalidValue;
    const int group = n_heads / n_kv_heads;
    const int heads_per_block = group >= 4 ? 4 : group == 3 ? 2 : group;     // 1, 2 or 4: divides the 4 warps
    const int passes = (group + heads_per_block - 1) / heads_per_block;
    const int tiles_per_block = kWarps / heads_per_block;
    const int rows_per_block = kTile * tiles_per_block;
    const int blocks = (n_tokens + rows_per_block - 1) / rows_per_block + n_seqs;   // every sequence may leave a ragged block
    const dim3 grid(blocks, n_kv_heads * passes);
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedBytes);
        if (status != cudaSuccess) return static_cast<int>(status);
        configured = true;
    }
    tau_launch(attention_prefill_kernel, dim3(grid), dim3(kWarps * 32), kSharedBytes, static_cast<cudaStream_t>(stream), 
        static_cast<const bf16*>(queries), static_cast<const bf16*>(keys), static_cast<const bf16*>(values), static_cast<bf16*>(out),
        cu_seqlens, seq_start, page_rows, page_stride, page_tokens, n_seqs, n_heads, n_kv_heads, heads_per_block, passes, scale, window);
    return tau_launch_status();
}
