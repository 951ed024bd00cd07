// Decode attention: one new token per sequence over its cached context, split along the context.
//
// Compiled for one head size and dtype (-DTAU_HEAD_DIM=..., -DTAU_DTYPE=0|1), so a model compiles the one
// variant it needs.  Reference counterpart: crates/cuda-kernels/src/kernels/decode_attention.cu:186-250
// (`attention`: grid (heads, splits), 32-bit dot per key, `* rsqrt(d)`, max, exp, sum, probabilities times V)
// and :255-278 (`combine_attention`: merge of the splits' (max, sum, context) records).  Here a block serves
// one KV head of one sequence and all the query heads of its group at once, so keys and values are read once
// for the group; lengths and page lists are per sequence and come from device memory, so one captured graph
// serves every step.
//
// grid (splits, n_kv_heads * passes, sequences); a pass covers up to 8 query heads of a group.
// Partial results go to scratch: o[seq][head][split][D] (not normalised) and ml[seq][head][split][2] (max, sum).
#include "common.cuh"

#ifndef TAU_HEAD_DIM
#error "compile with -DTAU_HEAD_DIM=<multiple of 16 up to 256>"
#endif
#ifndef TAU_DTYPE
#error "compile with -DTAU_DTYPE=0 (float32) or 1 (bfloat16)"
#endif

namespace {

constexpr int D = TAU_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head_dim must be a multiple of 16 between 16 and 256");
#if TAU_DTYPE == 1
typedef bf16 T;
constexpr int kVec = 8;   // elements per 16-byte load
#else
typedef float T;
constexpr int kVec = 4;
#endif
constexpr int kWarps = 4;
#if TAU_DTYPE == 1
__device__ __forceinline__ float exponential(float value) { return __expf(value); }
#else
__device__ __forceinline__ float exponential(float value) { return expf(value); }   // the 32-bit path keeps the accurate one
#endif
constexpr int PER = (D + 31) / 32;            // value columns per lane
constexpr bool kContiguous = (D % 32 == 0);   // lane owns PER neighbouring columns, else columns lane, lane + 32, ...

[[maybe_unused]] __device__ __forceinline__ void load_vec(const T* source, float (&out)[kVec]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(source);
#if TAU_DTYPE == 1
    const unsigned words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // a bfloat16 is the upper half of a float
        out[2 * i] = __uint_as_float(words[i] << 16);
        out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
#else
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
    out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
#endif
}

__device__ __forceinline__ int column_of(int lane, int i) { return kContiguous ? lane * PER + i : lane + 32 * i; }

[[maybe_unused]] __device__ __forceinline__ void load_columns(const T* row, int lane, float (&out)[PER]) {
    if constexpr (kContiguous && PER * sizeof(T) == 16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + lane * PER);
        const unsigned words[4] = {raw.x, raw.y, raw.z, raw.w};
#if TAU_DTYPE == 1
#pragma unroll
        for (int i = 0; i < 4; ++i) { out[2 * i] = __uint_as_float(words[i] << 16); out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u); }
#else
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = __uint_as_float(words[i]);
#endif
    } else if constexpr (kContiguous && PER * sizeof(T) == 8) {
        const uint2 raw = *reinterpret_cast<const uint2*>(row + lane * PER);
#if TAU_DTYPE == 1
        out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
        out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
#else
        out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
#endif
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = column_of(lane, i);
            out[i] = c < D ? to_float(row[c]) : 0.0f;
        }
    }
}

template <int GH>
__global__ void __launch_bounds__(kWarps * 32)
decode_partial_kernel(const T* __restrict__ queries, const T* __restrict__ keys, const T* __restrict__ values,
                      T* __restrict__ out, float* __restrict__ partial_o, float* __restrict__ partial_ml,
                      const int* __restrict__ seq_len, const int* __restrict__ page_rows, int page_stride, int page_tokens,
                      int n_heads, int n_kv_heads, int passes, float scale, int window, int splits) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ __align__(16) float q_shared[GH][D];
    __shared__ float merge_o[kWarps][GH][D];
    __shared__ float merge_ml[kWarps][GH][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x, seq = blockIdx.z;
    const int kv_head = blockIdx.y / passes, pass = blockIdx.y % passes;
    const int group = n_heads / n_kv_heads;
    const int head0 = kv_head * group + pass * GH;                      // first query head of this block
    const int heads_here = min(GH, group - pass * GH);                  // > 0 by construction of `passes`
    const int length = seq_len[seq];
    const int first = (window > 0 && length > window) ? length - window : 0;
    const int span = length - first;
    const int per_split = ((span + splits - 1) / splits + 31) / 32 * 32;
    const int lo = first + split * per_split;
    const int hi = min(length, lo + per_split);
    const size_t record = (static_cast<size_t>(seq) * n_heads + head0) * splits + split;   // + h * splits per head

    if (lo >= hi) {   // nothing for this split: an empty record
        if (splits > 1 && threadIdx.x < heads_here) {
            partial_ml[(record + static_cast<size_t>(threadIdx.x) * splits) * 2] = -INFINITY;
            partial_ml[(record + static_cast<size_t>(threadIdx.x) * splits) * 2 + 1] = 0.0f;
        }
        return;
    }
    for (int index = threadIdx.x; index < GH * D; index += kWarps * 32) {
        const int h = index / D, e = index % D;
        q_shared[h][e] = h < heads_here ? to_float(queries[(static_cast<size_t>(seq) * n_heads + head0 + h) * D + e]) * scale : 0.0f;
    }
    __syncthreads();

    const int* pages = page_rows + static_cast<size_t>(seq) * page_stride;
    const size_t head_stride = static_cast<size_t>(page_tokens) * D;
    float running_max[GH], running_sum[GH], acc[GH][PER];
#pragma unroll
    for (int h = 0; h < GH; ++h) {
        running_max[h] = -INFINITY;
        running_sum[h] = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[h][i] = 0.0f;
    }

    for (int start = lo + warp * 32; start < hi; start += kWarps * 32) {
        const int key = start + lane;
        const bool live = key < hi;
        float score[GH];
#pragma unroll
        for (int h = 0; h < GH; ++h) score[h] = 0.0f;
        if (live) {
            const int page = pages[key / page_tokens];
            const T* key_row = keys + (static_cast<size_t>(page) * n_kv_heads + kv_head) * head_stride +
                               static_cast<size_t>(key % page_tokens) * D;
#pragma unroll 4
            for (int e = 0; e < D; e += kVec) {
                float k[kVec];
                load_vec(key_row + e, k);
#pragma unroll
                for (int h = 0; h < GH; ++h) {
#pragma unroll
                    for (int i = 0; i < kVec; i += 4) {
                        const float4 q4 = *reinterpret_cast<const float4*>(&q_shared[h][e + i]);
                        score[h] = fmaf(k[i], q4.x, score[h]);
                        score[h] = fmaf(k[i + 1], q4.y, score[h]);
                        score[h] = fmaf(k[i + 2], q4.z, score[h]);
                        score[h] = fmaf(k[i + 3], q4.w, score[h]);
                    }
                }
            }
        }
        float weight[GH];
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            const float s = live ? score[h] : -INFINITY;
            const float new_max = fmaxf(running_max[h], warp_max(s));   // finite: lane 0 of the group is live
            const float correction = exponential(running_max[h] - new_max);
            weight[h] = live ? exponential(s - new_max) : 0.0f;
            running_sum[h] = running_sum[h] * correction + warp_sum(weight[h]);
            running_max[h] = new_max;
#pragma unroll
            for (int i = 0; i < PER; ++i) acc[h][i] *= correction;
        }
        const int count = min(32, hi - start);
        for (int j = 0; j < count; ++j) {
            const int key_j = start + j;
            const int page = pages[key_j / page_tokens];
            const T* value_row = values + (static_cast<size_t>(page) * n_kv_heads + kv_head) * head_stride +
                                 static_cast<size_t>(key_j % page_tokens) * D;
            float v[PER];
            load_columns(value_row, lane, v);
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                const float w = __shfl_sync(0xffffffffu, weight[h], j);
#pragma unroll
                for (int i = 0; i < PER; ++i) acc[h][i] = fmaf(w, v[i], acc[h][i]);
            }
        }
    }
    // Merge the warps.
#pragma unroll
    for (int h = 0; h < GH; ++h) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = column_of(lane, i);
            if (c < D) merge_o[warp][h][c] = acc[h][i];
        }
        if (lane == 0) {
            merge_ml[warp][h][0] = running_max[h];
            merge_ml[warp][h][1] = running_sum[h];
        }
    }
    __syncthreads();
    for (int index = threadIdx.x; index < heads_here * D; index += kWarps * 32) {
        const int h = index / D, c = index % D;
        float total_max = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) total_max = fmaxf(total_max, merge_ml[w][h][0]);
        float o = 0.0f, sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float factor = exponential(merge_ml[w][h][0] - total_max);   // 0 for a warp that saw no key
            o += merge_o[w][h][c] * factor;
            sum += merge_ml[w][h][1] * factor;
        }
        if (splits == 1) {
            out[(static_cast<size_t>(seq) * n_heads + head0 + h) * D + c] = from_float<T>(o / sum);
        } else {
            const size_t slot = record + static_cast<size_t>(h) * splits;
            partial_o[slot * D + c] = o;
            if (c == 0) {
                partial_ml[slot * 2] = total_max;
                partial_ml[slot * 2 + 1] = sum;
            }
        }
    }
}

#if TAU_DTYPE == 1
// ---- bfloat16: the same split on the tensor cores ----------------------------------------------------------
// A warp takes blocks of 16 keys and works on the transposed problem, so that the 16 rows of a product are keys (all
// of them real) and its 8 columns are the group's query heads: scores S^T = K Q^T are mma.sync m16n8k16 products
// whose A fragments are 16-byte loads of two key rows (8 consecutive elements each; a load feeds two products,
// which permutes the head dimension inside a chunk of 32 identically for keys and queries).  A thread then holds
// the scores of keys g and g + 8 for heads 2t and 2t + 1, keeps the running maximum and sum of its two heads
// itself, and turns its probabilities into the B fragment of the second product, O^T = V^T P, with two movmatrix
// transposes.  The A fragments of that product are assembled from 16-byte loads of value rows (one key, 8
// consecutive columns) with byte permutes: row g of tile i in round r is output column 64 r + 8 g + 2 i, row g + 8
// the column after it.  Accumulators are 4 registers per 16 output columns, half of what the untransposed form needs.
constexpr int kQkChunks = (D + 31) / 32;   // chunks of 32 head elements for the score products
constexpr int kRounds = (D + 63) / 64;     // rounds of 64 output columns

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_bf16(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const unsigned*>(&pair);
}

// What the fused form needs to prepare queries and the new key and value itself (decode_attention.cu:120-181 of the
// reference does this in a kernel of its own).  `projected == nullptr`: queries are ready and the cache is complete.
struct DecodePrepare {
    const bf16* projected;        // [sequences, (n_heads + 2 n_kv_heads) D] as the stacked projection left it
    long long projected_stride;
    const float* q_weight;        // per-head norm weights, or nullptr for no norm
    const float* k_weight;
    float eps;
    const float* cos_table;       // [positions, rotary_dim / 2], or nullptr
    const float* sin_table;
    int rotary_dim;
    int write_cache;              // 0: another run wrote this position's key and value already
};

// A lane's share of a position's rotation coefficients: elements lane, lane + 32, ... of the half-width tables.
constexpr int kRotationsPerLane = (D / 2 + 31) / 32;

// One warp: per-head norm (rounded to bfloat16), rotation of the first `rotary_dim` elements in 32-bit, rounded again.
__device__ __forceinline__ void prepare_head(const bf16* __restrict__ source, const float* __restrict__ weight, float eps,
                                             const float (&cosines)[kRotationsPerLane], const float (&sines)[kRotationsPerLane], int rotary_dim,
                                             bf16* __restrict__ target, int lane) {
    float inverse = 1.0f;
    if (weight) {
        float squares = 0.0f;
        for (int e = lane; e < D; e += 32) {
            const float value = __bfloat162float(source[e]);
            squares += value * value;
        }
        inverse = rsqrtf(warp_sum(squares) / static_cast<float>(D) + eps);
    }
    auto normalized = [&](int e) {
        const float value = __bfloat162float(source[e]);
        return weight ? __bfloat162float(__float2bfloat16_rn(value * inverse * weight[e])) : value;
    };
    const int half = rotary_dim / 2;
#pragma unroll
    for (int i = 0; i < kRotationsPerLane; ++i) {
        const int j = lane + 32 * i;
        if (j < half) {
            const float first = normalized(j), second = normalized(j + half);
            const float c = cosines[i], s = sines[i];
            target[j] = __float2bfloat16_rn(first * c - second * s);
            target[j + half] = __float2bfloat16_rn(second * c + first * s);
        }
    }
    for (int e = rotary_dim + lane; e < D; e += 32) target[e] = __float2bfloat16_rn(normalized(e));
}

#ifndef TAU_DECODE_CLUSTER
#define TAU_DECODE_CLUSTER 16
#endif
constexpr int kClusterSplits = TAU_DECODE_CLUSTER;   // the most splits that merge inside a thread-block cluster (above 8: not portable)
#ifndef TAU_DECODE_MIN_BLOCKS
#define TAU_DECODE_MIN_BLOCKS 4
#endif
template <int GH>
__global__ void __launch_bounds__(kWarps * 32, TAU_DECODE_MIN_BLOCKS)
decode_partial_mma_kernel(const bf16* __restrict__ queries, bf16* __restrict__ keys, bf16* __restrict__ values,
                          bf16* __restrict__ out, float* __restrict__ partial_o, float* __restrict__ partial_ml, int* __restrict__ tickets,
                          const int* __restrict__ seq_len, const int* __restrict__ page_rows, int page_stride, int page_tokens,
                          int n_heads, int n_kv_heads, int passes, float scale, int window, int splits, DecodePrepare prepare,
                          int clustered) {
    grid_dependents_launch();
    __shared__ float merge_o[kWarps][GH][D];
    __shared__ float merge_ml[kWarps][GH][2];
    __shared__ float block_ml[GH][2];        // clustered: this block's maximum (log2 units) and sum per head
    __shared__ __align__(16) bf16 q_shared[GH][D];
    __shared__ int is_last_block;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, seq = blockIdx.z;
    const int kv_head = blockIdx.y / passes, pass = blockIdx.y % passes;
    const int group = n_heads / n_kv_heads;
    const int head0 = kv_head * group + pass * GH;
    const int heads_here = min(GH, group - pass * GH);
    // What the step brought with it (lengths, page rows) and the tables were there before the step's first kernel began,
    // so they are read while the kernel before this one is still at work: the newest position's page and this lane's
    // rotation coefficients are here when that kernel's projection is.
    const int length = seq_len[seq];
    int newest_page = 0;
    float cosines[kRotationsPerLane], sines[kRotationsPerLane];
    if (prepare.projected != nullptr && length > 0) {
        newest_page = page_rows[static_cast<size_t>(seq) * page_stride + (length - 1) / page_tokens];
#pragma unroll
        for (int i = 0; i < kRotationsPerLane; ++i) {
            const int j = lane + 32 * i;
            const bool live = j < prepare.rotary_dim / 2;
            const size_t place = static_cast<size_t>(length - 1) * (prepare.rotary_dim / 2) + j;
            cosines[i] = live ? prepare.cos_table[place] : 1.0f;
            sines[i] = live ? prepare.sin_table[place] : 0.0f;
        }
    }
    grid_dependency_wait();
    const int first = (window > 0 && length > window) ? length - window : 0;
    const int span = length - first;
    const int per_split = ((span + splits - 1) / splits + 31) / 32 * 32;
    const int lo = first + split * per_split;
    const int hi = min(length, lo + per_split);
    const size_t record = (static_cast<size_t>(seq) * n_heads + head0) * splits + split;
    const int* pages = page_rows + static_cast<size_t>(seq) * page_stride;
    const size_t head_stride = static_cast<size_t>(page_tokens) * D;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    if (prepare.projected != nullptr && lo < hi) {
        // Tasks: the query heads of this pass; and, in the block whose range holds the newest position, its key and value.
        const int position = length - 1;
        // Every pass needs the newest row, so every pass whose range holds it writes it (the same values) and reads its own.
        const bool owns_newest = prepare.write_cache && lo <= position && position < hi;
        const bf16* row = prepare.projected + static_cast<size_t>(seq) * prepare.projected_stride;
        const size_t newest = (static_cast<size_t>(newest_page) * n_kv_heads + kv_head) * head_stride + static_cast<size_t>(position % page_tokens) * D;
        for (int task = warp; task < heads_here + (owns_newest ? 2 : 0); task += kWarps) {
            if (task < heads_here) {
                prepare_head(row + static_cast<size_t>(head0 + task) * D, prepare.q_weight, prepare.eps, cosines, sines, prepare.rotary_dim,
                             q_shared[task], lane);
            } else if (task == heads_here) {
                prepare_head(row + static_cast<size_t>(n_heads + kv_head) * D, prepare.k_weight, prepare.eps, cosines, sines,
                             prepare.rotary_dim, keys + newest, lane);
            } else {
                const bf16* source = row + static_cast<size_t>(n_heads + n_kv_heads + kv_head) * D;
                for (int e = lane; e < D; e += 32) values[newest + e] = source[e];
            }
        }
        __threadfence();   // the newest key and value are read back from the cache by this block below
    }
    __syncthreads();

    // Query fragments (B operand of the score product): head g of this pass, elements 32 c + 8 t .. + 8 of chunk c.
    uint4 q_frag[kQkChunks];
    {
        const bool head_live = g < heads_here && lo < hi;
        const bf16* q_row = prepare.projected != nullptr ? q_shared[head_live ? g : 0]
                                                         : queries + (static_cast<size_t>(seq) * n_heads + head0 + (head_live ? g : 0)) * D;
#pragma unroll
        for (int c = 0; c < kQkChunks; ++c) {
            const int e = 32 * c + 8 * t;
            q_frag[c] = (head_live && e + 8 <= D) ? *reinterpret_cast<const uint4*>(q_row + e) : zero4;
        }
    }
    const float scale_log2 = scale * 1.4426950408889634f;
    // This thread's two heads, 2t and 2t + 1: running maximum (log2 units) and this thread's share of the sum.
    float running_max[2] = {-INFINITY, -INFINITY}, running_sum[2] = {0.0f, 0.0f};
    float acc[kRounds][4][4];   // [round][tile][c0..c3]: c0, c1 = column 64 r + 8 g + 2 i of heads 2t, 2t+1; c2, c3 = the column after it
#pragma unroll
    for (int r = 0; r < kRounds; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[r][i][j] = 0.0f;

    auto row_offset = [&](int key) {   // a key beyond the range is replaced by the last one; its probability is zero
        const int k = min(key, hi - 1);
        return (static_cast<size_t>(pages[k / page_tokens]) * n_kv_heads + kv_head) * head_stride + static_cast<size_t>(k % page_tokens) * D;
    };

    for (int base = lo + warp * 16; base < hi; base += kWarps * 16) {
        // Value rows of keys base + {2t, 2t+1, 2t+8, 2t+9}, columns 64 r + 8 g .. + 8: requested together with the keys, used after the softmax.
        uint4 v_frag[kRounds][4];
        {
            const int slots[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const bf16* value_row = values + row_offset(base + slots[s]);
#pragma unroll
                for (int r = 0; r < kRounds; ++r) {
                    const int e = 64 * r + 8 * g;
                    v_frag[r][s] = (e + 8 <= D) ? __ldcg(reinterpret_cast<const uint4*>(value_row + e)) : zero4;
                }
            }
        }
        // Scores of 16 keys x 8 heads: rows g and g + 8 are keys base + g and base + g + 8.
        float score[4] = {0.0f, 0.0f, 0.0f, 0.0f}, score_odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        {
            const bf16* key_lo = keys + row_offset(base + g);
            const bf16* key_hi = keys + row_offset(base + g + 8);
            uint4 k_lo[kQkChunks], k_hi[kQkChunks];
#pragma unroll
            for (int c = 0; c < kQkChunks; ++c) {
                const int e = 32 * c + 8 * t;
                k_lo[c] = (e + 8 <= D) ? __ldcg(reinterpret_cast<const uint4*>(key_lo + e)) : zero4;
                k_hi[c] = (e + 8 <= D) ? __ldcg(reinterpret_cast<const uint4*>(key_hi + e)) : zero4;
            }
#pragma unroll
            for (int c = 0; c < kQkChunks; ++c) {   // two chains, so that consecutive products do not wait for each other
                mma_bf16(score, k_lo[c].x, k_hi[c].x, k_lo[c].y, k_hi[c].y, q_frag[c].x, q_frag[c].y);
                mma_bf16(score_odd, k_lo[c].z, k_hi[c].z, k_lo[c].w, k_hi[c].w, q_frag[c].z, q_frag[c].w);
            }
        }
        // score[0], [1]: key base + g, heads 2t and 2t + 1; score[2], [3]: key base + g + 8, the same heads.
        const bool live_lo = base + g < hi, live_hi = base + g + 8 < hi;
        float block_max[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            score[h] = live_lo ? (score[h] + score_odd[h]) * scale_log2 : -INFINITY;
            score[2 + h] = live_hi ? (score[2 + h] + score_odd[2 + h]) * scale_log2 : -INFINITY;
            block_max[h] = fmaxf(score[h], score[2 + h]);
            block_max[h] = fmaxf(block_max[h], __shfl_xor_sync(0xffffffffu, block_max[h], 4));
            block_max[h] = fmaxf(block_max[h], __shfl_xor_sync(0xffffffffu, block_max[h], 8));
            block_max[h] = fmaxf(block_max[h], __shfl_xor_sync(0xffffffffu, block_max[h], 16));
        }
        float correction[2], p[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float new_max = fmaxf(running_max[h], block_max[h]);   // finite: key `base` is inside the range
            correction[h] = exp2f(running_max[h] - new_max);
            running_max[h] = new_max;
            p[h] = exp2f(score[h] - new_max);
            p[2 + h] = exp2f(score[2 + h] - new_max);
            running_sum[h] = running_sum[h] * correction[h] + p[h] + p[2 + h];
        }
        // Probabilities as the B operand of the second product: transpose (key on g, head on t) into (key on t, head on g).
        unsigned pb0 = pack_bf16(p[0], p[1]), pb1 = pack_bf16(p[2], p[3]);
        asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb0) : "r"(pb0));
        asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb1) : "r"(pb1));
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const unsigned* k0 = reinterpret_cast<const unsigned*>(&v_frag[r][0]);   // key 2t
            const unsigned* k1 = reinterpret_cast<const unsigned*>(&v_frag[r][1]);   // key 2t + 1
            const unsigned* k8 = reinterpret_cast<const unsigned*>(&v_frag[r][2]);   // key 2t + 8
            const unsigned* k9 = reinterpret_cast<const unsigned*>(&v_frag[r][3]);   // key 2t + 9
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // Word i of a vector holds columns 2 i (low half) and 2 i + 1 (high half) of its key.
                const unsigned a0 = __byte_perm(k0[i], k1[i], 0x5410u), a1 = __byte_perm(k0[i], k1[i], 0x7632u);
                const unsigned a2 = __byte_perm(k8[i], k9[i], 0x5410u), a3 = __byte_perm(k8[i], k9[i], 0x7632u);
                acc[r][i][0] *= correction[0];
                acc[r][i][1] *= correction[1];
                acc[r][i][2] *= correction[0];
                acc[r][i][3] *= correction[1];
                mma_bf16(acc[r][i], a0, a1, a2, a3, pb0, pb1);
            }
        }
    }
    // Sums over the keys of this warp: over the 8 threads that share t.
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 4);
        running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 8);
        running_sum[h] += __shfl_xor_sync(0xffffffffu, running_sum[h], 16);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int head = 2 * t + h;
        if (head < GH) {
#pragma unroll
            for (int r = 0; r < kRounds; ++r)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c0 = 64 * r + 8 * g + 2 * i;
                    if (c0 < D) {
                        merge_o[warp][head][c0] = acc[r][i][h];
                        merge_o[warp][head][c0 + 1] = acc[r][i][2 + h];
                    }
                }
            if (g == 0) {
                merge_ml[warp][head][0] = running_max[h];
                merge_ml[warp][head][1] = running_sum[h];
            }
        }
    }
    __syncthreads();
    if (lo < hi) {
        for (int index = threadIdx.x; index < heads_here * D; index += kWarps * 32) {
            const int h = index / D, c = index % D;
            float total_max = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) total_max = fmaxf(total_max, merge_ml[w][h][0]);
            float o = 0.0f, sum = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float factor = exp2f(merge_ml[w][h][0] - total_max);   // 0 for a warp that saw no key
                if (factor > 0.0f) {
                    o += merge_o[w][h][c] * factor;
                    sum += merge_ml[w][h][1] * factor;
                }
            }
            if (splits == 1) {
                out[(static_cast<size_t>(seq) * n_heads + head0 + h) * D + c] = __float2bfloat16_rn(o / sum);
            } else if (clustered) {
                merge_o[0][h][c] = o;   // this thread alone reads and writes (h, c) of the first warp's buffer
                if (c == 0) {
                    block_ml[h][0] = total_max;
                    block_ml[h][1] = sum;
                }
            } else {
                const size_t slot = record + static_cast<size_t>(h) * splits;
                partial_o[slot * D + c] = o;
                if (c == 0) {
                    partial_ml[slot * 2] = total_max * 0.6931471805599453f;   // records are kept in natural-log units
                    partial_ml[slot * 2 + 1] = sum;
                }
            }
        }
    } else if (splits > 1 && clustered) {
        if (threadIdx.x < heads_here) {
            block_ml[threadIdx.x][0] = -INFINITY;
            block_ml[threadIdx.x][1] = 0.0f;
        }
    } else if (splits > 1 && threadIdx.x < heads_here) {   // nothing for this split: an empty record
        partial_ml[(record + static_cast<size_t>(threadIdx.x) * splits) * 2] = -INFINITY;
        partial_ml[(record + static_cast<size_t>(threadIdx.x) * splits) * 2 + 1] = 0.0f;
    }
    if (splits == 1) return;
    if (clustered) {
        // The splits of one sequence and KV head are one thread-block cluster: their results stay in shared memory, the
        // blocks meet, and each merges and stores a share of the heads' columns, reading the others' results through
        // distributed shared memory in the order of the splits.  Every thread of every block reaches both meetings.
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const unsigned rank = blockIdx.x;   // the cluster spans the grid's x
        for (int index = rank * (kWarps * 32) + threadIdx.x; index < heads_here * D; index += splits * kWarps * 32) {
            const int h = index / D, c = index % D;
            const unsigned o_address = static_cast<unsigned>(__cvta_generic_to_shared(&merge_o[0][h][c]));
            const unsigned ml_address = static_cast<unsigned>(__cvta_generic_to_shared(&block_ml[h][0]));
            float split_max[kClusterSplits], split_sum[kClusterSplits], split_o[kClusterSplits];
#pragma unroll
            for (int s = 0; s < kClusterSplits; ++s) {
                split_max[s] = -INFINITY;
                split_sum[s] = 0.0f;
                split_o[s] = 0.0f;
                if (s < splits) {
                    unsigned remote_ml, remote_o;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_ml) : "r"(ml_address), "r"(s));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_o) : "r"(o_address), "r"(s));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(split_max[s]) : "r"(remote_ml) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(split_sum[s]) : "r"(remote_ml + 4) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(split_o[s]) : "r"(remote_o) : "memory");
                }
            }
            float total_max = -INFINITY;
#pragma unroll
            for (int s = 0; s < kClusterSplits; ++s) total_max = fmaxf(total_max, split_max[s]);
            float o = 0.0f, sum = 0.0f;
#pragma unroll
            for (int s = 0; s < kClusterSplits; ++s) {
                const float factor = exp2f(split_max[s] - total_max);   // 0 for an empty split, whose context is not used
                if (factor > 0.0f) {
                    o += split_o[s] * factor;
                    sum += split_sum[s] * factor;
                }
            }
            out[(static_cast<size_t>(seq) * n_heads + head0 + h) * D + c] = __float2bfloat16_rn(o / sum);
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");   // nobody leaves while its results are read
        return;
    }
    // The block that finishes last for this sequence and KV head merges the splits' records
    // (the reference's `combine_attention`, decode_attention.cu:255-278, without a launch of its own).
    __threadfence();
    __syncthreads();
    int* ticket = tickets + static_cast<size_t>(seq) * gridDim.y + blockIdx.y;
    if (threadIdx.x == 0) is_last_block = atomicAdd(ticket, 1) == splits - 1;
    __syncthreads();
    if (!is_last_block) return;
    __threadfence();
    // The records' maxima and sums go through shared memory first (one round trip for all of them), so that the
    // sums over the splits below are independent loads and not a chain.  The merge buffers are free by now.
    float* record_max = &merge_o[0][0][0];               // [heads_here][splits]
    float* record_sum = record_max + GH * splits;        // [heads_here][splits]   (2 GH splits <= kWarps GH D floats: splits <= 2 D)
    for (int index = threadIdx.x; index < heads_here * splits; index += kWarps * 32) {
        const int h = index / splits, s = index % splits;
        const size_t slot = (static_cast<size_t>(seq) * n_heads + head0 + h) * splits + s;
        record_max[h * splits + s] = __ldcg(partial_ml + slot * 2);
        record_sum[h * splits + s] = __ldcg(partial_ml + slot * 2 + 1);
    }
    __syncthreads();
    if (threadIdx.x < heads_here) {   // per head: the factor of each split, and one over the total sum in merge_ml[0][h][0]
        const int h = threadIdx.x;
        float total_max = -INFINITY;
        for (int s = 0; s < splits; ++s) total_max = fmaxf(total_max, record_max[h * splits + s]);
        float sum = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float factor = __expf(record_max[h * splits + s] - total_max);   // 0 for an empty split
            sum += record_sum[h * splits + s] * factor;
            record_max[h * splits + s] = factor;
        }
        merge_ml[0][h][0] = 1.0f / sum;
    }
    __syncthreads();
    for (int index = threadIdx.x; index < heads_here * D; index += kWarps * 32) {
        const int h = index / D, c = index % D;
        const float* column = partial_o + (static_cast<size_t>(seq) * n_heads + head0 + h) * splits * D + c;
        float o = 0.0f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            const float factor = record_max[h * splits + s];
            const float value = __ldcg(column + static_cast<size_t>(s) * D);
            o += factor > 0.0f ? value * factor : 0.0f;   // an empty split wrote no context: whatever lies there is not used
        }
        out[(static_cast<size_t>(seq) * n_heads + head0 + h) * D + c] = __float2bfloat16_rn(o * merge_ml[0][h][0]);
    }
    if (threadIdx.x == 0) *ticket = 0;   // ready for the next launch
}
#endif  // TAU_DTYPE == 1

[[maybe_unused]] __global__ void decode_combine_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                      T* __restrict__ out, int n_heads, int splits) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int head = blockIdx.x, seq = blockIdx.y;
    const size_t base = (static_cast<size_t>(seq) * n_heads + head) * splits;
    float total_max = -INFINITY;
    for (int s = 0; s < splits; ++s) total_max = fmaxf(total_max, partial_ml[(base + s) * 2]);
    float sum = 0.0f;
    for (int s = 0; s < splits; ++s) sum += partial_ml[(base + s) * 2 + 1] * exponential(partial_ml[(base + s) * 2] - total_max);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float o = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float factor = exponential(partial_ml[(base + s) * 2] - total_max);
            if (factor > 0.0f) o += partial_o[(base + s) * D + c] * factor;   // an empty split wrote no context
        }
        out[(static_cast<size_t>(seq) * n_heads + head) * D + c] = from_float<T>(o / sum);
    }
}

}  // namespace

TAU_EXPORT int tau_attention_decode_head_dim() { return D; }
TAU_EXPORT int tau_attention_decode_dtype() { return TAU_DTYPE; }

// Floats of scratch that a launch needs.
TAU_EXPORT long long tau_attention_decode_scratch(int n_seqs, int n_heads, int splits) {
    return splits <= 1 ? 0 : static_cast<long long>(n_seqs) * n_heads * splits * (D + 2);
}

// Ints of zeroed ticket memory that a bfloat16 launch with more than one split needs (they are left at zero).
TAU_EXPORT long long tau_attention_decode_tickets(int n_seqs, int n_heads, int n_kv_heads) {
    const int group = n_heads / n_kv_heads;
    const int gh = group >= 8 ? 8 : group > 2 ? 4 : group;
    return static_cast<long long>(n_seqs) * n_kv_heads * ((group + gh - 1) / gh);
}

// `projected` != nullptr (bfloat16 only): queries, the newest key and the newest value are taken from the stacked
// projection `[sequences, (n_heads + 2 n_kv_heads) D]`, normalised and rotated here, and the key and value are
// written to their cache pages (`write_cache`); `queries` is then not read.
TAU_EXPORT int tau_attention_decode(const void* queries, void* keys, void* values, void* out, const int* seq_len,
                                    const int* page_rows, int page_stride, int page_tokens, int n_seqs, int n_heads, int n_kv_heads,
                                    float scale, int window, int splits, float* scratch, long long scratch_floats, int* tickets,
                                    const void* projected, long long projected_stride, const float* q_weight, const float* k_weight,
                                    float eps, const float* cos_table, const float* sin_table, int rotary_dim, int write_cache,
                                    int cluster_merge, void* stream) {
    if (n_seqs <= 0) return 0;
    if ((!queries && !projected) || !keys || !values || !out || !seq_len || !page_rows || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads != 0 || page_tokens <= 0 || window < 0 || splits < 1 || splits > 256 ||
        (splits > 1 && (!scratch || scratch_floats < tau_attention_decode_scratch(n_seqs, n_heads, splits))) ||
        (projected && (rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1) || (rotary_dim > 0 && (!cos_table || !sin_table)))))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int group = n_heads / n_kv_heads;
    const int gh = group >= 8 ? 8 : group > 2 ? 4 : group;      // heads per pass: 1, 2, 4 or 8
    const int passes = (group + gh - 1) / gh;
    const dim3 grid(splits, n_kv_heads * passes, n_seqs);
    float* partial_o = scratch;
    float* partial_ml = scratch ? scratch + static_cast<size_t>(n_seqs) * n_heads * splits * D : nullptr;
#if TAU_DTYPE == 1
    if (splits > 1 && (!tickets || splits > 2 * D)) return cudaErrorInvalidValue;   // the merge reuses 2 GH splits floats of shared memory
    DecodePrepare prepare = {static_cast<const bf16*>(projected), projected_stride, q_weight, k_weight, eps, cos_table, sin_table,
                             rotary_dim, write_cache};
    // Launched after the previous kernel has finished, not beside it: blocks that start on SMs which still hold the
    // blocks of the projection before them (100 KB of shared memory each) ran the whole kernel a half slower at batch 64
    // (138 us against 92 us per layer at 2,048 tokens of context), and at batch 8 starting early gained nothing.
    // Up to 16 splits form a thread-block cluster (above 8: a cluster size that is not portable, allowed on this part) and
    // merge through shared memory; more meet in global memory by tickets.
    const bool clustered = splits > 1 && splits <= kClusterSplits && cluster_merge != 0;
    if (clustered && splits > 8) {
        static bool allowed[4] = {false, false, false, false};
        const int which = gh == 1 ? 0 : gh == 2 ? 1 : gh == 4 ? 2 : 3;
        if (!allowed[which]) {
            cudaError_t status = gh == 1   ? cudaFuncSetAttribute(decode_partial_mma_kernel<1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1)
                                 : gh == 2 ? cudaFuncSetAttribute(decode_partial_mma_kernel<2>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1)
                                 : gh == 4 ? cudaFuncSetAttribute(decode_partial_mma_kernel<4>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1)
                                           : cudaFuncSetAttribute(decode_partial_mma_kernel<8>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (status != cudaSuccess) return static_cast<int>(status);
            allowed[which] = true;
        }
    }
#define TAU_LAUNCH(GH) do {                                                                                                        \
    if (clustered)                                                                                                                  \
        tau_launch_clusters_as(false, splits, decode_partial_mma_kernel<GH>, grid, dim3(kWarps * 32), 0, s, static_cast<const bf16*>(queries),       \
                               static_cast<bf16*>(keys), static_cast<bf16*>(values), static_cast<bf16*>(out), partial_o, partial_ml, tickets, seq_len, \
                               page_rows, page_stride, page_tokens, n_heads, n_kv_heads, passes, scale, window, splits, prepare, 1);   \
    else                                                                                                                            \
        tau_launch_as(false, decode_partial_mma_kernel<GH>, grid, dim3(kWarps * 32), 0, s, static_cast<const bf16*>(queries), static_cast<bf16*>(keys), \
                      static_cast<bf16*>(values), static_cast<bf16*>(out), partial_o, partial_ml, tickets, seq_len, page_rows, page_stride,  \
                      page_tokens, n_heads, n_kv_heads, passes, scale, window, splits, prepare, 0); } while (0)
    if (gh == 1) TAU_LAUNCH(1);
    else if (gh == 2) TAU_LAUNCH(2);
    else if (gh == 4) TAU_LAUNCH(4);
    else TAU_LAUNCH(8);
#undef TAU_LAUNCH
    return tau_launch_status();
#else
    if (projected) return cudaErrorInvalidValue;   // the 32-bit path prepares with the kernel of its own
#define TAU_LAUNCH(GH)                                                                                                             \
    tau_launch(decode_partial_kernel<GH>, grid, dim3(kWarps * 32), 0, s, static_cast<const T*>(queries), static_cast<const T*>(keys),   \
               static_cast<const T*>(values), static_cast<T*>(out), partial_o, partial_ml, seq_len, page_rows, page_stride,         \
               page_tokens, n_heads, n_kv_heads, passes, scale, window, splits)
    if (gh == 1) TAU_LAUNCH(1);
    else if (gh == 2) TAU_LAUNCH(2);
    else if (gh == 4) TAU_LAUNCH(4);
    else TAU_LAUNCH(8);
#undef TAU_LAUNCH
    int status = tau_launch_status();
    if (status || splits == 1) return status;
    tau_launch(decode_combine_kernel, dim3(n_heads, n_seqs), dim3(D < 128 ? D : 128), 0, s, partial_o, partial_ml, static_cast<T*>(out), n_heads, splits);
    return tau_launch_status();
#endif
}
