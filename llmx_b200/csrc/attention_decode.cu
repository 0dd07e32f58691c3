// Split-KV attention over block tables for requests that bring one or a few rows (decoding).
//
// A block serves one (request, kv head, key range): the request's `n` new rows times the
// `ratio = heads / kv_heads` query heads of the group form at most 16 query rows that share
// every key and value they read, so each page is fetched once for the whole group.
//
//   producer warp    walks the request's block table and fetches its pages with TMA
//                    (boxes of [16 slots, 64 columns], 128-byte swizzle), four pages a stage, one
//                    lane issuing each page's copy, three stages in flight; stages whose pages lie wholly
//                    below the request's history (earlier steps' keys) are asked for before the kernel
//                    waits for the kernel before it
//   4 consumer warps warps 0-1 take the even stages, warps 2-3 the odd ones; of a stage's four pages a warp
//                    takes two as one tile of 32 keys: S = Q K^T (mma.sync m16n8k16, bfloat16 in,
//                    float32 out), masks (causal, window, end of the key range), online softmax
//                    in float32 (base 2), O += P V
//   at the end       the four warps' (m, l, O) are merged through shared memory; with one key
//                    range the result is written, else a partial (m, l, O) goes to the
//                    workspace and `attn_merge_kernel` combines the ranges.
//
// This kernel is bound by the cache bytes it reads; the matrix work on 16-row tiles is a
// small fraction of what the SM can do, which is why it uses the warp-level instruction rather
// than tcgen05 (whose 64/128-row tiles would be 75-97 % padding here).
// Reference counterpart: llmx_attention_vec and its merge (src/backends/gpu/kernels/f32.gpu:1640-1715, :1863).
#include "attn_common.cuh"
#include <math.h>

namespace {

constexpr int PAGE = 16;
constexpr int PAGES_PER_STAGE = 4;
constexpr int STAGES = 3;
constexpr int CONSUMERS = 4;
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int MAX_ROWS = 16;
enum : int { ERR_DEC_PRODUCER = 201, ERR_DEC_CONSUMER = 202 };

template <int D>
struct Cfg {
    static constexpr int BOXES = D / attn::BOX_COLS;
    static constexpr int BOX_BYTES = PAGE * 128;
    static constexpr int PLANE_BYTES = BOXES * BOX_BYTES;       // one page's keys (or values) of one head
    static constexpr int PAGE_BYTES = 2 * PLANE_BYTES;
    static constexpr int STAGE_BYTES = PAGES_PER_STAGE * PAGE_BYTES;
    static constexpr int MERGE_BYTES = CONSUMERS * MAX_ROWS * (D + 2) * 4;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES > MERGE_BYTES ? STAGES * STAGE_BYTES : MERGE_BYTES;
    static constexpr int MADE_BYTES = 3 * MAX_ROWS * D * 2 + 64;     // queries, new keys, new values (bfloat16), flags
    static constexpr int SMEM_BYTES = TILE_BYTES + 1024 + 128 + MADE_BYTES;
};

// Optional input for blocks that make their own queries and new keys and values from the product's float32
// output (head width 128, rotated whole or not at all): what the separate norm / rotation / cache-write kernel
// would have done for these rows, in the same arithmetic.
struct QkvInput {
    const float* qkv;              // [rows, stride]: q heads, then k heads at k_offset, v heads at v_offset; null: unused
    int stride, k_offset, v_offset;
    const float* q_weight;         // per-head norm weights [128] or null
    const float* k_weight;
    float eps;
    const float* cos_table;        // [positions, 64] or null
    const float* sin_table;
    const int* slots;              // per row: page * page_size + slot of its key and value, negative: not written
    __nv_bfloat16* cache;          // [pages, 2, kv_heads, 16, 128]
};

// ---- thread-block clusters: a barrier over all threads of all blocks of the cluster, this block's rank, and loads
// from another block's shared memory.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// One row of 128 values by one warp, lane l holding values 4l .. 4l+3: RMSNorm with `weight` (skipped when
// null), then rotation of the pairs (i, i + 64) by the angles of `pos` (skipped when the tables are null).
// The arithmetic is that of head_norm_rope_128_kernel (rowwise.cu), operation for operation.
__device__ __forceinline__ float4 norm_rope_row_128(const float* src, const float* weight, float eps,
                                                    const float* cos_table, const float* sin_table, int pos, int lane) {
    float4 v = reinterpret_cast<const float4*>(src)[lane];
    if (weight) {
        float s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
        s = warp_sum(s);
        const float rr = 1.0f / sqrtf(s / 128.0f + eps);
        const float4 w4 = reinterpret_cast<const float4*>(weight)[lane];
        v.x *= rr * w4.x; v.y *= rr * w4.y; v.z *= rr * w4.z; v.w *= rr * w4.w;
    }
    if (cos_table) {
        const size_t base = (size_t)pos * 64 + 4 * (lane & 15);
        const float4 c = *reinterpret_cast<const float4*>(cos_table + base);
        const float4 sn = *reinterpret_cast<const float4*>(sin_table + base);
        float4 o;
        o.x = __shfl_xor_sync(0xffffffffu, v.x, 16); o.y = __shfl_xor_sync(0xffffffffu, v.y, 16);
        o.z = __shfl_xor_sync(0xffffffffu, v.z, 16); o.w = __shfl_xor_sync(0xffffffffu, v.w, 16);
        if (lane < 16) {
            v.x = fmaf(-o.x, sn.x, v.x * c.x); v.y = fmaf(-o.y, sn.y, v.y * c.y);
            v.z = fmaf(-o.z, sn.z, v.z * c.z); v.w = fmaf(-o.w, sn.w, v.w * c.w);
        } else {
            v.x = fmaf(o.x, sn.x, v.x * c.x); v.y = fmaf(o.y, sn.y, v.y * c.y);
            v.z = fmaf(o.z, sn.z, v.z * c.z); v.w = fmaf(o.w, sn.w, v.w * c.w);
        }
    }
    return v;
}

__device__ __forceinline__ uint2 pack4_bf16(float4 v) {
    return make_uint2(attn::pack_bf16(v.x, v.y), attn::pack_bf16(v.z, v.w));
}

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const __grid_constant__ CUtensorMap cache_map, const __nv_bfloat16* __restrict__ q,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ partial, const int* __restrict__ req_list,
                   const int* __restrict__ row_start, const int* __restrict__ row_count,
                   const int* __restrict__ history, const int* __restrict__ block_tables, int table_stride, int heads,
                   int kv_heads, int window, float scale_log2, int splits, const int* __restrict__ chunk_ptr,
                   int chunk_keys, int* __restrict__ counters, int* error_word, const QkvInput made, int cluster_merge) {
    pdl_trigger();
    // What the kernel before this one writes (the queries or the product's output, this step's keys and values) is
    // touched only after pdl_wait(), which every warp reaches on its own path below.  The step's metadata and the
    // pages that lie wholly below the request's history were written before the step began: the producer asks for
    // those pages at once, while the kernel before still runs.
    using cfg = Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int is_last;
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(tiles + cfg::TILE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    volatile int* abort_flag = (volatile int*)(empty_bar + STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, g = blockIdx.y, r = req_list[blockIdx.z];
    const int ratio = heads / kv_heads;
    const int n_q = row_count[r], q0 = row_start[r], hist = history[r];
    const int M = n_q * ratio;
    const int len = hist + n_q;
    const int chunk = chunk_ptr ? *chunk_ptr : chunk_keys;
    int kv_begin = split * chunk;
    const int kv_end = min(len, kv_begin + chunk);
    if (window > 0) {
        const int lowest = max(0, hist - window + 1);          // the first row's lowest key
        kv_begin = max(kv_begin, (lowest / PAGE) * PAGE);
    }
    const int n_pages = kv_end > kv_begin ? (kv_end - kv_begin + PAGE - 1) / PAGE : 0;
    const int iters = (n_pages + PAGES_PER_STAGE - 1) / PAGES_PER_STAGE;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], CONSUMERS);          // every consumer warp has seen the stage full (two read it)
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    // What the block makes itself when it is given the product's output instead of finished queries.
    __nv_bfloat16* q_made = (__nv_bfloat16*)(tiles + cfg::TILE_BYTES + 128);      // [MAX_ROWS][D]
    __nv_bfloat16* kv_made = q_made + MAX_ROWS * D;                              // [MAX_ROWS][2][D]
    int* kv_patch = (int*)(kv_made + 2 * MAX_ROWS * D);                          // [MAX_ROWS]: the row is to be used
    __syncthreads();          // the barriers are ready
    // The producer warp starts the key stages at once; the other warps meanwhile make the block's queries and new
    // keys (if it is given the product's output) and meet at a barrier of their own before they use them.
    if (warp != CONSUMERS) pdl_wait();
    if constexpr (D == 128) {
        if (made.qkv && warp < CONSUMERS) {
            for (int i = warp; i < M; i += CONSUMERS) {
                const int ti = i / ratio, h = g * ratio + i % ratio;
                const float4 v = norm_rope_row_128(made.qkv + (size_t)(q0 + ti) * made.stride + h * D, made.q_weight,
                                                   made.eps, made.cos_table, made.sin_table, hist + ti, lane);
                *reinterpret_cast<uint2*>(q_made + i * D + 4 * lane) = pack4_bf16(v);
            }
            // The new keys and values that lie in this block's key range: to the cache for later steps, and kept
            // here to be laid over their page when it arrives (the copy may have read the page before or after
            // the store above landed).
            for (int t = warp; t < n_q; t += CONSUMERS) {
                const int p = hist + t;
                const int slot = made.slots[q0 + t];
                const bool mine = p >= kv_begin && p < kv_end && slot >= 0;
                if (lane == 0) kv_patch[t] = mine ? 1 : 0;
                if (mine) {
                    const float* row = made.qkv + (size_t)(q0 + t) * made.stride;
                    const float4 k = norm_rope_row_128(row + made.k_offset + g * D, made.k_weight, made.eps,
                                                       made.cos_table, made.sin_table, p, lane);
                    const float4 v = reinterpret_cast<const float4*>(row + made.v_offset + g * D)[lane];
                    const uint2 kb = pack4_bf16(k), vb = pack4_bf16(v);
                    *reinterpret_cast<uint2*>(kv_made + (t * 2 + 0) * D + 4 * lane) = kb;
                    *reinterpret_cast<uint2*>(kv_made + (t * 2 + 1) * D + 4 * lane) = vb;
                    const int page = slot / PAGE, off = slot % PAGE;
                    const size_t key_base = ((((size_t)page * 2 + 0) * kv_heads + g) * PAGE + off) * D;
                    const size_t value_base = ((((size_t)page * 2 + 1) * kv_heads + g) * PAGE + off) * D;
                    *reinterpret_cast<uint2*>(made.cache + key_base + 4 * lane) = kb;
                    *reinterpret_cast<uint2*>(made.cache + value_base + 4 * lane) = vb;
                }
            }
        }
    }
    if (warp < CONSUMERS) asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");

    // Per-thread accumulators of the consumer warps (rows r0 = lane / 4 and r0 + 8 of the 16-row tile).
    float o[D / 8][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
#pragma unroll
    for (int t = 0; t < D / 8; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[t][e] = 0.0f;

    if (warp == CONSUMERS) {
        // One lane per page of a stage: each reads its page's id from the block table (one stage ahead, so the
        // table's latency is off the copies' path) and issues its copy; a single thread issuing all of a
        // stage's copies was what bounded a block's rate.
        bool waited = false;
        if (n_pages > 0 && lane < PAGES_PER_STAGE) {
            if (lane == 0) tc::tma_prefetch_desc(&cache_map);
            const int* table = block_tables + (size_t)r * table_stride + kv_begin / PAGE;
            int id_next = lane < n_pages ? max(table[lane], 0) : 0;      // (a page given back, -1, is never needed: see kv_begin)
            for (int it = 0; it < iters; ++it) {
                const int stage = it % STAGES;
                const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
                // A stage whose pages end at or below the history holds earlier steps' keys only: no need to wait.
                if (!waited && kv_begin + (it + 1) * PAGES_PER_STAGE * PAGE > hist) {
                    pdl_wait();
                    waited = true;
                }
                const int id = id_next;
                const int nxt = (it + 1) * PAGES_PER_STAGE + lane;
                id_next = nxt < n_pages ? max(table[nxt], 0) : 0;
                bool ok = tc::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, error_word, ERR_DEC_PRODUCER);
                const int here = min(PAGES_PER_STAGE, n_pages - it * PAGES_PER_STAGE);
                // The bytes a phase expects must be announced before any of its copies can land (a copy that
                // completes first is not counted later): lane 0 announces, then the lanes issue.
                if (lane == 0 && ok) tc::mbar_expect_tx(&full_bar[stage], (uint32_t)(here * cfg::PAGE_BYTES));
                ok = __all_sync((1u << PAGES_PER_STAGE) - 1u, ok);
                if (!ok) break;
                // One copy brings the head's keys and values of the page: [plane][half][slot][64 columns].
                if (lane < here)
                    tc::tma_load_5d(tiles + stage * cfg::STAGE_BYTES + lane * cfg::PAGE_BYTES, &cache_map, 0, 0, 0, g,
                                    id * 2, &full_bar[stage]);
            }
        }
        if (!waited) pdl_wait();      // every thread has waited before the block's results are written
    } else {
        // ---- query fragments: row i of the tile is (new row i / ratio, head g * ratio + i % ratio)
        uint32_t qa[D / 16][4];
        const int r0 = lane >> 2, r1 = r0 + 8;
        int pos[2], lo[2];
        bool valid[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = half ? r1 : r0;
            valid[half] = row < M;
            const int ti = row / ratio;
            pos[half] = hist + ti;
            lo[half] = window > 0 ? max(0, pos[half] - window + 1) : 0;
            const __nv_bfloat16* src = made.qkv ? q_made + min(row, MAX_ROWS - 1) * D
                                                : q + ((size_t)(q0 + ti) * heads + g * ratio + row % ratio) * D;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int d = kk * 16 + (lane & 3) * 2;
                qa[kk][half] = valid[half] ? *reinterpret_cast<const uint32_t*>(src + d) : 0u;
                qa[kk][half + 2] = valid[half] ? *reinterpret_cast<const uint32_t*>(src + d + 8) : 0u;
            }
        }
        // Warps 0 and 1 take the even stages, warps 2 and 3 the odd ones; of a stage's four pages a warp takes
        // two, as one tile of 32 keys: twice the independent work between a warp's waits, half the rescaling.
        // Every warp waits for every stage, also those it does not read, and tells the producer so: a wait tells
        // a barrier's phases apart by their parity only, so a warp must neither skip a phase nor be so far behind
        // that the stage is filled again before it has looked.
        const int pair = warp & 1, group = warp >> 1;
        for (int it = 0; it < iters; ++it) {
            const int stage = it % STAGES;
            const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
            if (!tc::mbar_wait(&full_bar[stage], phase, abort_flag, error_word, ERR_DEC_CONSUMER)) break;
            if ((it & 1) != group) {
                if (lane == 0) tc::mbar_arrive(&empty_bar[stage]);
                continue;
            }
            const int page_index = it * PAGES_PER_STAGE + 2 * pair;
            if (page_index < n_pages) {
                const int key0 = kv_begin + page_index * PAGE;
                const uint32_t kbase = tc::smem_u32(tiles + stage * cfg::STAGE_BYTES + 2 * pair * cfg::PAGE_BYTES);
                const uint32_t vbase = kbase + cfg::PLANE_BYTES;
                if (D == 128 && made.qkv && key0 + 2 * PAGE > hist) {
                    // The step's own keys and values among these 32: laid over what the copy brought.
                    for (int t = 0; t < n_q; ++t) {
                        const int at = hist + t - key0;
                        if (at >= 0 && at < 2 * PAGE && kv_patch[t]) {
                            const int plane = lane >> 4, c = lane & 15;           // 16 chunks of 8 values a row
                            const uint4 val = *reinterpret_cast<const uint4*>(kv_made + (t * 2 + plane) * D + c * 8);
                            const uint32_t addr = kbase + (at / PAGE) * cfg::PAGE_BYTES + plane * cfg::PLANE_BYTES +
                                                  (c >> 3) * cfg::BOX_BYTES + attn::swz(at % PAGE, c & 7);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(val.x), "r"(val.y),
                                         "r"(val.z), "r"(val.w) : "memory");
                        }
                    }
                    __syncwarp();
                }
                if (key0 + 2 * PAGE > kv_end) {
                    // Slots past the request's last key hold whatever an earlier owner left, and a page past
                    // the range's last one was not fetched at all: zero those values so that a stale
                    // non-finite number cannot reach the sum through a zero weight.
                    const int first_bad = kv_end - key0;                 // 1 .. 31, counted over both pages
                    for (int i = lane; i < (2 * PAGE - first_bad) * cfg::BOXES * 8; i += 32) {
                        const int row = first_bad + i / (cfg::BOXES * 8), c = i % (cfg::BOXES * 8);
                        const uint32_t addr = vbase + (row / PAGE) * cfg::PAGE_BYTES + (c >> 3) * cfg::BOX_BYTES +
                                              attn::swz(row % PAGE, c & 7);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
                    }
                    __syncwarp();
                }
                // ---- S = Q K^T for the 32 keys: s[2 * page + j] is the 8-key column block j of the page
                float s[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const int dchunk = 2 * kk + ((lane >> 3) & 1);
                    const int key = ((lane >> 4) << 3) + (lane & 7);
                    const uint32_t off = (dchunk >> 3) * cfg::BOX_BYTES + attn::swz(key, dchunk & 7);
                    uint32_t b0, b1, b2, b3, c0, c1, c2, c3;
                    attn::ldmatrix_x4(kbase + off, b0, b1, b2, b3);
                    attn::ldmatrix_x4(kbase + cfg::PAGE_BYTES + off, c0, c1, c2, c3);
                    attn::mma_16816(s[0], qa[kk], b0, b1);
                    attn::mma_16816(s[1], qa[kk], b2, b3);
                    attn::mma_16816(s[2], qa[kk], c0, c1);
                    attn::mma_16816(s[3], qa[kk], c2, c3);
                }
                // ---- mask, online softmax (base 2)
                float rowmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1;
                        const int key = key0 + 8 * j + (lane & 3) * 2 + (e & 1);
                        // (a pair's second page may lie past the range: those keys are another block's)
                        const bool ok = valid[half] && key >= lo[half] && key <= pos[half] && key < kv_end;
                        s[j][e] = ok ? s[j][e] * scale_log2 : -INFINITY;
                        rowmax[half] = fmaxf(rowmax[half], s[j][e]);
                    }
                float alpha[2], base[2];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    rowmax[half] = fmaxf(rowmax[half], __shfl_xor_sync(0xffffffffu, rowmax[half], 1));
                    rowmax[half] = fmaxf(rowmax[half], __shfl_xor_sync(0xffffffffu, rowmax[half], 2));
                    const float m_new = fmaxf(m_run[half], rowmax[half]);
                    alpha[half] = m_new == -INFINITY ? 1.0f : exp2f(m_run[half] - m_new);
                    base[half] = m_new == -INFINITY ? 0.0f : m_new;
                    m_run[half] = m_new;
                }
                float psum[2] = {0.0f, 0.0f};
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        s[j][e] = exp2f(s[j][e] - base[e >> 1]);
                        psum[e >> 1] += s[j][e];
                    }
                l_run[0] = l_run[0] * alpha[0] + psum[0];
                l_run[1] = l_run[1] * alpha[1] + psum[1];
                uint32_t pa[2][4];          // P of the first and of the second page as A operands (16 x 16 each)
#pragma unroll
                for (int pg = 0; pg < 2; ++pg) {
                    pa[pg][0] = attn::pack_bf16(s[2 * pg][0], s[2 * pg][1]);
                    pa[pg][1] = attn::pack_bf16(s[2 * pg][2], s[2 * pg][3]);
                    pa[pg][2] = attn::pack_bf16(s[2 * pg + 1][0], s[2 * pg + 1][1]);
                    pa[pg][3] = attn::pack_bf16(s[2 * pg + 1][2], s[2 * pg + 1][3]);
                }
                // ---- O = O * alpha + P V
#pragma unroll
                for (int t = 0; t < D / 8; t += 2) {
                    o[t][0] *= alpha[0]; o[t][1] *= alpha[0]; o[t][2] *= alpha[1]; o[t][3] *= alpha[1];
                    o[t + 1][0] *= alpha[0]; o[t + 1][1] *= alpha[0]; o[t + 1][2] *= alpha[1]; o[t + 1][3] *= alpha[1];
                    const int key = (((lane >> 3) & 1) << 3) + (lane & 7);
                    const int dchunk = t + (lane >> 4);
                    const uint32_t off = (dchunk >> 3) * cfg::BOX_BYTES + attn::swz(key, dchunk & 7);
                    uint32_t b0, b1, b2, b3, c0, c1, c2, c3;
                    attn::ldmatrix_x4_trans(vbase + off, b0, b1, b2, b3);
                    attn::ldmatrix_x4_trans(vbase + cfg::PAGE_BYTES + off, c0, c1, c2, c3);
                    attn::mma_16816(o[t], pa[0], b0, b1);
                    attn::mma_16816(o[t + 1], pa[0], b2, b3);
                    attn::mma_16816(o[t], pa[1], c0, c1);
                    attn::mma_16816(o[t + 1], pa[1], c2, c3);
                }
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty_bar[stage]);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
        }
    }
    __syncthreads();   // every page has been consumed: the tile memory can hold the merge buffer

    float* merge = (float*)tiles;   // [CONSUMERS][MAX_ROWS][D + 2]
    constexpr int XCHG_STRIDE = D + 4;                                        // rows of 16 bytes' multiple
    float* xchg = merge + CONSUMERS * MAX_ROWS * (D + 2);                     // [MAX_ROWS][XCHG_STRIDE]: this range's result
    if (warp < CONSUMERS) {
        const int r0 = lane >> 2;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = r0 + 8 * half;
            if (row < M) {
                float* mine = merge + ((size_t)warp * MAX_ROWS + row) * (D + 2);
#pragma unroll
                for (int t = 0; t < D / 8; ++t) {
                    const int d = 8 * t + (lane & 3) * 2;
                    mine[d] = o[t][2 * half];
                    mine[d + 1] = o[t][2 * half + 1];
                }
                if ((lane & 3) == 0) {
                    mine[D] = m_run[half];
                    mine[D + 1] = l_run[half];
                }
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < M * D; idx += THREADS) {
        const int row = idx / D, d = idx % D;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) mm = fmaxf(mm, merge[((size_t)w * MAX_ROWS + row) * (D + 2) + D]);
        float acc = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) {
            const float* src = merge + ((size_t)w * MAX_ROWS + row) * (D + 2);
            const float f = src[D] == -INFINITY ? 0.0f : exp2f(src[D] - mm);
            acc += src[d] * f;
            l += src[D + 1] * f;
        }
        const int ti = row / ratio, h = g * ratio + row % ratio;
        const size_t out_row = (size_t)(q0 + ti) * heads + h;
        if (splits == 1) {
            out[out_row * D + d] = __float2bfloat16_rn(acc / l);
        } else if (cluster_merge) {
            // The key ranges' blocks are one cluster: the range's result stays in this block's shared memory,
            // where the others read it.
            float* dst = xchg + row * XCHG_STRIDE;
            dst[d] = acc;
            if (d == 0) {
                dst[D] = mm;
                dst[D + 1] = l;
            }
        } else {
            float* dst = partial + (out_row * splits + split) * (D + 2);
            dst[d] = acc;
            if (d == 0) {
                dst[D] = mm;
                dst[D + 1] = l;
            }
        }
    }
    if (splits > 1 && cluster_merge) {
        // The ranges' blocks of a (request, kv head) are a thread-block cluster.  When all have their results in
        // shared memory (first barrier), each block combines its share of the (row, four values) items, reading
        // every range's maximum, sum and values through distributed shared memory; no block leaves before all
        // have read (second barrier).  Every thread of every block gets here on every path: nothing above returns.
        cluster_barrier();
        const uint32_t rank = cluster_rank();
        const int items = M * (D / 4);
        const int per = (items + splits - 1) / splits;
        const int last = min(items, (int)(rank + 1) * per);
        for (int idx = (int)rank * per + threadIdx.x; idx < last; idx += THREADS) {
            const int row = idx / (D / 4), d = (idx % (D / 4)) * 4;
            const uint32_t mine = tc::smem_u32(xchg + row * XCHG_STRIDE);
            float mm = -INFINITY;
            for (int s2 = 0; s2 < splits; ++s2) mm = fmaxf(mm, ld_cluster_f32(cluster_map(mine + D * 4, s2)));
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float l = 0.0f;
            for (int s2 = 0; s2 < splits; ++s2) {
                const uint32_t theirs = cluster_map(mine, s2);
                const float ms = ld_cluster_f32(theirs + D * 4);
                const float f = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
                const float4 o = ld_cluster_f32x4(theirs + d * 4);
                acc.x = fmaf(o.x, f, acc.x); acc.y = fmaf(o.y, f, acc.y);
                acc.z = fmaf(o.z, f, acc.z); acc.w = fmaf(o.w, f, acc.w);
                l = fmaf(ld_cluster_f32(theirs + (D + 1) * 4), f, l);
            }
            const float inv = 1.0f / l;
            const size_t out_row = (size_t)(q0 + row / ratio) * heads + g * ratio + row % ratio;
            *reinterpret_cast<uint2*>(out + out_row * D + d) =
                make_uint2(attn::pack_bf16(acc.x * inv, acc.y * inv), attn::pack_bf16(acc.z * inv, acc.w * inv));
        }
        cluster_barrier();
    } else if (splits > 1 && counters) {
        // The block that finishes last among the key ranges of this (request, kv head) combines them.
        // Nobody waits: each block counts itself in and only the one that sees the others' count goes on.
        __threadfence();
        __syncthreads();
        int* counter = counters + (size_t)blockIdx.z * kv_heads + g;
        if (threadIdx.x == 0) is_last = atomicAdd(counter, 1) == splits - 1;
        __syncthreads();
        if (is_last) {
            __threadfence();
            // One round trip to memory: every thread first asks for the maxima and sums of the ranges
            // (rows x ranges pairs, to shared memory) and for its share of the partial outputs (to
            // registers), and only then are the ranges' weights worked out and applied.
            float* stats = (float*)tiles;                        // [MAX_ROWS][splits][2]: maximum, sum
            constexpr int PER_THREAD = (MAX_ROWS * D + THREADS - 1) / THREADS;
            constexpr int SPLITS_IN_REGS = 8;
            float held[PER_THREAD][SPLITS_IN_REGS];
            const bool in_regs = splits <= SPLITS_IN_REGS;
            if (in_regs) {
#pragma unroll
                for (int i = 0; i < PER_THREAD; ++i) {
                    const int idx = threadIdx.x + i * THREADS;
                    if (idx < M * D) {
                        const int row = idx / D, d = idx % D;
                        const size_t out_row = (size_t)(q0 + row / ratio) * heads + g * ratio + row % ratio;
                        const float* src = partial + out_row * splits * (D + 2) + d;
#pragma unroll
                        for (int s2 = 0; s2 < SPLITS_IN_REGS; ++s2)
                            if (s2 < splits) held[i][s2] = __ldcg(src + (size_t)s2 * (D + 2));
                    }
                }
            }
            for (int idx = threadIdx.x; idx < M * splits; idx += THREADS) {
                const int row = idx / splits, s2 = idx % splits;
                const size_t orow = (size_t)(q0 + row / ratio) * heads + g * ratio + row % ratio;
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(partial + (orow * splits + s2) * (D + 2) + D));
                stats[2 * idx] = ml.x;
                stats[2 * idx + 1] = ml.y;
            }
            __syncthreads();
            float* row_scale = stats + 2 * MAX_ROWS * splits;    // [MAX_ROWS]: 1 / l
            if (threadIdx.x < M) {
                const int row = threadIdx.x;
                float mm = -INFINITY;
                for (int s2 = 0; s2 < splits; ++s2) mm = fmaxf(mm, stats[2 * (row * splits + s2)]);
                float l = 0.0f;
                for (int s2 = 0; s2 < splits; ++s2) {
                    const float ms = stats[2 * (row * splits + s2)];
                    const float f = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
                    l += stats[2 * (row * splits + s2) + 1] * f;
                    stats[2 * (row * splits + s2)] = f;          // the range's weight from here on
                }
                row_scale[row] = 1.0f / l;
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < PER_THREAD; ++i) {
                const int idx = threadIdx.x + i * THREADS;
                if (idx < M * D) {
                    const int row = idx / D, d = idx % D;
                    const size_t out_row = (size_t)(q0 + row / ratio) * heads + g * ratio + row % ratio;
                    float acc = 0.0f;
                    if (in_regs) {
#pragma unroll
                        for (int s2 = 0; s2 < SPLITS_IN_REGS; ++s2)
                            if (s2 < splits) acc = fmaf(held[i][s2], stats[2 * (row * splits + s2)], acc);
                    } else {
                        const float* src = partial + out_row * splits * (D + 2) + d;
#pragma unroll 8
                        for (int s2 = 0; s2 < splits; ++s2)
                            acc = fmaf(__ldcg(src + (size_t)s2 * (D + 2)), stats[2 * (row * splits + s2)], acc);
                    }
                    out[out_row * D + d] = __float2bfloat16_rn(acc * row_scale[row]);
                }
            }
            if (threadIdx.x == 0) *counter = 0;      // ready for the next launch
        }
    }
}

// out[row, head, :] = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m) over the key ranges.
template <int D>
__global__ void attn_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                  const int* __restrict__ req_list, const int* __restrict__ row_start,
                                  const int* __restrict__ row_count, int heads, int splits) {
    pdl_trigger();
    pdl_wait();
    const int r = req_list[blockIdx.z];
    if ((int)blockIdx.y >= row_count[r]) return;
    const size_t out_row = (size_t)(row_start[r] + blockIdx.y) * heads + blockIdx.x;
    const float* src = partial + out_row * splits * (D + 2);
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, src[(size_t)s * (D + 2) + D]);
    float l = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = src[(size_t)s * (D + 2) + D];
        l += ms == -INFINITY ? 0.0f : src[(size_t)s * (D + 2) + D + 1] * exp2f(ms - mm);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float ms = src[(size_t)s * (D + 2) + D];
            if (ms != -INFINITY) acc += src[(size_t)s * (D + 2) + d] * exp2f(ms - mm);
        }
        out[out_row * D + d] = __float2bfloat16_rn(acc / l);
    }
}

constexpr int MAX_CLUSTER = 16;     // blocks a cluster may have (more than 8 is allowed on request: B200 takes 16)
int g_cluster_merge = 1;            // llmx_attn_decode_cluster_merge(0) turns the clusters off

// Whether a cluster of `size` of these blocks can run at all on this device (asked once per size).
// How many clusters of `size` of these blocks the device runs at once (0: such a cluster cannot run; -1: the device
// gave no answer; asked once).
template <int D>
int max_clusters(int size) {
    static int known[MAX_CLUSTER + 1] = {0};         // 0: not asked yet, -1: none, -2: no answer, else the number
    if (!known[size]) {
        cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM_BYTES);
        if (size > 8 && cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
                            cudaSuccess)
            cudaGetLastError();         // then the query below says that such a cluster cannot run
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3(size, 1, 1);
        lc.blockDim = dim3(THREADS);
        lc.dynamicSmemBytes = Cfg<D>::SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)size;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
        int clusters = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, attn_decode_kernel<D>, &lc);
        if (e != cudaSuccess) cudaGetLastError();
        known[size] = e != cudaSuccess ? -2 : clusters > 0 ? clusters : -1;
    }
    return known[size] > 0 ? known[size] : known[size] == -2 ? -1 : 0;
}

template <int D>
int launch(const CUtensorMap& map, const void* q, void* out, float* partial, const int* req_list, int n_req,
           const int* row_start, const int* row_count, const int* history, const int* block_tables, int table_stride,
           int heads, int kv_heads, int window, float scale, int splits, const int* chunk_ptr, int chunk_keys,
           int max_rows, int* counters, int* error_word, cudaStream_t stream, const QkvInput& made = QkvInput{}) {
    using cfg = Cfg<D>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES) !=
            cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    dim3 grid(splits, kv_heads, n_req);
    // Key ranges that are few enough to be one thread-block cluster meet in shared memory (no trip through
    // memory, no counter); the caller's `counters` say that it wants the ranges combined by this launch.
    if (counters && splits > 1 && splits <= MAX_CLUSTER && g_cluster_merge && max_clusters<D>(splits) > 0) {
        cudaLaunchConfig_t lc = {};
        lc.gridDim = grid;
        lc.blockDim = dim3(THREADS);
        lc.dynamicSmemBytes = cfg::SMEM_BYTES;
        lc.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = llmx_pdl_enabled() ? 2 : 1;
        cudaLaunchKernelEx(&lc, attn_decode_kernel<D>, map, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, partial, req_list,
                           row_start, row_count, history, block_tables, table_stride, heads, kv_heads, window,
                           scale * attn::LOG2E, splits, chunk_ptr, chunk_keys, counters, error_word, made, 1);
        return launch_status();
    }
    launch_kernel(attn_decode_kernel<D>, grid, dim3(THREADS), cfg::SMEM_BYTES, stream,
        map, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, partial, req_list, row_start, row_count, history,
        block_tables, table_stride, heads, kv_heads, window, scale * attn::LOG2E, splits, chunk_ptr, chunk_keys,
        counters, error_word, made, 0);
    int e = launch_status();
    if (e || splits == 1 || counters) return e;
    dim3 mgrid(heads, max_rows, n_req);
    launch_kernel(attn_merge_kernel<D>, mgrid, dim3(D < 128 ? D : 128), 0, stream, (const float*)partial,
                  (__nv_bfloat16*)out, req_list, row_start, row_count, heads, splits);
    return launch_status();
}

}  // namespace

// Key ranges of up to sixteen meet in a thread-block cluster's shared memory (on, the default) or, like more ranges,
// through memory and a counter (off); returns the setting before.
LLMX_EXPORT int llmx_attn_decode_cluster_merge(int on) {
    const int before = g_cluster_merge;
    g_cluster_merge = on ? 1 : 0;
    return before;
}

// How many clusters of `size` blocks (2..16) of the kernel for this head width the device runs at once; 0 if none
// (or if clusters are turned off), -1 if the device could not be asked: more (request, kv head) pairs than this and some clusters wait for a second round.
LLMX_EXPORT int llmx_attn_decode_max_clusters(int head_dim, int size) {
    if (size < 2 || size > MAX_CLUSTER || !g_cluster_merge) return 0;
    if (head_dim == 128) return max_clusters<128>(size);
    if (head_dim == 64) return max_clusters<64>(size);
    return 0;
}

// The TMA descriptor of one layer's cache [pages, 2, kv_heads, page_size, head_dim] (bfloat16): 128 bytes at `out`.
LLMX_EXPORT int llmx_attn_cache_map(void* out, const void* cache, long long pages, int kv_heads, int page_size,
                                    int head_dim) {
    if (head_dim % attn::BOX_COLS || page_size != PAGE || ((uintptr_t)cache & 15)) return LLMX_ERR_UNSUPPORTED;
    return llmx_make_cache_map((CUtensorMap*)out, cache, (uint64_t)pages, (uint64_t)kv_heads, (uint32_t)page_size,
                               (uint64_t)head_dim);
}

// Attention for the requests req_list[0..n_req): each brings row_count[r] rows (at most 16 / (heads / kv_heads))
// starting at row row_start[r] of q/out [rows, heads, head_dim]; history[r] keys precede them.
// Key ranges: `splits` ranges of `chunk` keys (a multiple of 64; read from chunk_ptr on the device when given).
// `partial` (float32, rows * heads * splits * (head_dim + 2)) is needed when splits > 1.
// `counters` (optional): n_req * kv_heads ints, zero before the first use and left zero by every launch; with
// them the block that finishes a (request, kv head) last combines its key ranges and no second kernel runs.
LLMX_EXPORT int llmx_attn_decode_fused(const void* cache_map, const void* q, void* out, float* partial,
                                       const int* req_list, int n_req, const int* row_start, const int* row_count,
                                       const int* history, const int* block_tables, int table_stride, int heads,
                                       int kv_heads, int head_dim, int page_size, int window, float scale, int splits,
                                       const int* chunk_ptr, int chunk_keys, int max_rows, int* counters,
                                       int* error_word, cudaStream_t stream) {
    if (n_req <= 0) return 0;
    if (page_size != PAGE || heads % kv_heads || heads / kv_heads > MAX_ROWS || splits < 1 || n_req > 65535 ||
        kv_heads > 65535 || (chunk_keys % 64) || max_rows < 1 || max_rows * (heads / kv_heads) > MAX_ROWS)
        return LLMX_ERR_UNSUPPORTED;
    if (splits > 1 && !partial) return LLMX_ERR_BAD_ARGUMENT;
    if (counters && splits > 256) return LLMX_ERR_UNSUPPORTED;     // the ranges' weights go through shared memory
    const CUtensorMap& map = *(const CUtensorMap*)cache_map;
    switch (head_dim) {
        case 64: return launch<64>(map, q, out, partial, req_list, n_req, row_start, row_count, history, block_tables,
                                   table_stride, heads, kv_heads, window, scale, splits, chunk_ptr, chunk_keys, max_rows,
                                   counters, error_word, stream);
        case 128: return launch<128>(map, q, out, partial, req_list, n_req, row_start, row_count, history, block_tables,
                                     table_stride, heads, kv_heads, window, scale, splits, chunk_ptr, chunk_keys,
                                     max_rows, counters, error_word, stream);
        default: return LLMX_ERR_UNSUPPORTED;
    }
}

// The same for a step in which every request brings few rows, given the float32 output of the q/k/v product
// [rows, qkv_stride] instead of finished queries: each block norms and rotates its own queries, and the block
// whose key range holds a new row norms and rotates that key, stores key and value to the cache and lays them
// over the page it has fetched.  Head width 128, rotated whole (cos/sin [positions, 64]) or not at all (null).
// `slots` [rows]: page * 16 + slot of a row's key and value, negative when this layer does not write them.
LLMX_EXPORT int llmx_attn_decode_qkv(const void* cache_map, const float* qkv, int qkv_stride, int k_offset,
                                     int v_offset, const float* q_weight, const float* k_weight, float eps,
                                     const float* cos_table, const float* sin_table, const int* slots, void* cache,
                                     void* out, float* partial, const int* req_list, int n_req, const int* row_start,
                                     const int* row_count, const int* history, const int* block_tables,
                                     int table_stride, int heads, int kv_heads, int head_dim, int page_size, int window,
                                     float scale, int splits, const int* chunk_ptr, int chunk_keys, int max_rows,
                                     int* counters, int* error_word, cudaStream_t stream) {
    if (n_req <= 0) return 0;
    if (head_dim != 128 || page_size != PAGE || heads % kv_heads || heads / kv_heads > MAX_ROWS || splits < 1 ||
        n_req > 65535 || kv_heads > 65535 || (chunk_keys % 64) || max_rows < 1 ||
        max_rows * (heads / kv_heads) > MAX_ROWS)
        return LLMX_ERR_UNSUPPORTED;
    if (!qkv || !slots || !cache || (splits > 1 && (!partial || !counters)) || (!cos_table) != (!sin_table))
        return LLMX_ERR_BAD_ARGUMENT;
    if (qkv_stride % 4 || k_offset % 4 || v_offset % 4 || ((uintptr_t)qkv & 15) || ((uintptr_t)cache & 15) ||
        ((uintptr_t)q_weight & 15) || ((uintptr_t)k_weight & 15) || ((uintptr_t)cos_table & 15) ||
        ((uintptr_t)sin_table & 15))
        return LLMX_ERR_UNSUPPORTED;
    if (splits > 256) return LLMX_ERR_UNSUPPORTED;
    QkvInput made;
    made.qkv = qkv; made.stride = qkv_stride; made.k_offset = k_offset; made.v_offset = v_offset;
    made.q_weight = q_weight; made.k_weight = k_weight; made.eps = eps;
    made.cos_table = cos_table; made.sin_table = sin_table; made.slots = slots; made.cache = (__nv_bfloat16*)cache;
    return launch<128>(*(const CUtensorMap*)cache_map, nullptr, out, partial, req_list, n_req, row_start, row_count,
                       history, block_tables, table_stride, heads, kv_heads, window, scale, splits, chunk_ptr, chunk_keys,
                       max_rows, counters, error_word, stream, made);
}

// The same with a second kernel combining the key ranges (no counters needed).
LLMX_EXPORT int llmx_attn_decode(const void* cache_map, const void* q, void* out, float* partial, const int* req_list,
                                 int n_req, const int* row_start, const int* row_count, const int* history,
                                 const int* block_tables, int table_stride, int heads, int kv_heads, int head_dim,
                                 int page_size, int window, float scale, int splits, const int* chunk_ptr,
                                 int chunk_keys, int max_rows, int* error_word, cudaStream_t stream) {
    return llmx_attn_decode_fused(cache_map, q, out, partial, req_list, n_req, row_start, row_count, history,
                                  block_tables, table_stride, heads, kv_heads, head_dim, page_size, window, scale, splits,
                                  chunk_ptr, chunk_keys, max_rows, nullptr, error_word, stream);
}

// ---------------------------------------------------------------------------------------------
// A variant of llmx_attn_decode for callers that cannot allocate device memory (declared in
// attention_decode_static.h).  The partial results of the key ranges go to a fixed array in this
// library's own device memory instead of a workspace the caller provides.
// ---------------------------------------------------------------------------------------------
#include "attention_decode_static.h"

namespace {
// Held by every GPU that loads this library, from load until the process exits.
static __device__ __align__(256) float g_static_partial[LLMX_ATTN_DECODE_STATIC_FLOATS];
constexpr int MAX_DEVICES = 64;
float* g_static_partial_ptr[MAX_DEVICES] = {nullptr};
}  // namespace

LLMX_EXPORT int llmx_attn_decode_static(const void* cache_map, const void* q, void* out, const int* req_list,
                                        int n_req, const int* row_start, const int* row_count, const int* history,
                                        const int* block_tables, int table_stride, int total_rows, int heads,
                                        int kv_heads, int head_dim, int page_size, int window, float scale,
                                        int splits, int chunk_keys, int max_rows, int* error_word,
                                        cudaStream_t stream) {
    if (n_req <= 0) return 0;
    if (total_rows <= 0 || heads <= 0 || splits < 1 || head_dim <= 0) return LLMX_ERR_BAD_ARGUMENT;
    // The partial results of every (row, head, key range): refuse what the fixed array cannot hold.
    const long long need = (long long)total_rows * heads * splits * (head_dim + 2);
    if (splits > 1 && need > (long long)LLMX_ATTN_DECODE_STATIC_FLOATS) return LLMX_ERR_TOO_LARGE;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return LLMX_ERR_BAD_ARGUMENT;
    if (!g_static_partial_ptr[device]) {
        // In host code the array's name is only a handle; the kernel needs its address on this device.
        float* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_partial);
        if (e != cudaSuccess || !ptr) return e != cudaSuccess ? (int)e : LLMX_ERR_BAD_ARGUMENT;
        g_static_partial_ptr[device] = ptr;
    }
    return llmx_attn_decode(cache_map, q, out, g_static_partial_ptr[device], req_list, n_req, row_start, row_count,
                            history, block_tables, table_stride, heads, kv_heads, head_dim, page_size, window, scale,
                            splits, nullptr, chunk_keys, max_rows, error_word, stream);
}
