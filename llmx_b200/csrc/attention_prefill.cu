// Tiled causal attention over block tables for requests that bring a portion of a prompt.
//
// A block serves one (request, kv head, tile of new rows): `tokens_per_tile` consecutive new rows
// times the `ratio` query heads of the group make up to 128 query rows, 16 per consumer warp, that
// share the keys and values streamed through shared memory (measured: eight consumer warps in one
// block per SM beat four in each of two blocks, 32.9 against 34.9 ms for a 36-layer 2,048-token step):
//
//   producer warp     fetches the request's pages with TMA (boxes of [16 slots, 64 columns],
//                     128-byte swizzle), 64 keys a stage, three stages in flight
//   8 consumer warps  each holds 16 query rows: S = Q K^T over the stage's 64 keys (mma.sync
//                     m16n8k16), causal / window / tail masks where the tile touches them, online
//                     softmax in float32 (base 2), O += P V; at the end O / l is written as bfloat16.
//
// Row i of a tile is (new row i / ratio, head g * ratio + i % ratio), so any head ratio up to 16
// works; rows beyond the tile's tokens are masked.  History keys (earlier portions of the same
// prompt) are read from the same pages, so a prompt cut anywhere gives the same sums in the same
// order for a row: key tiles always start at a multiple of 64 keys from the request's first page.
// Reference counterpart: llmx_attention_tile (src/backends/gpu/kernels/f32.gpu:1498-1636).
#include "attn_common.cuh"
#include <math.h>

namespace {

constexpr int PAGE = 16;
constexpr int KEYS = 64;                 // keys per stage
constexpr int PAGES_PER_STAGE = KEYS / PAGE;
constexpr int STAGES = 3;
constexpr int CONSUMERS = 8;
constexpr int ROWS = CONSUMERS * 16;
constexpr int THREADS = (CONSUMERS + 1) * 32;
enum : int { ERR_PRE_PRODUCER = 301, ERR_PRE_CONSUMER = 302 };

template <int D>
struct Cfg {
    static constexpr int BOXES = D / attn::BOX_COLS;
    static constexpr int BOX_BYTES = PAGE * 128;
    static constexpr int PLANE_BYTES = BOXES * BOX_BYTES;
    static constexpr int PAGE_BYTES = 2 * PLANE_BYTES;
    static constexpr int STAGE_BYTES = PAGES_PER_STAGE * PAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 128;
};

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const __grid_constant__ CUtensorMap cache_map, const __nv_bfloat16* __restrict__ q,
                    __nv_bfloat16* __restrict__ out, const int* __restrict__ req_list,
                    const int* __restrict__ row_start, const int* __restrict__ row_count,
                    const int* __restrict__ history, const int* __restrict__ block_tables, int table_stride,
                    int heads, int kv_heads, int window, float scale_log2, int tokens_per_tile, int* error_word) {
    pdl_trigger();
    pdl_wait();
    using cfg = Cfg<D>;
    const int r = req_list[blockIdx.z], g = blockIdx.y;
    const int n_q = row_count[r];
    const int n_tiles = (n_q + tokens_per_tile - 1) / tokens_per_tile;
    if ((int)blockIdx.x >= n_tiles) return;
    const int tile = n_tiles - 1 - blockIdx.x;          // the tiles with the most keys start first
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(tiles + STAGES * cfg::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    volatile int* abort_flag = (volatile int*)(empty_bar + STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ratio = heads / kv_heads;
    const int q0 = row_start[r], hist = history[r];
    const int t0 = tile * tokens_per_tile;                          // first new row of the tile
    const int t_count = min(tokens_per_tile, n_q - t0);
    const int M = t_count * ratio;
    const int len = hist + n_q;
    const int last_pos = hist + t0 + t_count - 1;
    int kv_begin = 0;
    if (window > 0) kv_begin = (max(0, hist + t0 - window + 1) / KEYS) * KEYS;
    const int kv_end = last_pos + 1;
    const int iters = (kv_end - kv_begin + KEYS - 1) / KEYS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], CONSUMERS);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();

    if (warp == CONSUMERS) {
        if (tc::elect_one()) {
            tc::tma_prefetch_desc(&cache_map);
            const int* table = block_tables + (size_t)r * table_stride + kv_begin / PAGE;
            const int n_pages = (kv_end - kv_begin + PAGE - 1) / PAGE;
            // The page ids of a stage are read one stage ahead, so the table's latency is off the critical path.  With a
            // window the first stage starts at a stage boundary below the lowest key a row needs, where the request may
            // have given its pages back (id -1): those keys are masked whatever they hold, so page 0 stands in.
            int ids[PAGES_PER_STAGE], ids_next[PAGES_PER_STAGE];
#pragma unroll
            for (int p = 0; p < PAGES_PER_STAGE; ++p) ids_next[p] = p < n_pages ? max(table[p], 0) : 0;
            for (int it = 0; it < iters; ++it) {
                const int stage = it % STAGES;
                const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
#pragma unroll
                for (int p = 0; p < PAGES_PER_STAGE; ++p) {
                    ids[p] = ids_next[p];
                    const int nxt = (it + 1) * PAGES_PER_STAGE + p;
                    ids_next[p] = nxt < n_pages ? max(table[nxt], 0) : 0;
                }
                if (!tc::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, error_word, ERR_PRE_PRODUCER)) break;
                const int here = min(PAGES_PER_STAGE, n_pages - it * PAGES_PER_STAGE);
                tc::mbar_expect_tx(&full_bar[stage], (uint32_t)(here * cfg::PAGE_BYTES));
#pragma unroll
                for (int p = 0; p < PAGES_PER_STAGE; ++p) {
                    if (p >= here) break;
                    const int page = ids[p];
                    uint8_t* dst = tiles + stage * cfg::STAGE_BYTES + p * cfg::PAGE_BYTES;
                    // One copy brings the head's keys and values of the page: [plane][half][slot][64 columns].
                    tc::tma_load_5d(dst, &cache_map, 0, 0, 0, g, page * 2, &full_bar[stage]);
                }
            }
        }
        return;
    }

    // ---- consumers: 16 query rows each
    uint32_t qa[D / 16][4];
    float o[D / 8][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    int pos[2], lo[2];
    bool valid[2];
    const int r0 = warp * 16 + (lane >> 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = r0 + 8 * half;
        valid[half] = row < M;
        const int ti = t0 + row / ratio;
        pos[half] = hist + ti;
        lo[half] = window > 0 ? max(0, pos[half] - window + 1) : 0;
        const __nv_bfloat16* src = q + ((size_t)(q0 + ti) * heads + g * ratio + row % ratio) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int d = kk * 16 + (lane & 3) * 2;
            qa[kk][half] = valid[half] ? *reinterpret_cast<const uint32_t*>(src + d) : 0u;
            qa[kk][half + 2] = valid[half] ? *reinterpret_cast<const uint32_t*>(src + d + 8) : 0u;
        }
    }
#pragma unroll
    for (int t = 0; t < D / 8; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[t][e] = 0.0f;
    // What this warp's rows can see: keys up to the position of its last row, from the lowest `lo` on.
    const int warp_first_row = warp * 16, warp_last_row = min(warp * 16 + 15, M - 1);
    const bool warp_active = warp_first_row < M;
    const int warp_max_pos = warp_active ? hist + t0 + warp_last_row / ratio : -1;
    const int warp_min_pos = hist + t0 + warp_first_row / ratio;
    const int warp_lo = window > 0 ? max(0, warp_min_pos - window + 1) : 0;

    for (int it = 0; it < iters; ++it) {
        const int stage = it % STAGES;
        const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
        if (!tc::mbar_wait(&full_bar[stage], phase, abort_flag, error_word, ERR_PRE_CONSUMER)) break;
        const int key0 = kv_begin + it * KEYS;
        if (warp_active && key0 <= warp_max_pos && key0 + KEYS > warp_lo) {
            const uint32_t sbase = tc::smem_u32(tiles + stage * cfg::STAGE_BYTES);
            // Keys the tile may not use: past the request's last key (stale contents of a reused page) or in
            // pages of this stage that were not fetched (shared memory never written).  Their scores are
            // masked; their values are zeroed so that a non-finite leftover cannot reach the sum through a
            // zero weight.
            const int usable_end = min(len, kv_begin + ((kv_end - kv_begin + PAGE - 1) / PAGE) * PAGE);
            if (key0 + KEYS > usable_end) {
                const int first_bad = max(usable_end - key0, 0);
                for (int i = lane; i < (KEYS - first_bad) * cfg::BOXES * 8; i += 32) {
                    const int key = first_bad + i / (cfg::BOXES * 8), c = i % (cfg::BOXES * 8);
                    const uint32_t addr = sbase + (key / PAGE) * cfg::PAGE_BYTES + cfg::PLANE_BYTES +
                                          (c >> 3) * cfg::BOX_BYTES + attn::swz(key % PAGE, c & 7);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
                }
                __syncwarp();
            }
            float s[KEYS / 8][4];
#pragma unroll
            for (int j = 0; j < KEYS / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int dchunk = 2 * kk + ((lane >> 3) & 1);
#pragma unroll
                for (int jp = 0; jp < KEYS / 16; ++jp) {         // 16 keys = one page = two n-tiles
                    const int key = ((lane >> 4) << 3) + (lane & 7);
                    uint32_t b0, b1, b2, b3;
                    attn::ldmatrix_x4(sbase + jp * cfg::PAGE_BYTES + (dchunk >> 3) * cfg::BOX_BYTES +
                                      attn::swz(key, dchunk & 7), b0, b1, b2, b3);
                    attn::mma_16816(s[2 * jp], qa[kk], b0, b1);
                    attn::mma_16816(s[2 * jp + 1], qa[kk], b2, b3);
                }
            }
            // Masks are needed only where the tile of keys reaches past a row's position or below its window.
            const bool need_mask = key0 + KEYS - 1 > warp_min_pos || (window > 0 && key0 < max(0, warp_max_pos - window + 1)) ||
                                   !valid[1];
            float rowmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < KEYS / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    float v = s[j][e] * scale_log2;
                    if (need_mask) {
                        const int key = key0 + 8 * j + (lane & 3) * 2 + (e & 1);
                        if (!(valid[half] && key >= lo[half] && key <= pos[half])) v = -INFINITY;
                    }
                    s[j][e] = v;
                    rowmax[half] = fmaxf(rowmax[half], v);
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
            for (int j = 0; j < KEYS / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[j][e] = exp2f(s[j][e] - base[e >> 1]);
                    psum[e >> 1] += s[j][e];
                }
            l_run[0] = l_run[0] * alpha[0] + psum[0];
            l_run[1] = l_run[1] * alpha[1] + psum[1];
#pragma unroll
            for (int t = 0; t < D / 8; ++t) {
                o[t][0] *= alpha[0]; o[t][1] *= alpha[0]; o[t][2] *= alpha[1]; o[t][3] *= alpha[1];
            }
#pragma unroll
            for (int jp = 0; jp < KEYS / 16; ++jp) {
                uint32_t pa[4];
                pa[0] = attn::pack_bf16(s[2 * jp][0], s[2 * jp][1]);
                pa[1] = attn::pack_bf16(s[2 * jp][2], s[2 * jp][3]);
                pa[2] = attn::pack_bf16(s[2 * jp + 1][0], s[2 * jp + 1][1]);
                pa[3] = attn::pack_bf16(s[2 * jp + 1][2], s[2 * jp + 1][3]);
                const uint32_t vbase = sbase + jp * cfg::PAGE_BYTES + cfg::PLANE_BYTES;
#pragma unroll
                for (int t = 0; t < D / 8; t += 2) {
                    const int key = (((lane >> 3) & 1) << 3) + (lane & 7);
                    const int dchunk = t + (lane >> 4);
                    uint32_t b0, b1, b2, b3;
                    attn::ldmatrix_x4_trans(vbase + (dchunk >> 3) * cfg::BOX_BYTES + attn::swz(key, dchunk & 7), b0, b1, b2, b3);
                    attn::mma_16816(o[t], pa, b0, b1);
                    attn::mma_16816(o[t + 1], pa, b2, b3);
                }
            }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&empty_bar[stage]);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
        l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
        const int row = r0 + 8 * half;
        if (row >= M) continue;
        const int ti = t0 + row / ratio;
        __nv_bfloat16* dst = out + ((size_t)(q0 + ti) * heads + g * ratio + row % ratio) * D;
        const float inv = 1.0f / l_run[half];
#pragma unroll
        for (int t = 0; t < D / 8; ++t) {
            const int d = 8 * t + (lane & 3) * 2;
            *reinterpret_cast<uint32_t*>(dst + d) = attn::pack_bf16(o[t][2 * half] * inv, o[t][2 * half + 1] * inv);
        }
    }
}

template <int D>
int launch(const CUtensorMap& map, const void* q, void* out, const int* req_list, int n_req, const int* row_start,
           const int* row_count, const int* history, const int* block_tables, int table_stride, int heads,
           int kv_heads, int window, float scale, int max_rows, int* error_word, cudaStream_t stream) {
    using cfg = Cfg<D>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 cfg::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int ratio = heads / kv_heads;
    const int tokens_per_tile = ROWS / ratio;
    dim3 grid((max_rows + tokens_per_tile - 1) / tokens_per_tile, kv_heads, n_req);
    launch_kernel(attn_prefill_kernel<D>, grid, dim3(THREADS), cfg::SMEM_BYTES, stream,
        map, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, req_list, row_start, row_count, history, block_tables,
        table_stride, heads, kv_heads, window, scale * attn::LOG2E, tokens_per_tile, error_word);
    return launch_status();
}

}  // namespace

// Attention for the requests req_list[0..n_req), each bringing row_count[r] (<= max_rows) new rows after
// history[r] keys.  The cache map is the one llmx_attn_cache_map (attention_decode.cu) makes.
LLMX_EXPORT int llmx_attn_prefill(const void* cache_map, const void* q, void* out, const int* req_list, int n_req,
                                  const int* row_start, const int* row_count, const int* history,
                                  const int* block_tables, int table_stride, int heads, int kv_heads, int head_dim,
                                  int page_size, int window, float scale, int max_rows, int* error_word,
                                  cudaStream_t stream) {
    if (n_req <= 0 || max_rows <= 0) return 0;
    if (page_size != PAGE || heads % kv_heads || heads / kv_heads > 16 || n_req > 65535 || kv_heads > 65535)
        return LLMX_ERR_UNSUPPORTED;
    const CUtensorMap& map = *(const CUtensorMap*)cache_map;
    switch (head_dim) {
        case 64: return launch<64>(map, q, out, req_list, n_req, row_start, row_count, history, block_tables,
                                   table_stride, heads, kv_heads, window, scale, max_rows, error_word, stream);
        case 128: return launch<128>(map, q, out, req_list, n_req, row_start, row_count, history, block_tables,
                                     table_stride, heads, kv_heads, window, scale, max_rows, error_word, stream);
        default: return LLMX_ERR_UNSUPPORTED;
    }
}
