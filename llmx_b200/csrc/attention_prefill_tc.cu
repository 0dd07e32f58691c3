// Tiled causal attention for prompt portions on the 5th-generation tensor cores (head width 128).
//
// A work item is one (request, kv head, 2 * (128 / ratio) consecutive new rows): two row tiles, each 128 / ratio
// (rounded down) new rows times the `ratio` query heads of the group = the 128 rows of both products (with a ratio
// that does not divide 128 the last rows of a tile are padding: 25 tokens x 5 heads = 125 rows and 3 idle ones),
//     S[128 rows, 128 keys] = Q K^T        O[128 rows, 128 columns] += P V
// issued as tcgen05.mma by one thread.  The two row tiles share every key stage and take turns on the tensor
// core: while one tile's softmax runs, the other's products do.  A launch has one block of threads per SM at
// most; a block walks its share of the items (heavy and light ones in turn) without giving up its barriers
// and tensor memory, and fetches an item's first keys while the item before drains.
//
//   tensor memory   S of tile 0, S of tile 1, O of tile 0, O of tile 1: 4 x 128 columns.  P (bfloat16, two to a
//                   column) is written over the first 64 columns of the tile's S and is the P V product's A
//                   operand straight from tensor memory; O stays in tensor memory for the whole item.
//   warp 0          TMA producer: both Q tiles once (a 5-D box lays [token][head] rows out as the instruction's
//                   K-major operand), then 128 keys a stage, two stages, keys and values on barriers of their
//                   own; every lane issues one of the stage's 32 copies (8 pages x 2 halves x keys/values).
//                   Keys are K-major for Q K^T, values the MN-major operand of P V: neither is transposed.
//   warp 1          allocates tensor memory and issues the products in the order
//                   P V (tile 0, j), Q K^T (tile 0, j + 1), P V (tile 1, j), Q K^T (tile 1, j + 1), ...
//   warps 2-5, 6-9  one thread per query row of tile 0 / tile 1: read the row's 128 scores (tcgen05.ld), mask
//                   (causal, window), online softmax in float32 (base 2), write P (tcgen05.st).  The exponent
//                   uses a row maximum that is only raised when the true one has grown by more than 2^8; then
//                   the thread rescales its row of O in tensor memory.  P <= 256 and the sums stay exact
//                   in the same sense: O / l does not depend on which maximum was used, beyond rounding.
//                   At the end O / l is written.
//
// Every wait on an mbarrier is bounded (see tc_common.cuh).  Shapes this kernel does not take (head width
// other than 128, more than 16 query heads a kv head, page size other than 16) run the warp-level
// kernel in attention_prefill.cu.
// Reference counterpart: llmx_attention_tile (src/backends/gpu/kernels/f32.gpu:1498-1636).
#include "attn_common.cuh"
#include <math.h>

namespace {

constexpr int D = 128;
constexpr int PAGE = 16;
constexpr int ROWS = 128;                 // query rows of a row tile (the instruction's M)
constexpr int KEYS = 128;                 // keys per stage (the instruction's N for Q K^T, its K for P V)
constexpr int PAGES_PER_STAGE = KEYS / PAGE;
constexpr int KV_STAGES = 2;
constexpr int TILE_WARPS = 4;             // softmax warps per row tile: one thread per row
constexpr int SOFTMAX_WARPS = 2 * TILE_WARPS;
constexpr int THREADS = 64 + SOFTMAX_WARPS * 32;
constexpr int HALF_BYTES = 128 * 128;     // 128 rows of 128 bytes: one 64-column half of an operand
constexpr int OPERAND_BYTES = 2 * HALF_BYTES;
constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;                      // keys, then values
constexpr int SMEM_Q = 0, SMEM_KV = 2 * OPERAND_BYTES;             // two Q tiles, then the stages
constexpr int SMEM_TILES = SMEM_KV + KV_STAGES * STAGE_BYTES;       // 196,608 bytes
constexpr int SMEM_BYTES = SMEM_TILES + 1024 + 256;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_O = 2 * KEYS;     // first column of the outputs
constexpr float RAISE = 8.0f;             // the exponent's maximum follows the true one when it is this far behind
constexpr int PART = D + 4;      // floats of one row's partial result: the output, the maximum, the sum (16-byte rows)
enum : int { ERR_TCA_PRODUCER = 401, ERR_TCA_MMA = 402, ERR_TCA_SOFTMAX = 403 };

// Instruction descriptors: bfloat16 in, float32 out, M = 128, N = 128; A K-major; B K-major (keys) or MN-major (values).
constexpr uint32_t IDESC_QK = tc::instr_desc_bf16(ROWS, KEYS);
constexpr uint32_t IDESC_PV = tc::instr_desc_bf16(ROWS, D) | (1u << 16);

// Shared-memory operand, MN-major, 128-byte swizzle: 64 elements of the MN dimension contiguous (128 bytes),
// rows (K) 128 bytes apart in groups of eight 1024 bytes apart (stride byte offset), the next 64-element
// block of the MN dimension `mn_block_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_block_bytes) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(mn_block_bytes >> 4) << 16) | (64ull << 32) |
           (1ull << 46) | (2ull << 61);
}

// 2^x in one instruction; -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Three-input maximum and two float32 operations per instruction (packed pairs in 64-bit registers).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap cache_map,
                       __nv_bfloat16* __restrict__ out, const int* __restrict__ req_list,
                       const int* __restrict__ row_start, const int* __restrict__ row_count,
                       const int* __restrict__ history, const int* __restrict__ block_tables, int table_stride,
                       int heads, int kv_heads, int window, float scale_log2, int n_req, int max_blocks, int item_tiles,
                       int key_splits, float* __restrict__ partial, int* error_word) {
    pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + SMEM_TILES);
    uint64_t* q_full = bars;                 // [1]
    uint64_t* k_full = bars + 1;             // [2 stages]
    uint64_t* v_full = bars + 3;             // [2 stages]
    uint64_t* k_empty = bars + 5;            // [2 stages]  free once the last Q K^T that reads the stage has run
    uint64_t* v_empty = bars + 7;            // [2 stages]  free once the last P V that reads the stage has run
    uint64_t* s_full = bars + 9;             // [2 tiles]   S of the tile is written (and, once more at the end, O)
    uint64_t* p_full = bars + 11;            // [2 tiles]   P of the tile is written, O rescaled if need be
    uint64_t* q_empty = bars + 13;           // [1]         the item's last Q K^T has run: Q may be overwritten
    uint64_t* o_read = bars + 14;            // [2 tiles]   the tile's softmax warps have read the item's output
    uint32_t* tmem_slot = (uint32_t*)(bars + 16);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ratio = heads / kv_heads;
    const int tokens_per_tile = ROWS / ratio;

    if (threadIdx.x == 0) {
        tc::mbar_init(q_full, 1);
        tc::mbar_init(q_empty, 1);
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(&k_full[i], 1);
            tc::mbar_init(&v_full[i], 1);
            tc::mbar_init(&k_empty[i], 1);
            tc::mbar_init(&v_empty[i], 1);
            tc::mbar_init(&s_full[i], 1);
            tc::mbar_init(&p_full[i], TILE_WARPS);
            tc::mbar_init(&o_read[i], TILE_WARPS);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::tma_prefetch_desc(&q_map);
        tc::tma_prefetch_desc(&cache_map);
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, TMEM_COLS);
        tc::tmem_relinquish();
    }
    // The value halves start as zeros: a stage's pages that are not fetched (past the block's last key)
    // then hold zeros or older finite values, never what the memory held before the launch.
    for (int i = threadIdx.x; i < KV_STAGES * OPERAND_BYTES / 16; i += THREADS) {
        const int stage = i / (OPERAND_BYTES / 16), off = i % (OPERAND_BYTES / 16);
        *reinterpret_cast<uint4*>(smem + SMEM_KV + stage * STAGE_BYTES + OPERAND_BYTES + off * 16) = make_uint4(0, 0, 0, 0);
    }
    // Rows of the Q tiles that no copy writes (a head ratio that does not divide 128 leaves 128 % ratio of them)
    // hold zeros: their scores and outputs are computed and never stored.  The 128-byte swizzle moves 16-byte pieces
    // within a row's 128 bytes only, so a row is the same bytes swizzled or not.
    for (int i = threadIdx.x; i < 4 * (ROWS - tokens_per_tile * ratio) * 8; i += THREADS) {
        const int half_of_tile = i / ((ROWS - tokens_per_tile * ratio) * 8), rest = i % ((ROWS - tokens_per_tile * ratio) * 8);
        *reinterpret_cast<uint4*>(smem + SMEM_Q + half_of_tile * HALF_BYTES + (tokens_per_tile * ratio + rest / 8) * 128 + (rest % 8) * 16) =
            make_uint4(0, 0, 0, 0);
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    // ---- The work: items (request, kv head, block of 2 x 128 / ratio new rows), the blocks with the most keys first.
    // A launch has at most one block of threads per SM; block c takes the items c, 2G - 1 - c, 2G + c, ... (G blocks:
    // back and forth over the list, so that each gets heavy and light ones), one after the other without giving up
    // its barriers and tensor memory.  Every role walks the same items and keeps count of the barrier phases it has
    // used, which go on from item to item.
    // With `key_splits` > 1 an item is further one of that many ranges of the block's key stages; its rows' sums over
    // the range (output not yet divided, maximum, sum) go to `partial`, and a second kernel adds the ranges up.
    const int per_block_row = kv_heads * n_req;
    const int per_block = per_block_row * key_splits;
    const int total_items = max_blocks * per_block;
    struct Item {
        int r, g, q0, hist, kv_begin, kv_end, n_iter, first_tile, last_tile, split;
        int tile_t0[2], tile_rows[2], tile_iters[2];
    };
    auto item_at = [&](int k, Item& it) -> bool {
        const int G = gridDim.x, c = blockIdx.x;
        const long long idx = (k & 1) ? (long long)(k + 1) * G - 1 - c : (long long)k * G + c;
        if (idx >= total_items) return false;
        const int xi = (int)(idx / per_block), rem2 = (int)(idx % per_block);
        const int rem = rem2 % per_block_row;
        it.split = rem2 / per_block_row;
        it.g = rem % kv_heads;
        it.r = req_list[rem / kv_heads];
        const int n_q = row_count[it.r];
        const int n_blocks = (n_q + item_tiles * tokens_per_tile - 1) / (item_tiles * tokens_per_tile);
        const bool active = xi < n_blocks;
        const int blk = active ? n_blocks - 1 - xi : 0;
        it.q0 = row_start[it.r];
        it.hist = history[it.r];
        const int t0 = blk * item_tiles * tokens_per_tile;
        const int begin0 = window > 0 ? (max(0, it.hist + t0 - window + 1) / KEYS) * KEYS : 0;
        // Per row tile: its first new row, how many it has, and how many key stages reach its last row.
        int full[2];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            it.tile_t0[t] = t0 + t * tokens_per_tile;
            const int count = active && t < item_tiles ? max(0, min(tokens_per_tile, n_q - it.tile_t0[t])) : 0;
            it.tile_rows[t] = count * ratio;
            full[t] = count > 0 ? (it.hist + it.tile_t0[t] + count - begin0 + KEYS - 1) / KEYS : 0;
        }
        // This item's share of the stages: the later rows see the most keys, so the block has max(full) of them.
        const int stages = max(full[0], full[1]);
        const int per = (stages + key_splits - 1) / key_splits;
        const int j0 = min(stages, it.split * per), j1 = min(stages, j0 + per);
#pragma unroll
        for (int t = 0; t < 2; ++t) it.tile_iters[t] = max(0, min(full[t], j1) - j0);
        it.first_tile = it.tile_iters[0] > 0 ? 0 : 1;
        it.last_tile = it.tile_iters[1] > 0 ? 1 : 0;
        it.n_iter = it.tile_iters[it.last_tile];
        it.kv_begin = begin0 + j0 * KEYS;
        it.kv_end = min(it.hist + min(n_q, t0 + item_tiles * tokens_per_tile), begin0 + j1 * KEYS);
        return true;
    };

    if (warp == 0) {
        // Lane = (keys or values, page of the stage, half of the head): one copy of 16 slots x 64 columns each.
        const int plane = lane >> 4, p = (lane >> 1) & 7, half = lane & 1;
        uint64_t* full = plane ? v_full : k_full;
        uint64_t* empty = plane ? v_empty : k_empty;
        uint32_t kv_uses = 0, items_done = 0;      // stage uses and items so far: they number the barriers' phases
        bool ok = true;
        Item it;
        for (int k = 0; ok && item_at(k, it); ++k) {
            if (it.n_iter == 0) continue;
            if (lane == 0) {
                // Q: rows [token][head of the group], one box per row tile and 64-column half (a half's rows are
                // tokens_per_tile * ratio <= 128, so the halves are copied apart, each to its own 16 KB); the item
                // before must be done with the buffer (its last Q K^T has run).
                ok = tc::mbar_wait(q_empty, (items_done & 1u) ^ 1u, abort_flag, error_word, ERR_TCA_PRODUCER);
                if (ok) {
                    tc::mbar_expect_tx(q_full, (uint32_t)((it.last_tile + 1) * 2 * tokens_per_tile * ratio * 128));
                    for (int t = 0; t <= it.last_tile; ++t)
                        for (int h = 0; h < 2; ++h)
                            tc::tma_load_5d(smem + SMEM_Q + t * OPERAND_BYTES + h * HALF_BYTES, &q_map, 0, 0, it.q0 + it.tile_t0[t], h,
                                            it.g, q_full);
                }
            }
            ++items_done;
            const int* table = block_tables + (size_t)it.r * table_stride + it.kv_begin / PAGE;
            const int n_pages = (it.kv_end - it.kv_begin + PAGE - 1) / PAGE;
            // A stage's page id is read one stage ahead, so the table's latency is off the copies' path.  With a window
            // the first stage starts at a stage boundary below the lowest key a row needs, where the request may have
            // given its pages back (id -1): those keys are masked whatever they hold, so page 0 stands in.
            int id_next = p < n_pages ? max(table[p], 0) : 0;
            for (int j = 0; j < it.n_iter; ++j, ++kv_uses) {
                const int st = kv_uses % KV_STAGES;
                const uint32_t ph = ((kv_uses / KV_STAGES) & 1u) ^ 1u;
                const int here = min(PAGES_PER_STAGE, n_pages - j * PAGES_PER_STAGE);
                const int id = id_next;
                const int nxt = (j + 1) * PAGES_PER_STAGE + p;
                id_next = nxt < n_pages ? max(table[nxt], 0) : 0;
                if (!tc::mbar_wait(&empty[st], ph, abort_flag, error_word, ERR_TCA_PRODUCER)) ok = false;
                // The bytes a phase expects must be announced before any of its copies can land (a copy that
                // completes first is not counted later): the half-warp's first lane announces, then all issue.
                if ((lane & 15) == 0 && ok) tc::mbar_expect_tx(&full[st], (uint32_t)(here * PAGE * D * 2));
                ok = __all_sync(plane ? 0xffff0000u : 0x0000ffffu, ok);
                if (!ok) break;
                if (p < here)
                    tc::tma_load_5d(smem + SMEM_KV + st * STAGE_BYTES + plane * OPERAND_BYTES + half * HALF_BYTES + p * PAGE * 128,
                                    &cache_map, 0, 0, half, it.g, id * 2 + plane, &full[st]);
            }
            ok = __all_sync(0xffffffffu, ok);
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            uint32_t kv_uses = 0, items_done = 0, p_done[2] = {0, 0}, tile_items[2] = {0, 0};
            bool ok = true;
            Item it;
            for (int k = 0; ok && item_at(k, it); ++k) {
                if (it.n_iter == 0) continue;
                ok = tc::mbar_wait(q_full, items_done & 1u, abort_flag, error_word, ERR_TCA_MMA);
                ++items_done;
                const uint32_t kv0 = kv_uses;              // the item's stage j is stage use kv0 + j
                // S of tile t = Q_t K_j^T.  The products of one thread run in the order they are issued, so this
                // one, issued after P V of (t, j - 1), also finds that product done with the columns it writes.
                auto issue_qk = [&](int t, int j) {
                    const uint32_t q_addr = tc::smem_u32(smem + SMEM_Q + t * OPERAND_BYTES);
                    const uint32_t k_addr = tc::smem_u32(smem + SMEM_KV + ((kv0 + j) % KV_STAGES) * STAGE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                        tc::mma_bf16_ss(tmem_base + t * KEYS, tc::smem_desc_k_sw128(q_addr + off),
                                        tc::smem_desc_k_sw128(k_addr + off), IDESC_QK, kk > 0 ? 1u : 0u);
                    }
                    tc::mma_commit(&s_full[t]);
                };
                // O of tile t += P V_j, P from the tile's tensor-memory columns.
                auto issue_pv = [&](int t, int j) -> bool {
                    const uint32_t use = kv0 + j;
                    const int st = use % KV_STAGES;
                    if (!tc::mbar_wait(&v_full[st], (use / KV_STAGES) & 1u, abort_flag, error_word, ERR_TCA_MMA)) return false;
                    if (!tc::mbar_wait(&p_full[t], p_done[t] & 1u, abort_flag, error_word, ERR_TCA_MMA)) return false;
                    ++p_done[t];
                    tc::tc_fence_after();
                    const uint32_t v_addr = tc::smem_u32(smem + SMEM_KV + st * STAGE_BYTES + OPERAND_BYTES);
#pragma unroll
                    for (int kk = 0; kk < KEYS / 16; ++kk)
                        tc::mma_bf16_ts(tmem_base + TMEM_O + t * D, tmem_base + t * KEYS + kk * 8,
                                        smem_desc_mn_sw128(v_addr + kk * 16 * 128, HALF_BYTES), IDESC_PV, (j > 0 || kk > 0) ? 1u : 0u);
                    return true;
                };
                if (ok) ok = tc::mbar_wait(&k_full[kv0 % KV_STAGES], (kv0 / KV_STAGES) & 1u, abort_flag, error_word, ERR_TCA_MMA);
                // A tile's first scores of an item complete s_full right after the item before completed it with
                // the tile's output; a waiter tells phases apart by parity only, so the tile's softmax warps must
                // have seen the one (and read the output) before the other may happen.
                for (int t = it.first_tile; t <= it.last_tile && ok; ++t) {
                    if (tile_items[t] > 0)
                        ok = tc::mbar_wait(&o_read[t], (tile_items[t] - 1) & 1u, abort_flag, error_word, ERR_TCA_MMA);
                    ++tile_items[t];
                }
                if (ok) {
                    tc::tc_fence_after();
                    for (int t = it.first_tile; t <= it.last_tile; ++t) issue_qk(t, 0);
                    tc::mma_commit(&k_empty[kv0 % KV_STAGES]);
                    if (it.n_iter == 1) tc::mma_commit(q_empty);          // the item's last Q K^T
                }
                for (int j = 0; j < it.n_iter && ok; ++j) {
                    for (int t = 0; t <= it.last_tile && ok; ++t) {
                        if (j >= it.tile_iters[t]) continue;
                        ok = issue_pv(t, j);
                        if (!ok) break;
                        if (t == it.last_tile) tc::mma_commit(&v_empty[(kv0 + j) % KV_STAGES]);
                        if (j + 1 < it.tile_iters[t]) {
                            const uint32_t use = kv0 + j + 1;
                            ok = tc::mbar_wait(&k_full[use % KV_STAGES], (use / KV_STAGES) & 1u, abort_flag, error_word, ERR_TCA_MMA);
                            if (!ok) break;
                            tc::tc_fence_after();
                            issue_qk(t, j + 1);
                            if (t == it.last_tile) {
                                tc::mma_commit(&k_empty[use % KV_STAGES]);
                                if (j + 2 == it.n_iter) tc::mma_commit(q_empty);      // the item's last Q K^T
                            }
                        } else {
                            tc::mma_commit(&s_full[t]);          // the tile's output is complete
                        }
                    }
                }
                kv_uses += it.n_iter;
            }
        }
    } else {
        // ---- one thread per query row: warps 2-5 serve tile 0, warps 6-9 tile 1; a warp may touch the
        // tensor-memory lanes 32 (warp % 4) .. + 31
        const int t = (warp - 2) / TILE_WARPS;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t s_addr = tmem_base + t * KEYS + ((uint32_t)(quarter * 32) << 16);
        const uint32_t o_addr = tmem_base + TMEM_O + t * D + ((uint32_t)(quarter * 32) << 16);
        uint32_t s_done = 0;                        // completions of this tile's s_full that have been waited for
        bool ok = true;
        Item it;
        for (int k = 0; ok && item_at(k, it); ++k) {
            const int M = it.tile_rows[t], iters = it.tile_iters[t];
            const int g = it.g, q0 = it.q0, hist = it.hist, kv_begin = it.kv_begin;
            const bool valid = row < M;
            const int ti = it.tile_t0[t] + min(row, max(M, 1) - 1) / ratio;
            // Where this row's sums over the item's key range go when the keys are cut into ranges.
            float* part = key_splits > 1
                ? partial + (((size_t)(q0 + ti) * heads + g * ratio + row % ratio) * key_splits + it.split) * PART
                : nullptr;
            if (iters == 0) {
                // None of the range's keys reach these rows: say so (maximum -inf, sum 0) and go on.
                if (part && valid) {
                    part[D] = -INFINITY;
                    part[D + 1] = 0.0f;
                }
                continue;
            }
            const int pos = hist + ti;
            const int lo = window > 0 ? max(0, pos - window + 1) : 0;
            float m_used = -INFINITY, l_run = 0.0f;
            for (int j = 0; j < iters; ++j) {
                ok = tc::mbar_wait(&s_full[t], s_done & 1u, abort_flag, error_word, ERR_TCA_SOFTMAX);
                if (!ok) break;
                ++s_done;
                tc::tc_fence_after();
                const int key0 = kv_begin + j * KEYS;
                const bool need_mask = key0 + KEYS - 1 > pos || key0 < lo;
                // ---- the row's raw scores (kept in registers) and their maximum; masked ones become -inf.
                // The scale is positive, so it is applied after the maximum and folded into the exponent's
                // multiply-add.
                uint32_t sc[KEYS];
#pragma unroll
                for (int c = 0; c < KEYS; c += 32) tc::tmem_ld_32x32(s_addr + c, *reinterpret_cast<uint32_t(*)[32]>(&sc[c]));
                tc::tmem_wait_ld();
                if (need_mask) {
#pragma unroll
                    for (int k = 0; k < KEYS; ++k) {
                        const int key = key0 + k;
                        if (key > pos || key < lo) sc[k] = __float_as_uint(-INFINITY);
                    }
                }
                // Four running maxima, three inputs an instruction: no long chain of dependent instructions.
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int k = 0; k < KEYS; k += 8) {
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        mx[u] = max3(mx[u], __uint_as_float(sc[k + 2 * u]), __uint_as_float(sc[k + 2 * u + 1]));
                }
                const float rowmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                const float cand = fmaxf(m_used, rowmax * scale_log2);
                // The maximum the exponent uses follows when, for some row of the warp, the true one is far ahead.
                const bool raise = j > 0 && __any_sync(0xffffffffu, cand > m_used + RAISE);
                const float factor = !raise || cand == -INFINITY ? 1.0f : exp2f(m_used - cand);
                if (j == 0 || raise) m_used = cand;
                const float base = m_used == -INFINITY ? 0.0f : m_used;
                // ---- P = 2^(s - m) as bfloat16, two keys to a column, over the scores' first 64 columns
                const uint64_t scale2 = pack2(scale_log2, scale_log2), minus_base2 = pack2(-base, -base);
                uint64_t sum2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
#pragma unroll
                for (int c = 0; c < KEYS; c += 32) {
                    uint32_t packed[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        const uint64_t x = fma2(pack2(__uint_as_float(sc[c + 2 * k]), __uint_as_float(sc[c + 2 * k + 1])),
                                                scale2, minus_base2);
                        float x0, x1;
                        unpack2(x, x0, x1);
                        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                        sum2[k & 1] = add2(sum2[k & 1], pack2(p0, p1));
                        packed[k] = attn::pack_bf16(p0, p1);
                    }
                    tc::tmem_st_32x16(s_addr + c / 2, packed);
                }
                float r0, r1, r2, r3;
                unpack2(sum2[0], r0, r1);
                unpack2(sum2[1], r2, r3);
                const float rowsum = (r0 + r1) + (r2 + r3);
                if (raise) {
                    // The row's output so far was summed against the old maximum.  P V of the stage before has
                    // finished (this stage's scores were written after it) and this stage's has not been
                    // issued (it waits for the arrival below), so O may be rewritten here.
#pragma unroll
                    for (int c = 0; c < D; c += 32) {
                        uint32_t v[32];
                        tc::tmem_ld_32x32(o_addr + c, v);
                        tc::tmem_wait_ld();
#pragma unroll
                        for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * factor);
                        tc::tmem_st_32x32(o_addr + c, v);
                    }
                    l_run *= factor;
                }
                l_run += rowsum;
                tc::tmem_wait_st();
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&p_full[t]);
            }
            // ---- O / l once the last P V has run
            if (ok) ok = tc::mbar_wait(&s_full[t], s_done & 1u, abort_flag, error_word, ERR_TCA_SOFTMAX);
            if (ok) {
                ++s_done;
                tc::tc_fence_after();
                const float inv = 1.0f / l_run;
                __nv_bfloat16* dst = out + ((size_t)(q0 + ti) * heads + g * ratio + row % ratio) * D;
                if (part && valid) {
                    part[D] = m_used;
                    part[D + 1] = l_run;
                }
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t v[32];
                    tc::tmem_ld_32x32(o_addr + c, v);
                    tc::tmem_wait_ld();
                    if (part) {
                        if (valid) {
#pragma unroll
                            for (int d = 0; d < 32; d += 4)
                                *reinterpret_cast<uint4*>(part + c + d) = make_uint4(v[d], v[d + 1], v[d + 2], v[d + 3]);
                        }
                    } else if (valid) {
#pragma unroll
                        for (int d = 0; d < 32; d += 8) {
                            const uint4 val = make_uint4(
                                attn::pack_bf16(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv),
                                attn::pack_bf16(__uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv),
                                attn::pack_bf16(__uint_as_float(v[d + 4]) * inv, __uint_as_float(v[d + 5]) * inv),
                                attn::pack_bf16(__uint_as_float(v[d + 6]) * inv, __uint_as_float(v[d + 7]) * inv));
                            *reinterpret_cast<uint4*>(dst + c + d) = val;
                        }
                    }
                }
                // The output has been read: the next item's products may write the tile's columns.
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&o_read[t]);
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Adds up the key ranges of a launch with `key_splits` > 1: one warp per (new row, head) reads the ranges' partial
// outputs o_s with their maxima m_s and sums l_s and writes  sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s.
__global__ void __launch_bounds__(128)
attn_prefill_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                          const int* __restrict__ req_list, const int* __restrict__ row_start,
                          const int* __restrict__ row_count, int heads, int key_splits) {
    pdl_trigger();
    pdl_wait();
    const int r = req_list[blockIdx.y];
    const int lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int ti = (int)(idx / heads), head = (int)(idx % heads);
    if (ti >= row_count[r]) return;
    const size_t slot = (size_t)(row_start[r] + ti) * heads + head;
    const float* base = partial + slot * key_splits * PART;
    float m = -INFINITY;
    for (int s = 0; s < key_splits; ++s) m = fmaxf(m, base[s * PART + D]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.0f;
    for (int s = 0; s < key_splits; ++s) {
        const float ls = base[s * PART + D + 1];
        if (ls > 0.0f) {                      // a range none of whose keys reached the row left its output unwritten
            const float w = exp2f(base[s * PART + D] - m);
            const float4 o = *reinterpret_cast<const float4*>(base + s * PART + 4 * lane);
            acc.x = fmaf(w, o.x, acc.x); acc.y = fmaf(w, o.y, acc.y);
            acc.z = fmaf(w, o.z, acc.z); acc.w = fmaf(w, o.w, acc.w);
            l = fmaf(w, ls, l);
        }
    }
    const float inv = 1.0f / l;
    *reinterpret_cast<uint2*>(out + slot * D + 4 * lane) =
        make_uint2(attn::pack_bf16(acc.x * inv, acc.y * inv), attn::pack_bf16(acc.z * inv, acc.w * inv));
}

// q [rows, heads, 128] bfloat16 as (64 columns) x (head within the group) x (row) x (half of the head) x (kv head):
// the box {64, ratio, 128 / ratio, 1, 1} is one half of a tile's Q operand, [row][head][64 columns] in shared memory.
int make_q_map(CUtensorMap* map, const void* q, uint64_t rows, int heads, int kv_heads) {
    llmx_encode_tiled_fn enc = llmx_encode_tiled();
    if (!enc) return 10003;
    const uint64_t ratio = heads / kv_heads;
    const cuuint64_t dims[5] = {64, ratio, rows, 2, (cuuint64_t)kv_heads};
    const cuuint64_t strides[4] = {D * 2, (cuuint64_t)heads * D * 2, 128, ratio * D * 2};
    const cuuint32_t box[5] = {64, (cuuint32_t)ratio, (cuuint32_t)(ROWS / ratio), 1, 1};
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(q), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 10003;
}

// The cache as (64 columns) x (slot) x (half) x (kv head) x (page * 2 + plane), box {64, 16, 1, 1, 1}: one half of
// one page's keys or values of one head, 16 rows of 128 bytes.
int make_cache_half_map(CUtensorMap* map, const void* cache, uint64_t pages, uint64_t kv_heads) {
    llmx_encode_tiled_fn enc = llmx_encode_tiled();
    if (!enc) return 10003;
    const cuuint64_t dims[5] = {64, PAGE, 2, kv_heads, pages * 2};
    const cuuint64_t strides[4] = {D * 2, 128, (cuuint64_t)PAGE * D * 2, kv_heads * PAGE * D * 2};
    const cuuint32_t box[5] = {64, PAGE, 1, 1, 1};
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 10003;
}

}  // namespace

// The descriptor of one cache entry's storage [pages, 2, kv_heads, 16, 128] for this kernel: 128 bytes at `out`.
LLMX_EXPORT int llmx_attn_prefill_tc_cache_map(void* out, const void* cache, long long pages, int kv_heads,
                                               int page_size, int head_dim) {
    if (head_dim != D || page_size != PAGE || ((uintptr_t)cache & 15)) return LLMX_ERR_UNSUPPORTED;
    return make_cache_half_map((CUtensorMap*)out, cache, (uint64_t)pages, (uint64_t)kv_heads);
}

// Attention for the requests req_list[0..n_req), each bringing row_count[r] (<= max_rows) new rows after history[r]
// keys; q/out [total_rows, heads, 128] bfloat16.  `item_tiles`: row tiles a work item holds (1 or 2; 0: chosen here).
// `key_splits` > 1 cuts every item's keys into that many ranges, whose results meet in `partial` (float32,
// total_rows * heads * key_splits * 132 values, 16-byte aligned) and are added up by a second kernel.
LLMX_EXPORT int llmx_attn_prefill_tc(const void* cache_map, const void* q, void* out, int total_rows,
                                     const int* req_list, int n_req, const int* row_start, const int* row_count,
                                     const int* history, const int* block_tables, int table_stride, int heads,
                                     int kv_heads, int head_dim, int page_size, int window, float scale, int max_rows,
                                     int item_tiles, int key_splits, float* partial, int* error_word,
                                     cudaStream_t stream) {
    if (n_req <= 0 || max_rows <= 0) return 0;
    if (head_dim != D || page_size != PAGE || heads % kv_heads || heads / kv_heads > 16 || n_req > 65535 ||
        kv_heads > 65535 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15))
        return LLMX_ERR_UNSUPPORTED;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
            cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    CUtensorMap q_map;
    if (int e = make_q_map(&q_map, q, (uint64_t)total_rows, heads, kv_heads)) return e;
    if (item_tiles < 0 || item_tiles > 2 || key_splits < 1 || (key_splits > 1 && (!partial || ((uintptr_t)partial & 15))))
        return LLMX_ERR_BAD_ARGUMENT;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    // A work item is two row tiles that share their key stages and take turns on the tensor core -- unless twice as
    // many items of one tile still find an SM each (a short portion, few kv heads): the longest item is what the
    // kernel's time comes to then, and a one-tile item is half as long (512 rows after 4,096 keys: 77 -> 69 us).
    const int tokens_per_tile = ROWS / (heads / kv_heads);
    if (item_tiles == 0) {
        const long long pairs = (long long)((max_rows + 2 * tokens_per_tile - 1) / (2 * tokens_per_tile)) * kv_heads * n_req;
        item_tiles = 2 * pairs <= sm_count ? 1 : 2;
    }
    const int tokens_per_block = item_tiles * tokens_per_tile;
    const int max_blocks = (max_rows + tokens_per_block - 1) / tokens_per_block;
    // One block of threads per SM at most (a block takes the SM's shared and tensor memory); each walks its items.
    const long long items = (long long)max_blocks * kv_heads * n_req * key_splits;
    if (items >= (1ll << 31)) return LLMX_ERR_UNSUPPORTED;
    dim3 grid((unsigned)(items < sm_count ? items : sm_count), 1, 1);
    launch_kernel(attn_prefill_tc_kernel, grid, dim3(THREADS), (size_t)SMEM_BYTES, stream, q_map,
                  *(const CUtensorMap*)cache_map, (__nv_bfloat16*)out, req_list, row_start, row_count, history,
                  block_tables, table_stride, heads, kv_heads, window, scale * attn::LOG2E, n_req, max_blocks, item_tiles,
                  key_splits, partial, error_word);
    if (int e = launch_status()) return e;
    if (key_splits > 1) {
        const long long warps = (long long)max_rows * heads;
        launch_kernel(attn_prefill_merge_kernel, dim3((unsigned)((warps + 3) / 4), (unsigned)n_req, 1), dim3(128), 0, stream,
                      (const float*)partial, (__nv_bfloat16*)out, req_list, row_start, row_count, heads, key_splits);
    }
    return launch_status();
}
