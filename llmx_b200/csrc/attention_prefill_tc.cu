// Tiled causal attention for prompt portions on the 5th-generation tensor cores (head width 128).
//
// A block serves one (request, kv head, tile of new rows): 128 / ratio consecutive new rows times the
// `ratio` query heads of the group are the 128 rows of both products,
//     S[128 rows, 128 keys] = Q K^T        O[128 rows, 128 columns] += P V
// issued as tcgen05.mma by one thread, with S and P V in tensor memory:
//
//   warp 0      TMA producer: the Q tile once (a 5-D box that lays [token][head] rows out as the
//               instruction's K-major operand), then 128 keys a stage, two stages: the request's pages
//               into [half of the head][key][64 columns] (keys K-major for Q K^T, values as the
//               MN-major operand of P V, so neither is transposed)
//   warp 1      allocates tensor memory (two S and two P V accumulators, 512 columns) and issues the
//               products: Q K^T of tile j + 1 goes out before P V of tile j, so the tensor core works
//               while tile j's softmax runs; P has two buffers too, so tile j + 1's P is written while
//               P V of tile j reads its own
//   warps 2-9   two threads per query row, each with 64 of the row's 128 columns: read S from tensor
//               memory (tcgen05.ld), mask (causal, window), online softmax in float32 (base 2; the two
//               halves of a row exchange their maxima through shared memory), write P as bfloat16
//               into shared memory in the operand layout, then fold the finished P V of the tile
//               before into the row's running output (registers): O = O * 2^(m_old - m_new) + P V.
//               At the end O / l is written.
//
// Every wait on an mbarrier is bounded (see tc_common.cuh).  Shapes this kernel does not take (head width
// other than 128, a head ratio that does not divide 128, page size other than 16) run the warp-level
// kernel in attention_prefill.cu.
// Reference counterpart: llmx_attention_tile (src/backends/gpu/kernels/f32.gpu:1498-1636).
#include "attn_common.cuh"
#include <math.h>

namespace {

constexpr int D = 128;
constexpr int PAGE = 16;
constexpr int ROWS = 128;                 // query rows of a tile (the instruction's M)
constexpr int KEYS = 128;                 // keys per stage (the instruction's N for Q K^T, its K for P V)
constexpr int PAGES_PER_STAGE = KEYS / PAGE;
constexpr int KV_STAGES = 2;
constexpr int SOFTMAX_WARPS = 8;          // two warps per 32 rows: each takes 64 of a row's 128 columns
constexpr int THREADS = 64 + SOFTMAX_WARPS * 32;
constexpr int HALF_BYTES = 128 * 128;     // 128 rows of 128 bytes: one 64-column half of an operand
constexpr int OPERAND_BYTES = 2 * HALF_BYTES;
constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;                      // keys, then values
constexpr int SMEM_Q = 0, SMEM_P = OPERAND_BYTES, SMEM_KV = 3 * OPERAND_BYTES;    // Q, two P buffers, then the stages
constexpr int SMEM_TILES = SMEM_KV + KV_STAGES * STAGE_BYTES;       // 229,376 bytes
constexpr int SMEM_BYTES = SMEM_TILES + 1024 + 256 + 2 * ROWS * 4;   // + the rows' maxima of both column halves
constexpr uint32_t TMEM_COLS = 512;
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

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap cache_map,
                       __nv_bfloat16* __restrict__ out, const int* __restrict__ req_list,
                       const int* __restrict__ row_start, const int* __restrict__ row_count,
                       const int* __restrict__ history, const int* __restrict__ block_tables, int table_stride,
                       int heads, int kv_heads, int window, float scale_log2, int* error_word) {
    pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + SMEM_TILES);
    uint64_t* q_full = bars;                 // [1]
    uint64_t* kv_full = bars + 1;            // [2]
    uint64_t* k_empty = bars + 3;            // [2]  keys of a stage are free once Q K^T has read them
    uint64_t* s_full = bars + 5;             // [2]
    uint64_t* s_empty = bars + 7;            // [2]
    uint64_t* o_full = bars + 9;             // [2]
    uint64_t* o_empty = bars + 11;           // [2]
    uint64_t* p_full = bars + 13;            // [2]
    uint64_t* p_empty = bars + 15;           // [2]
    uint64_t* v_empty = bars + 17;           // [2]  values of a stage are free once P V has read them
    uint64_t* k_full = bars + 19;            // [2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 21);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* half_max = (float*)(smem + SMEM_TILES + 256);         // [2][ROWS]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ratio = heads / kv_heads;
    const int tokens_per_tile = ROWS / ratio;

    if (threadIdx.x == 0) {
        tc::mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(&kv_full[i], 1);      // values
            tc::mbar_init(&k_full[i], 1);       // keys
            tc::mbar_init(&k_empty[i], 1);
            tc::mbar_init(&v_empty[i], 1);
            tc::mbar_init(&p_full[i], SOFTMAX_WARPS);
            tc::mbar_init(&p_empty[i], 1);
            tc::mbar_init(&s_full[i], 1);
            tc::mbar_init(&s_empty[i], SOFTMAX_WARPS);
            tc::mbar_init(&o_full[i], 1);
            tc::mbar_init(&o_empty[i], SOFTMAX_WARPS);
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
    // The value halves start as zeros: a stage's pages that are not fetched (past the tile's last key)
    // then hold zeros or older finite values, never what the memory held before the launch.
    for (int i = threadIdx.x; i < KV_STAGES * OPERAND_BYTES / 16; i += THREADS) {
        const int stage = i / (OPERAND_BYTES / 16), off = i % (OPERAND_BYTES / 16);
        *reinterpret_cast<uint4*>(smem + SMEM_KV + stage * STAGE_BYTES + OPERAND_BYTES + off * 16) = make_uint4(0, 0, 0, 0);
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    // Which tile this block serves (after the wait: the metadata may come from the step's copy).
    const int r = req_list[blockIdx.z], g = blockIdx.y;
    const int n_q = row_count[r];
    const int n_tiles = (n_q + tokens_per_tile - 1) / tokens_per_tile;
    const bool active = (int)blockIdx.x < n_tiles;
    const int tile = active ? n_tiles - 1 - blockIdx.x : 0;          // the tiles with the most keys start first
    const int q0 = row_start[r], hist = history[r];
    const int t0 = tile * tokens_per_tile;
    const int t_count = min(tokens_per_tile, n_q - t0);
    const int M = t_count * ratio;
    const int last_pos = hist + t0 + t_count - 1;
    int kv_begin = 0;
    if (window > 0) kv_begin = (max(0, hist + t0 - window + 1) / KEYS) * KEYS;
    const int kv_end = last_pos + 1;
    const int n_iter = active ? (kv_end - kv_begin + KEYS - 1) / KEYS : 0;

    if (warp == 0) {
        if (n_iter > 0 && tc::elect_one()) {
            // Q: rows [token][head of the group], both 64-column halves, one box.
            tc::mbar_expect_tx(q_full, (uint32_t)OPERAND_BYTES);
            tc::tma_load_5d(smem + SMEM_Q, &q_map, 0, 0, q0 + t0, 0, g, q_full);
            const int* table = block_tables + (size_t)r * table_stride + kv_begin / PAGE;
            const int n_pages = (kv_end - kv_begin + PAGE - 1) / PAGE;
            // The page ids of a stage are read one stage ahead (the copies' memory clobber keeps the compiler from
            // moving loads across them, and a table load is a round trip to L2 the copies must not wait for).
            int ids[PAGES_PER_STAGE], ids_next[PAGES_PER_STAGE];
#pragma unroll
            for (int p = 0; p < PAGES_PER_STAGE; ++p) ids_next[p] = p < n_pages ? table[p] : 0;
            for (int j = 0; j < n_iter; ++j) {
                const int st = j % KV_STAGES;
                const uint32_t ph = ((uint32_t)(j / KV_STAGES) & 1u) ^ 1u;
                const int here = min(PAGES_PER_STAGE, n_pages - j * PAGES_PER_STAGE);
                uint8_t* kbase = smem + SMEM_KV + st * STAGE_BYTES;
#pragma unroll
                for (int p = 0; p < PAGES_PER_STAGE; ++p) {
                    ids[p] = ids_next[p];
                    const int nxt = (j + 1) * PAGES_PER_STAGE + p;
                    ids_next[p] = nxt < n_pages ? table[nxt] : 0;
                }
                // Keys first (their slot is free as soon as Q K^T of the tile two back has run), then values.
                if (!tc::mbar_wait(&k_empty[st], ph, abort_flag, error_word, ERR_TCA_PRODUCER)) break;
                tc::mbar_expect_tx(&k_full[st], (uint32_t)(here * PAGE * D * 2));
#pragma unroll
                for (int p = 0; p < PAGES_PER_STAGE; ++p) {
                    if (p >= here) break;
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                        tc::tma_load_5d(kbase + half * HALF_BYTES + p * PAGE * 128, &cache_map, 0, 0, half, g, ids[p] * 2,
                                        &k_full[st]);
                }
                if (!tc::mbar_wait(&v_empty[st], ph, abort_flag, error_word, ERR_TCA_PRODUCER)) break;
                tc::mbar_expect_tx(&kv_full[st], (uint32_t)(here * PAGE * D * 2));
#pragma unroll
                for (int p = 0; p < PAGES_PER_STAGE; ++p) {
                    if (p >= here) break;
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                        tc::tma_load_5d(kbase + OPERAND_BYTES + half * HALF_BYTES + p * PAGE * 128, &cache_map, 0, 0, half,
                                        g, ids[p] * 2 + 1, &kv_full[st]);
                }
            }
        }
    } else if (warp == 1) {
        if (n_iter > 0 && tc::elect_one()) {
            bool ok = tc::mbar_wait(q_full, 0, abort_flag, error_word, ERR_TCA_MMA);
            const uint32_t q_addr = tc::smem_u32(smem + SMEM_Q), p_addr = tc::smem_u32(smem + SMEM_P);
            auto issue_pv = [&](int i) -> bool {
                const int bi = i & 1, st = i % KV_STAGES;
                if (!tc::mbar_wait(&kv_full[st], (uint32_t)(i / KV_STAGES) & 1u, abort_flag, error_word, ERR_TCA_MMA)) return false;
                if (!tc::mbar_wait(&p_full[bi], (uint32_t)(i / 2) & 1u, abort_flag, error_word, ERR_TCA_MMA)) return false;
                if (!tc::mbar_wait(&o_empty[bi], ((uint32_t)(i / 2) & 1u) ^ 1u, abort_flag, error_word, ERR_TCA_MMA)) return false;
                tc::tc_fence_after();
                const uint32_t v_addr = tc::smem_u32(smem + SMEM_KV + st * STAGE_BYTES + OPERAND_BYTES);
#pragma unroll
                for (int kk = 0; kk < KEYS / 16; ++kk) {
                    const uint64_t da = tc::smem_desc_k_sw128(p_addr + bi * OPERAND_BYTES + (kk >> 2) * HALF_BYTES + (kk & 3) * 32);
                    const uint64_t db = smem_desc_mn_sw128(v_addr + kk * 16 * 128, HALF_BYTES);
                    tc::mma_bf16_ss(tmem_base + 2 * KEYS + bi * D, da, db, IDESC_PV, kk > 0 ? 1u : 0u);
                }
                tc::mma_commit(&o_full[bi]);
                tc::mma_commit(&p_empty[bi]);
                tc::mma_commit(&v_empty[st]);
                return true;
            };
            for (int j = 0; j < n_iter && ok; ++j) {
                const int b = j & 1, st = j % KV_STAGES;
                ok = tc::mbar_wait(&k_full[st], (uint32_t)(j / KV_STAGES) & 1u, abort_flag, error_word, ERR_TCA_MMA) &&
                     tc::mbar_wait(&s_empty[b], ((uint32_t)(j / 2) & 1u) ^ 1u, abort_flag, error_word, ERR_TCA_MMA);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t k_addr = tc::smem_u32(smem + SMEM_KV + st * STAGE_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
                    tc::mma_bf16_ss(tmem_base + b * KEYS, tc::smem_desc_k_sw128(q_addr + off),
                                    tc::smem_desc_k_sw128(k_addr + off), IDESC_QK, kk > 0 ? 1u : 0u);
                }
                tc::mma_commit(&s_full[b]);
                tc::mma_commit(&k_empty[st]);
                if (j >= 1) ok = issue_pv(j - 1);
            }
            if (ok) issue_pv(n_iter - 1);
        }
    } else if (n_iter > 0) {
        // ---- two threads per query row: warp s serves rows 32 (s % 4) .. + 31, columns 64 (s / 4) .. + 63
        const int sw = warp - 2;
        const int quarter = warp & 3, half = sw >> 2;
        const int row = quarter * 32 + lane;
        const bool valid = row < M;
        const int ti = t0 + min(row, M - 1) / ratio;
        const int pos = hist + ti;
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        constexpr int HC = 64;                                   // columns per thread
        float o[HC];
#pragma unroll
        for (int d = 0; d < HC; ++d) o[d] = 0.0f;
        float m_run = -INFINITY, l_run = 0.0f, alpha_pending = 0.0f;
        bool ok = true;

        auto accumulate = [&](int i) -> bool {
            const int bi = i & 1;
            if (!tc::mbar_wait(&o_full[bi], (uint32_t)(i / 2) & 1u, abort_flag, error_word, ERR_TCA_SOFTMAX)) return false;
            tc::tc_fence_after();
#pragma unroll
            for (int c = 0; c < HC; c += 32) {
                uint32_t v[32];
                tc::tmem_ld_32x32(tmem_base + 2 * KEYS + bi * D + half * HC + c + lane_addr, v);
                tc::tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 32; ++k) o[c + k] = fmaf(o[c + k], alpha_pending, __uint_as_float(v[k]));
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&o_empty[bi]);
            return true;
        };

        for (int j = 0; j < n_iter; ++j) {
            const int b = j & 1;
            const int key0 = kv_begin + j * KEYS + half * HC;
            if (ok) ok = tc::mbar_wait(&s_full[b], (uint32_t)(j / 2) & 1u, abort_flag, error_word, ERR_TCA_SOFTMAX);
            tc::tc_fence_after();
            const bool need_mask = key0 + HC - 1 > pos || key0 < lo;
            // ---- this half's raw scores (kept in registers) and their maximum; masked ones become -inf.
            // The scale is positive, so it is applied after the maximum and folded into the exponent's
            // multiply-add: one instruction per score here, three in the pass below.
            float sc[HC];
            float rowmax = -INFINITY;
            if (ok) {
#pragma unroll
                for (int c = 0; c < HC; c += 32) {
                    uint32_t v[32];
                    tc::tmem_ld_32x32(tmem_base + b * KEYS + half * HC + c + lane_addr, v);
                    tc::tmem_wait_ld();
                    if (need_mask) {
#pragma unroll
                        for (int k = 0; k < 32; ++k) {
                            const int key = key0 + c + k;
                            sc[c + k] = (key > pos || key < lo) ? -INFINITY : __uint_as_float(v[k]);
                            rowmax = fmaxf(rowmax, sc[c + k]);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 32; ++k) {
                            sc[c + k] = __uint_as_float(v[k]);
                            rowmax = fmaxf(rowmax, sc[c + k]);
                        }
                    }
                }
            }
            rowmax *= scale_log2;
            // S has been read: the tensor core may write the tile after next into it.
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0 && ok) tc::mbar_arrive(&s_empty[b]);
            // ---- the row's maximum over both halves (every softmax thread comes here, also after a failed wait)
            half_max[half * ROWS + row] = rowmax;
            asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
            rowmax = fmaxf(rowmax, half_max[(half ^ 1) * ROWS + row]);
            asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
            if (!ok) continue;
            const float m_new = fmaxf(m_run, rowmax);
            const float alpha = m_new == -INFINITY ? 1.0f : exp2f(m_run - m_new);
            const float base = m_new == -INFINITY ? 0.0f : m_new;
            m_run = m_new;
            // ---- P = 2^(s - m) as bfloat16 into the operand layout; P V of the tile before must have read P
            ok = tc::mbar_wait(&p_empty[b], ((uint32_t)(j / 2) & 1u) ^ 1u, abort_flag, error_word, ERR_TCA_SOFTMAX);
            if (!ok) continue;
            float rowsum = 0.0f;
            uint8_t* p_row = smem + SMEM_P + b * OPERAND_BYTES + half * HALF_BYTES + row * 128;
#pragma unroll
            for (int c8 = 0; c8 < HC / 8; ++c8) {
                uint32_t packed[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float p0 = fast_exp2(fmaf(sc[c8 * 8 + 2 * k], scale_log2, -base));
                    const float p1 = fast_exp2(fmaf(sc[c8 * 8 + 2 * k + 1], scale_log2, -base));
                    rowsum += p0 + p1;
                    packed[k] = attn::pack_bf16(p0, p1);
                }
                *reinterpret_cast<uint4*>(p_row + ((c8 ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            l_run = l_run * alpha + rowsum;
            tc::fence_proxy_async();          // the tensor core reads P through the async proxy
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&p_full[b]);
            // ---- fold the tile before into the running output while this tile's P V runs
            if (j >= 1) ok = accumulate(j - 1);
            alpha_pending = alpha;
        }
        if (ok) ok = accumulate(n_iter - 1);
        // The row's sum over both halves.
        half_max[half * ROWS + row] = l_run;
        asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
        const float l_total = l_run + half_max[(half ^ 1) * ROWS + row];
        if (ok && valid) {
            const float inv = 1.0f / l_total;
            __nv_bfloat16* dst = out + ((size_t)(q0 + ti) * heads + g * ratio + row % ratio) * D + half * HC;
#pragma unroll
            for (int d = 0; d < HC; d += 8) {
                uint4 val = make_uint4(attn::pack_bf16(o[d] * inv, o[d + 1] * inv), attn::pack_bf16(o[d + 2] * inv, o[d + 3] * inv),
                                       attn::pack_bf16(o[d + 4] * inv, o[d + 5] * inv), attn::pack_bf16(o[d + 6] * inv, o[d + 7] * inv));
                *reinterpret_cast<uint4*>(dst + d) = val;
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

// q [rows, heads, 128] bfloat16 as (64 columns) x (head within the group) x (row) x (half of the head) x (kv head):
// the box {64, ratio, 128 / ratio, 2, 1} is a tile's Q operand, [half][row][head][64 columns] in shared memory.
int make_q_map(CUtensorMap* map, const void* q, uint64_t rows, int heads, int kv_heads) {
    llmx_encode_tiled_fn enc = llmx_encode_tiled();
    if (!enc) return 10003;
    const uint64_t ratio = heads / kv_heads;
    const cuuint64_t dims[5] = {64, ratio, rows, 2, (cuuint64_t)kv_heads};
    const cuuint64_t strides[4] = {D * 2, (cuuint64_t)heads * D * 2, 128, ratio * D * 2};
    const cuuint32_t box[5] = {64, (cuuint32_t)ratio, (cuuint32_t)(ROWS / ratio), 2, 1};
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
// keys; q/out [total_rows, heads, 128] bfloat16.
LLMX_EXPORT int llmx_attn_prefill_tc(const void* cache_map, const void* q, void* out, int total_rows,
                                     const int* req_list, int n_req, const int* row_start, const int* row_count,
                                     const int* history, const int* block_tables, int table_stride, int heads,
                                     int kv_heads, int head_dim, int page_size, int window, float scale, int max_rows,
                                     int* error_word, cudaStream_t stream) {
    if (n_req <= 0 || max_rows <= 0) return 0;
    if (head_dim != D || page_size != PAGE || heads % kv_heads || ROWS % (heads / kv_heads) || n_req > 65535 ||
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
    const int tokens_per_tile = ROWS / (heads / kv_heads);
    dim3 grid((max_rows + tokens_per_tile - 1) / tokens_per_tile, kv_heads, n_req);
    launch_kernel(attn_prefill_tc_kernel, grid, dim3(THREADS), (size_t)SMEM_BYTES, stream, q_map,
                  *(const CUtensorMap*)cache_map, (__nv_bfloat16*)out, req_list, row_start, row_count, history,
                  block_tables, table_stride, heads, kv_heads, window, scale * attn::LOG2E, error_word);
    return launch_status();
}
