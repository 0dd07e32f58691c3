// bfloat16 matrix product on the 5th-generation tensor cores:  C[M, N] (+)= A[M, K] * W[N, K]^T.
//
// Both operands are K-major (each row contiguous), which is how activations [tokens, in] and
// weights [out, in] lie in memory, so no operand is transposed.  The weight takes the 128-row
// side of the instruction and the tokens the narrow side (16..256), so one kernel serves a
// single decoded token and a 2,048-token prompt alike:
//     D[128 weight rows, BN tokens] (+)= Wtile[128, 64] * Atile[BN, 64]^T     per 64-wide k block
// Tiles reach shared memory by TMA (128-byte swizzle, out-of-range rows and columns read as
// zero, so M, N and K need not be multiples of the tile), the accumulator lives in tensor
// memory, one elected thread issues tcgen05.mma, and the epilogue reads the accumulator with
// tcgen05.ld and writes C with one warp store per 32 consecutive outputs of a token.
//
// The kernel is persistent with three roles:  warp 0 loads (TMA producer), warp 1 issues the
// matrix instructions, warps 2-5 are the epilogue.  Two accumulators in tensor memory let the
// epilogue of one piece of work overlap the products of the next.  Work is handed out in one
// of two ways:
//   tiles     a block walks whole output tiles (blockIdx.x, + gridDim.x, ...), optionally with K
//             cut into `splits` ranges that are added with float atomics; used for many tokens.
//   stream-K  all (tile, k block) units are cut into gridDim.x runs (the second half of the blocks a
//             little shorter ones, so that they leave early and the next kernel's blocks come in two
//             halves); a block's run may end
//             one tile and begin the next, and every piece is added to C with float atomics
//             (C is zeroed first when the product is to be stored).  A few tokens make few
//             tiles; this keeps every SM streaming weights whatever N is.
// A third form, DUAL, computes two products that share the token tile -- rows n and n + N/2 of
// the weight (gate and up of a gated feed-forward) -- into two accumulators and writes
// silu(gate) * up as bfloat16, so the [tokens, 2 * intermediate] float32 matrix never exists.
// A fourth form, HEADS, is the q/k/v product of an attention layer with heads of 128: the operands
// change sides (128 tokens on the instruction's M side, 128 or 256 weight rows = one or two whole heads on
// the narrow side), so that a thread of the epilogue holds whole heads of one token.  It norms and rotates
// them there and writes the queries and the cache rows as bfloat16: the float32 [tokens, q + 2 kv] matrix and
// the kernel that read it back never exist (src/model/arch/qwen3.hpp:280-290 for the order of operations).
//
// The reference has no tensor-core path for this product (its kernels: f32.gpu:1034-1084).
#include "tc_common.cuh"
#include "gemm_heads_epilogue.cuh"
#include <math.h>

namespace {

constexpr int BM = 128;      // weight rows per tile (the instruction's M)
constexpr int BK = 64;       // bfloat16 elements per k block: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 4;
// HEADS: with up to this many token tiles (2,048 tokens) neighbouring blocks take the same weight rows and
// different tokens (2,048 tokens: 88 -> 85 us); with more, the same tokens and different weight rows (8,192: 342 us
// against 359).
constexpr int HEADS_TOKEN_FIRST_TILES = 16;
constexpr int THREADS = 64 + EPI_WARPS * 32;

enum : int { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_ATOMIC = 2, MODE_SWIGLU = 3 };
enum : int { ERR_PRODUCER = 101, ERR_MMA_FULL = 102, ERR_MMA_ACC = 103, ERR_EPILOGUE = 104 };

template <int BN, bool DUAL>
struct Cfg {
    static constexpr int A_TILES = DUAL ? 2 : 1;
    static constexpr int A_BYTES = BM * BK * 2;          // one weight tile
    static constexpr int B_BYTES = BN * BK * 2;          // token tile
    static constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
    // Narrow token tiles (few tokens: the product streams weights) take half an SM's shared memory, so two
    // blocks share an SM and one's prologue and epilogue hide behind the other's loads; wide tiles take it all.
    static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1;
    static constexpr int BUDGET = (BN <= 64 ? 100 : 200) * 1024;
    static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
    static constexpr int ACC_COLS = A_TILES * BN;        // columns of one accumulator set
    static constexpr int TMEM_COLS = (2 * ACC_COLS) < 32 ? 32 : (2 * ACC_COLS);
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + 1024 /*norm weights*/;
    static_assert(TMEM_COLS <= 512, "two accumulator sets must fit tensor memory");
};

struct Work {
    int nt, mt, kb0, kb1;
};

// Hands a block its pieces of work, the same sequence in every role.
template <bool STREAMK>
struct Scheduler {
    int n_tiles, m_tiles, k_blocks, splits;
    bool wide_first;            // tiles schedule: the 128-row side's tiles vary fastest instead of the narrow side's
    long long cur, end;
    // `skew` (stream-K, percent): the first half of the blocks take that much more than an even share and the second
    // half what is left, so the second half leaves early (see llmx_gemm_tc).
    __device__ Scheduler(int n_tiles_, int m_tiles_, int k_blocks_, int splits_, bool wide_first_ = false, int skew = 0)
        : n_tiles(n_tiles_), m_tiles(m_tiles_), k_blocks(k_blocks_), splits(splits_), wide_first(wide_first_) {
        if (STREAMK) {
            const long long units = (long long)n_tiles * m_tiles * k_blocks;
            const long long blocks = gridDim.x, half = blocks / 2;
            if (skew > 0 && blocks >= 8) {
                const long long more = (units * (100 + skew) + 100 * blocks - 1) / (100 * blocks);
                const long long rest = units > more * half ? units - more * half : 0;
                const long long less = (rest + (blocks - half) - 1) / (blocks - half);
                const long long b = blockIdx.x;
                cur = b < half ? more * b : more * half + less * (b - half);
                end = cur + (b < half ? more : less);
                if (cur > units) cur = units;
                if (end > units) end = units;
            } else {
                const long long per = (units + blocks - 1) / blocks;
                cur = per * blockIdx.x;
                end = cur + per < units ? cur + per : units;
            }
        } else {
            cur = blockIdx.x;
            end = (long long)n_tiles * m_tiles * splits;
        }
    }
    __device__ bool next(Work& w) {
        if (cur >= end) return false;
        if (STREAMK) {
            const long long tile = cur / k_blocks;
            w.kb0 = (int)(cur % k_blocks);
            const long long left = end - cur;
            w.kb1 = (k_blocks - w.kb0) < left ? k_blocks : (int)(w.kb0 + left);
            w.mt = (int)(tile % m_tiles);
            w.nt = (int)(tile / m_tiles);
            cur += w.kb1 - w.kb0;
        } else {
            // Token tiles vary fastest, so neighbouring blocks share a weight tile.
            long long rest;
            if (wide_first) {
                w.nt = (int)(cur % n_tiles);
                rest = cur / n_tiles;
                w.mt = (int)(rest % m_tiles);
                rest /= m_tiles;
            } else {
                w.mt = (int)(cur % m_tiles);
                rest = cur / m_tiles;
                w.nt = (int)(rest % n_tiles);
                rest /= n_tiles;
            }
            const int sp = (int)rest;
            const int per = (k_blocks + splits - 1) / splits;
            w.kb0 = sp * per;
            w.kb1 = min(k_blocks, w.kb0 + per);
            cur += gridDim.x;
        }
        return true;
    }
};


template <int BN, bool STREAMK, bool DUAL, bool HEADS>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
               void* __restrict__ C_, int M, int N, int K, int mode, int splits, int skew, int* error_word,
               const HeadsEpilogue hp) {
    // HEADS: `map_w` is the tokens' map and N their number, `map_a` the weight's and M its rows.
    using cfg = Cfg<BN, DUAL>;
    pdl_trigger();      // the next kernel's blocks may start arriving; they wait for this one to finish
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* full_bar = (uint64_t*)(smem + cfg::STAGES * cfg::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + cfg::STAGES;
    uint64_t* acc_full = empty_bar + cfg::STAGES;     // [2]
    uint64_t* acc_empty = acc_full + 2;               // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* norm_w = (float*)(smem + cfg::STAGES * cfg::STAGE_BYTES + 256);      // HEADS: q weights, then k weights

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // DUAL: N counts the outputs (half the weight's rows); rows n and n + N belong together.
    const int n_tiles = (N + BM - 1) / BM, m_tiles = (M + BN - 1) / BN;
    const int k_blocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < cfg::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], EPI_WARPS);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::tma_prefetch_desc(&map_w);
        tc::tma_prefetch_desc(&map_a);
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, cfg::TMEM_COLS);
        tc::tmem_relinquish();
    }
    if (HEADS && threadIdx.x >= 64) {
        // Norm weights are written by no kernel: they may be read before pdl_wait().
        const int i = threadIdx.x - 64;
        norm_w[i] = hp.q_weight ? hp.q_weight[i] : 1.0f;
        norm_w[128 + i] = hp.k_weight ? hp.k_weight[i] : 1.0f;
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Barriers, tensor memory and descriptors are ready.  The weights are written by no kernel, so the
    // producer fetches its first stages of them at once; whatever another kernel writes (the activations,
    // the output) is touched only after pdl_wait(), when the kernel before has finished.
    if (warp == 0) {
        if (tc::elect_one()) {
            Scheduler<STREAMK> sched(n_tiles, m_tiles, k_blocks, splits, HEADS && n_tiles <= HEADS_TOKEN_FIRST_TILES, skew);
            Work w;
            uint32_t stage = 0, phase = 0;
            bool ok = true, waited = false;
            // The weight is the 128-row operand (A_TILES tiles at the stage's start) or, with HEADS, the BN-row one
            // behind it; the activations are the other.  Units (tile, k block) whose weights are in flight but
            // whose activations are not yet asked for:
            int early_kb[cfg::STAGES], early_row[cfg::STAGES], early = 0;
            constexpr int ACT_OFFSET = HEADS ? 0 : cfg::A_TILES * cfg::A_BYTES;
            const CUtensorMap* map_act = HEADS ? &map_w : &map_a;
            while (ok && sched.next(w)) {
                const int act_row = HEADS ? w.nt * BM : w.mt * BN;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!waited && early == cfg::STAGES) {
                        pdl_wait();
                        waited = true;
#pragma unroll
                        for (int e = 0; e < cfg::STAGES; ++e)
                            tc::tma_load_2d(tiles + e * cfg::STAGE_BYTES + ACT_OFFSET, map_act, early_kb[e] * BK,
                                            early_row[e], &full_bar[e]);
                    }
                    ok = tc::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, error_word, ERR_PRODUCER);
                    if (!ok) break;
                    uint8_t* a_dst = tiles + stage * cfg::STAGE_BYTES;
                    uint8_t* b_dst = a_dst + cfg::A_TILES * cfg::A_BYTES;
                    tc::mbar_expect_tx(&full_bar[stage], cfg::STAGE_BYTES);
                    if (HEADS) {
                        tc::tma_load_2d(b_dst, &map_a, kb * BK, w.mt * BN, &full_bar[stage]);
                    } else {
                        tc::tma_load_2d(a_dst, &map_w, kb * BK, w.nt * BM, &full_bar[stage]);
                        if (DUAL)
                            tc::tma_load_2d(a_dst + cfg::A_BYTES, &map_w, kb * BK, N + w.nt * BM, &full_bar[stage]);
                    }
                    if (waited) {
                        tc::tma_load_2d(a_dst + ACT_OFFSET, map_act, kb * BK, act_row, &full_bar[stage]);
                    } else {
                        early_kb[early] = kb;
                        early_row[early] = act_row;
                        ++early;
                    }
                    if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!waited) {
                // Fewer units than stages: their activations are still to be asked for.
                pdl_wait();
                for (int e = 0; e < early; ++e)
                    tc::tma_load_2d(tiles + e * cfg::STAGE_BYTES + ACT_OFFSET, map_act, early_kb[e] * BK, early_row[e],
                                    &full_bar[e]);
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc_bf16(BM, BN);
            Scheduler<STREAMK> sched(n_tiles, m_tiles, k_blocks, splits, HEADS && n_tiles <= HEADS_TOKEN_FIRST_TILES, skew);
            Work w;
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            while (ok && sched.next(w)) {
                ok = tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, error_word, ERR_MMA_ACC);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * cfg::ACC_COLS;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = tc::mbar_wait(&full_bar[stage], phase, abort_flag, error_word, ERR_MMA_FULL);
                    if (!ok) break;
                    tc::tc_fence_after();
                    const uint32_t a_addr = tc::smem_u32(tiles + stage * cfg::STAGE_BYTES);
                    const uint64_t desc_a = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t desc_b = tc::smem_desc_k_sw128(a_addr + cfg::A_TILES * cfg::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements = 32 bytes further along the swizzled row: +2 in the descriptor's 16-byte units.
                        const uint32_t accumulate = (kb > w.kb0 || k > 0) ? 1u : 0u;
                        tc::mma_bf16_ss(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, accumulate);
                        if (DUAL) {
                            const uint64_t desc_a2 = tc::smem_desc_k_sw128(a_addr + cfg::A_BYTES);
                            tc::mma_bf16_ss(tmem_d + BN, desc_a2 + 2 * k, desc_b + 2 * k, idesc, accumulate);
                        }
                    }
                    tc::mma_commit(&empty_bar[stage]);   // the stage is free once these instructions have read it
                    if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc::mma_commit(&acc_full[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // Epilogue: warp w may read the tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        Scheduler<STREAMK> sched(n_tiles, m_tiles, k_blocks, splits, HEADS && n_tiles <= HEADS_TOKEN_FIRST_TILES, skew);
        Work w;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        // Adding to the output is always by float atomics, also when a tile is the only one to add to its outputs
        // (then the sum is the same as a load, an add and a store would give): nothing comes back from memory, where
        // the loads' round trips made the last tile's epilogue the kernel's tail ([4096, 4096] at 2,048 tokens:
        // 63 -> 55 us).
        const bool atomic = STREAMK || mode == MODE_ATOMIC || mode == MODE_ACCUMULATE;
        pdl_wait();     // the output may be read or cleared by the kernel before
        while (ok && sched.next(w)) {
            ok = tc::mbar_wait(&acc_full[acc], acc_phase, abort_flag, error_word, ERR_EPILOGUE);
            if (!ok) break;
            tc::tc_fence_after();
            const int n = w.nt * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * cfg::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if constexpr (HEADS) {
                if constexpr (BN % 128 == 0) heads_epilogue<BN>(hp, norm_w, taddr, n, N, w.mt * BN, M);
            } else if (w.kb1 > w.kb0) {
                constexpr int CH = BN < 32 ? 16 : 32;
#pragma unroll 1
                for (int c = 0; c < BN; c += CH) {
                    uint32_t r[CH];
                    if constexpr (CH == 32) tc::tmem_ld_32x32(taddr + c, r);
                    else tc::tmem_ld_32x16(taddr + c, r);
                    if constexpr (DUAL) {
                        uint32_t u[CH];
                        if constexpr (CH == 32) tc::tmem_ld_32x32(taddr + BN + c, u);
                        else tc::tmem_ld_32x16(taddr + BN + c, u);
                        tc::tmem_wait_ld();
                        if (n < N) {
                            // silu(g) * u in float32 with the fast exponential and reciprocal (a few units in the
                            // last place, far below the bfloat16 rounding that follows): with short inner widths
                            // this epilogue, not the products, sets the kernel's time.
                            __nv_bfloat16* C = (__nv_bfloat16*)C_ + (size_t)(w.mt * BN + c) * N + n;
                            const int m_left = M - (w.mt * BN + c);
#pragma unroll
                            for (int j = 0; j < CH; ++j) {
                                const float g = __uint_as_float(r[j]), up = __uint_as_float(u[j]);
                                const float act = __fdividef(g, 1.0f + __expf(-g)) * up;
                                if (j < m_left) C[(size_t)j * N] = __float2bfloat16_rn(act);
                            }
                        }
                    } else {
                        tc::tmem_wait_ld();
                        if (n < N) {
                            float* C = (float*)C_ + (size_t)(w.mt * BN + c) * N + n;
                            const int m_left = M - (w.mt * BN + c);        // rows of this chunk inside the matrix
                            if (atomic) {
#pragma unroll
                                for (int j = 0; j < CH; ++j)
                                    if (j < m_left) atomicAdd(C + (size_t)j * N, __uint_as_float(r[j]));
                            } else {        // MODE_STORE
#pragma unroll
                                for (int j = 0; j < CH; ++j)
                                    if (j < m_left) C[(size_t)j * N] = __uint_as_float(r[j]);
                            }
                        }
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&acc_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, cfg::TMEM_COLS);
    }
}

int g_sm_count = 0;

template <int BN, bool STREAMK, bool DUAL>
int launch(const CUtensorMap& map_w, const void* A, void* C, int M, int N, int K, int mode, int splits,
           int* error_word, cudaStream_t stream) {
    using cfg = Cfg<BN, DUAL>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN, STREAMK, DUAL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 cfg::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    CUtensorMap map_a;
    if (int e = llmx_make_map_bf16_2d(&map_a, A, (uint64_t)M, (uint64_t)K, BN, BK)) return e;
    const int n_tiles = (N + BM - 1) / BM, m_tiles = (M + BN - 1) / BN, k_blocks = (K + BK - 1) / BK;
    long long grid;
    if (STREAMK) {
        // Every block at least four k blocks, so that a tiny product does not pay 148 prologues.
        const long long units = (long long)n_tiles * m_tiles * k_blocks;
        grid = (units + 3) / 4;
    } else {
        grid = (long long)n_tiles * m_tiles * splits;
    }
    if (grid > (long long)g_sm_count * cfg::CTAS_PER_SM) grid = (long long)g_sm_count * cfg::CTAS_PER_SM;
    if (grid < 1) grid = 1;
    // Stream-K: uneven shares.  With even shares all blocks of a product leave at one moment, the next kernel's blocks
    // all arrive, set up and ask for their first weights at one moment, and for those microseconds nothing streams.
    // With the second half of the blocks (the second block of every SM) given less, that half leaves early: the next
    // product's first blocks take its place, set up and fill their stages while the first half still streams, and
    // stream themselves while the rest arrives.  The shares differ by what the weights take to stream in STAGGER_NS
    // (measured at Qwen3-8B sizes, decode at batch 8: 4.457 ms a step even, 4.423 with 3 us, 4.383 with 4 to 5 us,
    // 4.463 with 7 us; batch 1: 3.309 -> 3.252).  Not for products that stream for less than that themselves (Qwen3-0.6B
    // sizes, batch 8: 1.368 ms a step even, 1.418 with uneven shares).
    int skew = 0;
    if (STREAMK && grid >= 8) {
        constexpr double STAGGER_NS = 4500.0, BYTES_PER_NS = 6500.0;
        const double stream_ns = (double)N * K * 2 / BYTES_PER_NS;
        if (stream_ns >= STAGGER_NS) skew = (int)(100.0 * STAGGER_NS / (2 * stream_ns) + 0.5);
    }
    launch_kernel(gemm_tc_kernel<BN, STREAMK, DUAL, false>, dim3((unsigned)grid), dim3(THREADS), cfg::SMEM_BYTES, stream, 
        map_w, map_a, C, M, N, K, mode, splits, skew, error_word, HeadsEpilogue{});
    return launch_status();
}

// HEADS: the weight's map has boxes of BN rows; the tokens take the 128-row side.
template <int BN>
int launch_heads(const CUtensorMap& map_weight, const void* A, int tokens, int features, int K,
                 const HeadsEpilogue& hp, int* error_word, cudaStream_t stream) {
    using cfg = Cfg<BN, false>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 cfg::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    CUtensorMap map_tokens;
    if (int e = llmx_make_map_bf16_2d(&map_tokens, A, (uint64_t)tokens, (uint64_t)K, BM, BK)) return e;
    long long grid = (long long)((tokens + BM - 1) / BM) * ((features + BN - 1) / BN);
    if (grid > g_sm_count) grid = g_sm_count;
    launch_kernel(gemm_tc_kernel<BN, false, false, true>, dim3((unsigned)grid), dim3(THREADS), cfg::SMEM_BYTES, stream,
        map_tokens, map_weight, (void*)nullptr, features, tokens, K, (int)MODE_STORE, 1, 0, error_word, hp);
    return launch_status();
}

void ensure_sm_count() {
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
}

}  // namespace

// The weight's tensor map (128 rows x 64 columns per box) can be made once and kept: 128 bytes at `out`.
LLMX_EXPORT int llmx_gemm_tc_weight_map(void* out, const void* W, int N, int K) {
    if (K % 8 || ((uintptr_t)W & 15)) return LLMX_ERR_UNSUPPORTED;
    return llmx_make_map_bf16_2d((CUtensorMap*)out, W, (uint64_t)N, (uint64_t)K, BM, BK);
}

// A weight's map with boxes of `box_rows` (128 or 256) rows, for the side of the product that `box_rows` names.
LLMX_EXPORT int llmx_gemm_tc_weight_map_box(void* out, const void* W, int N, int K, int box_rows) {
    if (K % 8 || ((uintptr_t)W & 15) || (box_rows != 128 && box_rows != 256)) return LLMX_ERR_UNSUPPORTED;
    return llmx_make_map_bf16_2d((CUtensorMap*)out, W, (uint64_t)N, (uint64_t)K, (uint32_t)box_rows, BK);
}

// The q/k/v product of a layer whose heads are 128 wide, finished in the epilogue: A [tokens, K] bfloat16; the
// weight [(heads + 2 kv_heads) * 128, K] (query rows, key rows, value rows) by a map of `head_tile`-row boxes
// (128 or 256); queries and keys normed (weights may be null) and rotated (tables [positions, 64], may be
// null), queries to q_out [tokens, heads * 128], keys and values to the cache [pages, 2, kv_heads, page_size,
// 128] at slots[token] (negative: not stored), all bfloat16.
LLMX_EXPORT int llmx_gemm_tc_heads(const void* weight_map, const void* A, int tokens, int K, int head_tile,
                                   const float* q_weight, const float* k_weight, float eps, const float* cos_table,
                                   const float* sin_table, const int* positions, const int* slots, void* q_out,
                                   void* cache, int heads, int kv_heads, int page_size, int* error_word,
                                   cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)A & 15) || ((uintptr_t)q_out & 15) || ((uintptr_t)cache & 15))
        return LLMX_ERR_UNSUPPORTED;
    if (heads <= 0 || kv_heads <= 0 || page_size <= 0 || !positions || !slots || !q_out || !cache ||
        (cos_table == nullptr) != (sin_table == nullptr))
        return LLMX_ERR_BAD_ARGUMENT;
    if (((uintptr_t)cos_table & 15) || ((uintptr_t)sin_table & 15)) return LLMX_ERR_UNSUPPORTED;
    ensure_sm_count();
    HeadsEpilogue hp;
    hp.q_weight = q_weight; hp.k_weight = k_weight; hp.cos_table = cos_table; hp.sin_table = sin_table;
    hp.positions = positions; hp.slots = slots;
    hp.q_out = (__nv_bfloat16*)q_out; hp.cache = (__nv_bfloat16*)cache;
    hp.eps = eps; hp.heads = heads; hp.kv_heads = kv_heads; hp.page_size = page_size;
    const int features = (heads + 2 * kv_heads) * 128;
    const CUtensorMap& map_w = *(const CUtensorMap*)weight_map;
    switch (head_tile) {
        case 128: return launch_heads<128>(map_w, A, tokens, features, K, hp, error_word, stream);
        case 256: return launch_heads<256>(map_w, A, tokens, features, K, hp, error_word, stream);
        default: return LLMX_ERR_BAD_ARGUMENT;
    }
}

// mode 0: C = A W^T;  mode 1: C += A W^T (float32 C [M, N]).
// schedule 0 (tiles): `splits` > 1 (only with mode 1) cuts K and adds with atomics.
// schedule 1 (stream-K): every piece is added with atomics; with mode 0 the caller zeroes C first.
// `token_tile` is 16, 32, 64, 128 or 256 (0: chosen from M).  `error_word`: device int, zero before first use.
LLMX_EXPORT int llmx_gemm_tc(const void* weight_map, const void* A, float* C, int M, int N, int K, int mode,
                             int splits, int token_tile, int schedule, int* error_word, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)A & 15) || ((uintptr_t)C & 3)) return LLMX_ERR_UNSUPPORTED;
    if (mode != MODE_STORE && mode != MODE_ACCUMULATE) return LLMX_ERR_BAD_ARGUMENT;
    if (splits < 1 || (splits > 1 && mode != MODE_ACCUMULATE)) return LLMX_ERR_BAD_ARGUMENT;
    ensure_sm_count();
    const int k_blocks = (K + BK - 1) / BK;
    if (splits > k_blocks) splits = k_blocks;
    int bn = token_tile;
    if (bn == 0) bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    const CUtensorMap& map_w = *(const CUtensorMap*)weight_map;
    if (schedule == 1) {
        switch (bn) {
            case 16: return launch<16, true, false>(map_w, A, C, M, N, K, mode, 1, error_word, stream);
            case 32: return launch<32, true, false>(map_w, A, C, M, N, K, mode, 1, error_word, stream);
            case 64: return launch<64, true, false>(map_w, A, C, M, N, K, mode, 1, error_word, stream);
            case 128: return launch<128, true, false>(map_w, A, C, M, N, K, mode, 1, error_word, stream);
            case 256: return launch<256, true, false>(map_w, A, C, M, N, K, mode, 1, error_word, stream);
            default: return LLMX_ERR_BAD_ARGUMENT;
        }
    }
    switch (bn) {
        case 16: return launch<16, false, false>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 32: return launch<32, false, false>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 64: return launch<64, false, false>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 128: return launch<128, false, false>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 256: return launch<256, false, false>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        default: return LLMX_ERR_BAD_ARGUMENT;
    }
}

// out[m, n] = silu(A W[n]^T) * (A W[n + N]^T) as bfloat16 [M, N]; the weight has 2 N rows (gate rows, then up rows).
LLMX_EXPORT int llmx_gemm_tc_swiglu(const void* weight_map, const void* A, void* out, int M, int N, int K,
                                    int token_tile, int* error_word, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)A & 15) || ((uintptr_t)out & 1)) return LLMX_ERR_UNSUPPORTED;
    ensure_sm_count();
    int bn = token_tile;
    if (bn == 0) bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    const CUtensorMap& map_w = *(const CUtensorMap*)weight_map;
    switch (bn) {
        case 16: return launch<16, false, true>(map_w, A, out, M, N, K, MODE_SWIGLU, 1, error_word, stream);
        case 32: return launch<32, false, true>(map_w, A, out, M, N, K, MODE_SWIGLU, 1, error_word, stream);
        case 64: return launch<64, false, true>(map_w, A, out, M, N, K, MODE_SWIGLU, 1, error_word, stream);
        case 128: return launch<128, false, true>(map_w, A, out, M, N, K, MODE_SWIGLU, 1, error_word, stream);
        default: return LLMX_ERR_BAD_ARGUMENT;
    }
}
