// bfloat16 matrix product on pairs of SMs (tcgen05 `cta_group::2`):  C[M, N] (+)= A[M, K] * W[N, K]^T  for many tokens.
//
// Two thread blocks of a cluster work on one output tile of 256 weight rows x BN tokens.  Each block holds its own 128
// weight rows (its half of the instruction's M = 256) and only HALF of the token tile (BN / 2 rows): the instruction
// reads the token operand from both blocks' shared memory, so a block takes in 16 KB + 16 KB a k block where the
// one-block kernel (gemm_tc.cu) takes 16 KB + 32 KB for the same multiply-adds.  One thread of the pair's first block
// issues tcgen05.mma.cta_group::2 for both; each block's accumulator (its 128 weight rows x BN tokens) lies in its own
// tensor memory and is written out by its own epilogue warps.
//
//   warp 0 (both blocks)   TMA producer: the block's weight rows and its half of the tokens, per k block, into the
//                          block's own shared memory; the bytes are counted on the FIRST block's barrier (loads
//                          without multicast: `cp.async.bulk.tensor...cta_group::2` only names whose barrier counts)
//   warp 1 (first block)   waits for a stage of both blocks, issues the products, and frees the stage in both blocks
//                          with one commit (`tcgen05.commit...multicast::cluster`, an arrival on each block's barrier)
//   warps 2-5 (both)       epilogue: tensor memory -> float32 output (stored, or added with float atomics), then an
//                          arrival on the first block's accumulator-empty barrier
//
// Work: the pair walks tiles pair, pair + pairs, ... (token tiles vary fastest), optionally with K cut into `splits`
// ranges that are added with atomics, or (`splits` 0) with only the last, partial round's tiles cut.  Every wait
// is bounded (tc_common.cuh); the pair meets at a cluster barrier
// after its barriers are initialised (before any block signals the other) and before either block exits (a block's
// shared memory and barriers are read and signalled by its partner until then).
//
// Three forms share the kernel.  PLAIN: float32 output, stored or added.  DUAL: two products that share the token
// tile -- weight rows n and n + N (gate and up of a gated feed-forward), two tiles of 128 rows a block and two
// accumulators -- written as silu(gate) * up in bfloat16.  HEADS: the q/k/v product of heads of 128; the operands
// change sides (the pair's 256 rows are tokens, 128 a block; the narrow side is 256 weight rows = two heads, of which
// each block loads one), so a thread of the epilogue holds two whole heads of one token, norms and rotates them and
// writes queries and cache rows as bfloat16 (gemm_heads_epilogue.cuh).
//
// The reference has no tensor-core path for this product (its kernels: f32.gpu:1034-1084).
#include "tc_common.cuh"
#include "gemm_heads_epilogue.cuh"

namespace {

constexpr int BM = 128;      // weight rows per block (half of the pair's 256)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 4;
constexpr int THREADS = 64 + EPI_WARPS * 32;
enum : int { MODE_STORE = 0, MODE_ACCUMULATE = 1 };
enum : int { ERR_PAIR_PRODUCER = 111, ERR_PAIR_MMA_FULL = 112, ERR_PAIR_MMA_ACC = 113, ERR_PAIR_EPILOGUE = 114 };

enum : int { PLAIN = 0, DUAL = 1, HEADS = 2 };

// The instruction's 256-row side is the "wide" operand (128 rows a block; DUAL: two such tiles), its BN-row side the
// "narrow" one (BN / 2 rows a block).
template <int BN, int FORM>
struct PairCfg {
    static constexpr int A_TILES = FORM == DUAL ? 2 : 1;
    static constexpr int A_BYTES = BM * BK * 2;                 // one tile of the block's wide rows
    static constexpr int B_BYTES = (BN / 2) * BK * 2;           // the block's half of the narrow tile
    static constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    static constexpr int ACC_COLS = A_TILES * BN;
    static constexpr int TMEM_COLS = 2 * ACC_COLS;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + 1024 /*norm weights*/;
    static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "two accumulator sets in tensor memory");
    static_assert(FORM != HEADS || BN == 256, "a block loads one whole head of the narrow side");
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of block `rank`'s copy of a shared-memory location of this block.
__device__ __forceinline__ uint32_t peer_addr(const void* local, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(tc::smem_u32(local)), "r"(rank));
    return a;
}
__device__ __forceinline__ void arrive_at(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
// A tile load into this block's shared memory whose bytes are counted on a barrier given by its cluster address.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(tc::smem_u32(smem_dst)), "l"(map), "r"(cluster_bar_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(smem_result)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// D[tensor memory of both blocks] (+)= A[128 rows in each block] * B[BN / 2 rows in each block]^T, one thread of the pair.
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this offset in each block of `mask`, once the pair's earlier products have finished.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(tc::smem_u32(bar)), "h"(mask)
                 : "memory");
}

struct Work {
    int wt, mt, kb0, kb1;
};

// Tiles in the order (k range, group of token tiles, weight tile, token tile of the group): neighbouring pairs share
// weight rows, and a group's token rows (`group` tiles of BN rows x K) stay in the L2 cache while every weight tile
// passes over them -- with all token tiles in one group, 4,096 tokens x 12,288 columns are 100 MB that each wave of
// pairs streams again (measured: 540 us against 300).
struct PairScheduler {
    int w_tiles, m_tiles, k_blocks, splits, group, tail;
    long long cur, end, step, whole;
    // `tail` > 0 (with `splits` 1): whole tiles for as many full rounds of the pairs as there are, then the remaining
    // tiles with K cut into `tail` ranges, range by range -- the pieces that run at one time are equally long and
    // neighbours read the same k blocks, so what they share still meets in the L2 cache (runs of arbitrary k blocks
    // a pair were tried: they lose that and were slower than the half-empty last round they avoid).
    __device__ PairScheduler(int w_tiles_, int m_tiles_, int k_blocks_, int splits_, int group_, int tail_)
        : w_tiles(w_tiles_), m_tiles(m_tiles_), k_blocks(k_blocks_), splits(splits_), group(group_), tail(tail_) {
        cur = blockIdx.x >> 1;
        step = gridDim.x >> 1;
        const long long tiles = (long long)w_tiles * m_tiles;
        whole = tail > 0 ? tiles / step * step : tiles * splits;
        end = tail > 0 ? whole + (tiles - whole) * tail : whole;
    }
    __device__ void tile_at(long long rest, Work& w) const {
        const long long per_group = (long long)w_tiles * group;
        const int g = (int)(rest / per_group);                     // the last group may hold fewer token tiles
        const int in_group = min(group, m_tiles - g * group);
        rest -= (long long)g * per_group;
        w.wt = (int)(rest / in_group);
        w.mt = g * group + (int)(rest % in_group);
    }
    __device__ bool next(Work& w) {
        if (cur >= end) return false;
        const long long per_split = (long long)w_tiles * m_tiles;
        int sp, ranges;
        if (tail > 0 && cur < whole) {
            sp = 0, ranges = 1;
            tile_at(cur, w);
        } else if (tail > 0) {
            const long long left = per_split - whole, at = cur - whole;
            sp = (int)(at / left), ranges = tail;
            tile_at(whole + at % left, w);
        } else {
            sp = (int)(cur / per_split), ranges = splits;
            tile_at(cur % per_split, w);
        }
        const int per = (k_blocks + ranges - 1) / ranges;
        w.kb0 = sp * per;
        w.kb1 = min(k_blocks, w.kb0 + per);
        cur += step;
        return true;
    }
};

// `map_wide` / `map_narrow`: the operands' maps (boxes of 128 and BN / 2 rows); `wide_rows` / `narrow_rows`: their
// extents.  PLAIN: wide = weight [N, K], narrow = tokens [M, K], C float32 [M, N].  DUAL: the weight has 2 N rows,
// C bfloat16 [M, N].  HEADS: wide = tokens, narrow = weight; the outputs are `hp`'s.
template <int BN, int FORM>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_wide, const __grid_constant__ CUtensorMap map_narrow,
                    void* __restrict__ C_, int wide_rows, int narrow_rows, int K, int mode, int splits, int group,
                    int tail, int* error_word, const HeadsEpilogue hp) {
    using cfg = PairCfg<BN, FORM>;
    pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* full_bar = (uint64_t*)(smem + cfg::STAGES * cfg::STAGE_BYTES);      // used in the first block
    uint64_t* empty_bar = full_bar + cfg::STAGES;                                 // one in each block
    uint64_t* acc_full = empty_bar + cfg::STAGES;                                 // [2], one in each block
    uint64_t* acc_empty = acc_full + 2;                                           // [2], used in the first block
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* norm_w = (float*)(smem + cfg::STAGES * cfg::STAGE_BYTES + 256);        // HEADS: q weights, then k weights

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int N = wide_rows, M = narrow_rows;       // as PLAIN and DUAL name them
    const int w_tiles = (wide_rows + 2 * BM - 1) / (2 * BM), m_tiles = (narrow_rows + BN - 1) / BN, k_blocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < cfg::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 2 * EPI_WARPS);        // the epilogue warps of both blocks
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::tma_prefetch_desc(&map_wide);
        tc::tma_prefetch_desc(&map_narrow);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, cfg::TMEM_COLS);
        tmem_relinquish_pair();
    }
    if (FORM == HEADS && threadIdx.x >= 64) {
        const int i = threadIdx.x - 64;             // norm weights are written by no kernel
        norm_w[i] = hp.q_weight ? hp.q_weight[i] : 1.0f;
        norm_w[128 + i] = hp.k_weight ? hp.k_weight[i] : 1.0f;
    }
    tc::tc_fence_before();
    __syncthreads();
    cluster_sync();           // both blocks' barriers exist before either signals the other
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();               // the activations and the output belong to the kernels before

    if (warp == 0) {
        if (tc::elect_one()) {
            PairScheduler sched(w_tiles, m_tiles, k_blocks, splits, group, tail);
            Work w;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            while (ok && sched.next(w)) {
                const int wide_row = (w.wt * 2 + (int)rank) * BM;
                const int narrow_row = w.mt * BN + (int)rank * (BN / 2);
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = tc::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, error_word, ERR_PAIR_PRODUCER);
                    if (!ok) break;
                    // The first block's barrier counts both blocks' bytes for the stage.
                    if (leader) tc::mbar_expect_tx(&full_bar[stage], 2 * cfg::STAGE_BYTES);
                    const uint32_t bar = peer_addr(&full_bar[stage], 0);
                    uint8_t* a_dst = tiles + stage * cfg::STAGE_BYTES;
                    tma_load_2d_pair(a_dst, &map_wide, kb * BK, wide_row, bar);
                    if (FORM == DUAL) tma_load_2d_pair(a_dst + cfg::A_BYTES, &map_wide, kb * BK, N + wide_row, bar);
                    tma_load_2d_pair(a_dst + cfg::A_TILES * cfg::A_BYTES, &map_narrow, kb * BK, narrow_row, bar);
                    if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (leader && tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc_bf16(2 * BM, BN);
            PairScheduler sched(w_tiles, m_tiles, k_blocks, splits, group, tail);
            Work w;
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            while (ok && sched.next(w)) {
                ok = tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, error_word, ERR_PAIR_MMA_ACC);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * cfg::ACC_COLS;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = tc::mbar_wait(&full_bar[stage], phase, abort_flag, error_word, ERR_PAIR_MMA_FULL);
                    if (!ok) break;
                    tc::tc_fence_after();
                    const uint32_t a_addr = tc::smem_u32(tiles + stage * cfg::STAGE_BYTES);
                    const uint64_t desc_a = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t desc_b = tc::smem_desc_k_sw128(a_addr + cfg::A_TILES * cfg::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint32_t accumulate = (kb > w.kb0 || k > 0) ? 1u : 0u;
                        mma_bf16_pair(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, accumulate);
                        if (FORM == DUAL) {
                            const uint64_t desc_a2 = tc::smem_desc_k_sw128(a_addr + cfg::A_BYTES);
                            mma_bf16_pair(tmem_d + BN, desc_a2 + 2 * k, desc_b + 2 * k, idesc, accumulate);
                        }
                    }
                    mma_commit_pair(&empty_bar[stage], 3);      // the stage is free in both blocks
                    if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                mma_commit_pair(&acc_full[acc], 3);             // both blocks' accumulators are complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        const int quarter = warp & 3;
        PairScheduler sched(w_tiles, m_tiles, k_blocks, splits, group, tail);
        Work w;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        const bool atomic = mode == MODE_ACCUMULATE || splits > 1;
        while (ok && sched.next(w)) {
            ok = tc::mbar_wait(&acc_full[acc], acc_phase, abort_flag, error_word, ERR_PAIR_EPILOGUE);
            if (!ok) break;
            tc::tc_fence_after();
            const int n = (w.wt * 2 + (int)rank) * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * cfg::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if constexpr (FORM == HEADS) {
                // n: this thread's token; the tile's two heads start at feature w.mt * BN
                heads_epilogue<BN>(hp, norm_w, taddr, n, wide_rows, w.mt * BN, narrow_rows);
            } else if (w.kb1 > w.kb0) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(taddr + c, r);
                    if constexpr (FORM == DUAL) {
                        uint32_t u[32];
                        tc::tmem_ld_32x32(taddr + BN + c, u);
                        tc::tmem_wait_ld();
                        if (n < N) {
                            // silu(g) * u in float32 with the fast exponential and reciprocal, as the one-block product
                            __nv_bfloat16* out = (__nv_bfloat16*)C_ + (size_t)(w.mt * BN + c) * N + n;
                            const int m_left = M - (w.mt * BN + c);
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const float g = __uint_as_float(r[j]), up = __uint_as_float(u[j]);
                                const float act = __fdividef(g, 1.0f + __expf(-g)) * up;
                                if (j < m_left) out[(size_t)j * N] = __float2bfloat16_rn(act);
                            }
                        }
                        continue;
                    }
                    tc::tmem_wait_ld();
                    if (n < N) {
                        float* out = (float*)C_ + (size_t)(w.mt * BN + c) * N + n;
                        const int m_left = M - (w.mt * BN + c);
                        if (atomic) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < m_left) atomicAdd(out + (size_t)j * N, __uint_as_float(r[j]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < m_left) out[(size_t)j * N] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_at(peer_addr(&acc_empty[acc], 0));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    cluster_sync();           // the partner no longer reads this block's shared memory or signals its barriers
    if (warp == 1) {
        tc::tc_fence_after();
        tmem_dealloc_pair(tmem_base, cfg::TMEM_COLS);
    }
}

int g_sm_count = 0;

void ensure_sm_count() {
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sm_count <= 0) g_sm_count = 148;
    }
}

// `wide` / `narrow`: the operands' maps with boxes of 128 and BN / 2 rows; their extents in rows.
template <int BN, int FORM>
int launch_pair(const CUtensorMap& wide, const CUtensorMap& narrow, void* C, int wide_rows, int narrow_rows, int K, int mode,
                int splits, const HeadsEpilogue& hp, int* error_word, cudaStream_t stream) {
    using cfg = PairCfg<BN, FORM>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, FORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int w_tiles = (wide_rows + 2 * BM - 1) / (2 * BM), m_tiles = (narrow_rows + BN - 1) / BN;
    // Narrow tiles a group: what 24 MB hold of the narrow operand's rows of one k range (at least one, at most all).
    const long long tile_bytes = (long long)BN * ((K + (splits ? splits : 1) - 1) / (splits ? splits : 1)) * 2;
    int group = (int)((24ll << 20) / (tile_bytes > 0 ? tile_bytes : 1));
    group = group < 1 ? 1 : group > m_tiles ? m_tiles : group;
    const long long tiles = (long long)w_tiles * m_tiles;
    long long pairs = tiles * (splits ? splits : 8);
    if (pairs > g_sm_count / 2) pairs = g_sm_count / 2;
    if (pairs < 1) pairs = 1;
    // `splits` 0: whole tiles while they fill every pair, the rest in k ranges -- as many as make the rest's rounds
    // shortest.  A piece's write-out runs beside the next piece's products and takes as long as 26 k blocks (the L2
    // cache adds about 500 G floats a second for all pairs together), so shorter pieces gain nothing.
    int tail = 0;
    if (splits == 0) {
        const long long left = tiles % pairs;
        const int k_blocks = (K + BK - 1) / BK;
        long long best = -1;
        tail = 1;
        for (int r = 1; left > 0 && r <= 8 && r <= k_blocks; ++r) {
            const int per = (k_blocks + r - 1) / r;
            if ((long long)(r - 1) * per >= k_blocks) continue;                 // an empty last range
            const long long cost = (left * r + pairs - 1) / pairs * (r > 1 && per < 26 ? 26 : per);
            if (best < 0 || cost < best) best = cost, tail = r;
        }
        splits = 1;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(2 * pairs));
    lc.blockDim = dim3(THREADS);
    lc.dynamicSmemBytes = cfg::SMEM_BYTES;
    lc.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = llmx_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&lc, gemm_tc_pair_kernel<BN, FORM>, wide, narrow, C, wide_rows, narrow_rows, K, mode, splits, group,
                       tail, error_word, hp);
    return launch_status();
}

}  // namespace

// C (+)= A W^T on pairs of SMs.  `weight_map`: the weight's tensor map with boxes of 128 rows x 64 columns (the one
// llmx_gemm_tc_weight_map makes); A [M, K] bfloat16; C float32 [M, N]; mode 0 stores, 1 adds (float atomics);
// `splits` > 1 (mode 1 only) cuts K into ranges; `splits` 0 (mode 1 only) runs whole tiles while they fill every pair
// and cuts only the remaining tiles' K, so that the last round is not half empty; `token_tile` 128 or 256.
LLMX_EXPORT int llmx_gemm_tc_pair(const void* weight_map, const void* A, float* C, int M, int N, int K, int mode, int splits,
                                  int token_tile, int* error_word, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)A & 15) || ((uintptr_t)C & 3)) return LLMX_ERR_UNSUPPORTED;
    if ((mode != MODE_STORE && mode != MODE_ACCUMULATE) || splits < 0 || (splits != 1 && mode != MODE_ACCUMULATE))
        return LLMX_ERR_BAD_ARGUMENT;
    if (token_tile != 128 && token_tile != 256) return LLMX_ERR_BAD_ARGUMENT;
    ensure_sm_count();
    const int k_blocks = (K + BK - 1) / BK;
    if (splits > k_blocks) splits = k_blocks;
    const CUtensorMap& map_w = *(const CUtensorMap*)weight_map;
    CUtensorMap map_a;
    if (int e = llmx_make_map_bf16_2d(&map_a, A, (uint64_t)M, (uint64_t)K, token_tile / 2, BK)) return e;
    if (token_tile == 128) return launch_pair<128, PLAIN>(map_w, map_a, C, N, M, K, mode, splits, HeadsEpilogue{}, error_word, stream);
    return launch_pair<256, PLAIN>(map_w, map_a, C, N, M, K, mode, splits, HeadsEpilogue{}, error_word, stream);
}

// out[m, n] = silu(A W[n]^T) * (A W[n + N]^T) as bfloat16 [M, N] on pairs of SMs; the weight has 2 N rows (gate rows,
// then up rows) and `weight_map` boxes of 128 rows.  A pair's tile: 256 outputs x 128 tokens.
LLMX_EXPORT int llmx_gemm_tc_pair_swiglu(const void* weight_map, const void* A, void* out, int M, int N, int K,
                                         int* error_word, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)A & 15) || ((uintptr_t)out & 1)) return LLMX_ERR_UNSUPPORTED;
    ensure_sm_count();
    const CUtensorMap& map_w = *(const CUtensorMap*)weight_map;
    CUtensorMap map_a;
    if (int e = llmx_make_map_bf16_2d(&map_a, A, (uint64_t)M, (uint64_t)K, 64, BK)) return e;
    return launch_pair<128, DUAL>(map_w, map_a, out, N, M, K, MODE_STORE, 1, HeadsEpilogue{}, error_word, stream);
}

// The q/k/v product of a layer whose heads are 128 wide, finished in the epilogue, on pairs of SMs: the arguments of
// llmx_gemm_tc_heads, with the weight's map of 128-row boxes (llmx_gemm_tc_weight_map).  A pair's tile: 256 tokens x
// two heads.
LLMX_EXPORT int llmx_gemm_tc_pair_heads(const void* weight_map, const void* A, int tokens, int K, const float* q_weight,
                                        const float* k_weight, float eps, const float* cos_table, const float* sin_table,
                                        const int* positions, const int* slots, void* q_out, void* cache, int heads,
                                        int kv_heads, int page_size, int* error_word, cudaStream_t stream) {
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
    CUtensorMap map_tokens;
    if (int e = llmx_make_map_bf16_2d(&map_tokens, A, (uint64_t)tokens, (uint64_t)K, BM, BK)) return e;
    return launch_pair<256, HEADS>(map_tokens, *(const CUtensorMap*)weight_map, nullptr, tokens, features, K, MODE_STORE, 1, hp,
                                   error_word, stream);
}
