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
// The kernel is persistent: a block walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// with three roles:  warp 0 loads (TMA producer), warp 1 issues the matrix instructions,
// warps 2-5 are the epilogue.  Two accumulators in tensor memory let the epilogue of one tile
// overlap the products of the next.  `splits` > 1 cuts K into ranges that are added into C
// with float atomics (only with accumulate, where C already holds the residual).
//
// The reference has no tensor-core path for this product (its kernels: f32.gpu:1034-1084).
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;      // weight rows per tile (the instruction's M)
constexpr int BK = 64;       // bfloat16 elements per k block: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 4;
constexpr int THREADS = 64 + EPI_WARPS * 32;

enum : int { MODE_STORE = 0, MODE_ACCUMULATE = 1 };
enum : int { ERR_PRODUCER = 101, ERR_MMA_FULL = 102, ERR_MMA_ACC = 103, ERR_EPILOGUE = 104 };

template <int BN>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2;          // weight tile
    static constexpr int B_BYTES = BN * BK * 2;          // token tile
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
               float* __restrict__ C, int M, int N, int K, int mode, int splits, int* error_word) {
    using cfg = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* full_bar = (uint64_t*)(smem + cfg::STAGES * cfg::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + cfg::STAGES;
    uint64_t* acc_full = empty_bar + cfg::STAGES;     // [2]
    uint64_t* acc_empty = acc_full + 2;               // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (N + BM - 1) / BM, m_tiles = (M + BN - 1) / BN;
    const int k_blocks_total = (K + BK - 1) / BK;
    const int k_per_split = (k_blocks_total + splits - 1) / splits;
    const int total = n_tiles * m_tiles * splits;

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
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // A work item is (n tile, m tile, k split); m tiles vary fastest so neighbouring blocks share a weight tile.
    if (warp == 0) {
        if (tc::elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
                const int mt = item % m_tiles, rest = item / m_tiles;
                const int nt = rest % n_tiles, sp = rest / n_tiles;
                const int kb0 = sp * k_per_split, kb1 = min(k_blocks_total, kb0 + k_per_split);
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = tc::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, error_word, ERR_PRODUCER);
                    if (!ok) break;
                    uint8_t* a_dst = tiles + stage * cfg::STAGE_BYTES;
                    uint8_t* b_dst = a_dst + cfg::A_BYTES;
                    tc::mbar_expect_tx(&full_bar[stage], cfg::STAGE_BYTES);
                    tc::tma_load_2d(a_dst, &map_w, kb * BK, nt * BM, &full_bar[stage]);
                    tc::tma_load_2d(b_dst, &map_a, kb * BK, mt * BN, &full_bar[stage]);
                    if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = tc::instr_desc_bf16(BM, BN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
                const int sp = item / (m_tiles * n_tiles);
                const int kb0 = sp * k_per_split, kb1 = min(k_blocks_total, kb0 + k_per_split);
                ok = tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, error_word, ERR_MMA_ACC);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = tc::mbar_wait(&full_bar[stage], phase, abort_flag, error_word, ERR_MMA_FULL);
                    if (!ok) break;
                    tc::tc_fence_after();
                    const uint32_t a_addr = tc::smem_u32(tiles + stage * cfg::STAGE_BYTES);
                    const uint64_t desc_a = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t desc_b = tc::smem_desc_k_sw128(a_addr + cfg::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements = 32 bytes further along the swizzled row: +2 in the descriptor's 16-byte units.
                        tc::mma_bf16_ss(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
            const int mt = item % m_tiles, rest = item / m_tiles;
            const int nt = rest % n_tiles, sp = rest / n_tiles;
            const int kb0 = sp * k_per_split, kb1 = min(k_blocks_total, kb0 + k_per_split);
            ok = tc::mbar_wait(&acc_full[acc], acc_phase, abort_flag, error_word, ERR_EPILOGUE);
            if (!ok) break;
            tc::tc_fence_after();
            const int n = nt * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
            const bool atomic = splits > 1;
            if (kb1 > kb0) {
                constexpr int CH = BN < 32 ? 16 : 32;
#pragma unroll 1
                for (int c = 0; c < BN; c += CH) {
                    uint32_t r[CH];
                    if constexpr (CH == 32) tc::tmem_ld_32x32(taddr + c, r);
                    else tc::tmem_ld_32x16(taddr + c, r);
                    tc::tmem_wait_ld();
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            const int m = mt * BN + c + j;
                            if (m < M) {
                                float* dst = C + (size_t)m * N + n;
                                const float v = __uint_as_float(r[j]);
                                if (mode == MODE_STORE) *dst = v;
                                else if (atomic) atomicAdd(dst, v);
                                else *dst += v;
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

template <int BN>
int launch(const CUtensorMap& map_w, const void* A, float* C, int M, int N, int K, int mode, int splits,
           int* error_word, cudaStream_t stream) {
    using cfg = Cfg<BN>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES) !=
            cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    CUtensorMap map_a;
    if (int e = llmx_make_map_bf16_2d(&map_a, A, (uint64_t)M, (uint64_t)K, BN, BK)) return e;
    const int n_tiles = (N + BM - 1) / BM, m_tiles = (M + BN - 1) / BN;
    const int total = n_tiles * m_tiles * splits;
    const int grid = total < g_sm_count ? total : g_sm_count;
    gemm_tc_kernel<BN><<<grid, THREADS, cfg::SMEM_BYTES, stream>>>(map_w, map_a, C, M, N, K, mode, splits, error_word);
    return launch_status();
}

}  // namespace

// The weight's tensor map (128 rows x 64 columns per box) can be made once and kept: 128 bytes at `out`.
LLMX_EXPORT int llmx_gemm_tc_weight_map(void* out, const void* W, int N, int K) {
    if (K % 8 || ((uintptr_t)W & 15)) return LLMX_ERR_UNSUPPORTED;
    return llmx_make_map_bf16_2d((CUtensorMap*)out, W, (uint64_t)N, (uint64_t)K, BM, BK);
}

// mode 0: C = A W^T;  mode 1: C += A W^T.  `splits` > 1 (only with mode 1) cuts K and adds with atomics.
// `token_tile` is 16, 32, 64, 128 or 256 (0: chosen from M).  `error_word`: device int, zero before first use.
LLMX_EXPORT int llmx_gemm_tc(const void* weight_map, const void* A, float* C, int M, int N, int K, int mode,
                             int splits, int token_tile, int* error_word, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)A & 15) || ((uintptr_t)C & 3)) return LLMX_ERR_UNSUPPORTED;
    if (splits < 1 || (splits > 1 && mode != MODE_ACCUMULATE)) return LLMX_ERR_BAD_ARGUMENT;
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    const int k_blocks = (K + BK - 1) / BK;
    if (splits > k_blocks) splits = k_blocks;
    int bn = token_tile;
    if (bn == 0) bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    const CUtensorMap& map_w = *(const CUtensorMap*)weight_map;
    switch (bn) {
        case 16: return launch<16>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 32: return launch<32>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 64: return launch<64>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 128: return launch<128>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        case 256: return launch<256>(map_w, A, C, M, N, K, mode, splits, error_word, stream);
        default: return LLMX_ERR_BAD_ARGUMENT;
    }
}
