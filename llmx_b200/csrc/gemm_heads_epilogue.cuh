// The epilogue of a q/k/v product that finishes heads of 128 values itself, shared by the one-block product
// (gemm_tc.cu) and the product on pairs of SMs (gemm_tc_pair.cu): a thread holds one token's row of the accumulator
// in tensor memory, norms and rotates its query and key heads and writes queries and cache rows as bfloat16
// (src/model/arch/qwen3.hpp:280-290 for the order of operations).
#pragma once
#include "tc_common.cuh"
#include <math.h>

namespace {

// What the HEADS epilogue needs to finish heads of 128 values: norm weights (null: no norm), the rotation's
// tables [positions, 64] (null: no rotation), each token's position and cache slot (negative: not stored),
// the queries' output [tokens, heads * 128] and the layer's cache [pages, 2, kv_heads, page_size, 128].
struct HeadsEpilogue {
    const float* q_weight;
    const float* k_weight;
    const float* cos_table;
    const float* sin_table;
    const int* positions;
    const int* slots;
    __nv_bfloat16* q_out;
    __nv_bfloat16* cache;
    float eps;
    int heads, kv_heads, page_size;
};

__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The HEADS epilogue for one thread: token `tok` (this thread's lane of tensor memory), the tile's heads in the
// columns from `tcol` on.  A query or key head is normed (the sum of squares in the order of the per-head kernel
// in rowwise.cu: lane partials of four values, then the butterfly's tree, so both give the same bits), rotated
// as pairs (i, i + 64) and stored; a value head is stored as it is.  Every thread issues the tensor-memory loads
// (they are warp-wide); only those with a token, and for keys and values a cache slot, store.
template <int BN>
__device__ __forceinline__ void heads_epilogue(const HeadsEpilogue& hp, const float* norm_w, uint32_t tcol, int tok,
                                               int tokens, int feature0, int features) {
    constexpr int HEADS_PER_TILE = BN / 128;
    const bool live = tok < tokens;
    const int pos = live ? hp.positions[tok] : 0;
    const int slot = live ? hp.slots[tok] : -1;
    const int q_width = hp.heads * 128, kv_width = hp.kv_heads * 128;
    // What each head of the tile is, where it goes (null: nowhere) and, for a normed one, its scale.
    const float* weight[HEADS_PER_TILE];
    __nv_bfloat16* dst[HEADS_PER_TILE];
    bool rotate[HEADS_PER_TILE], normed[HEADS_PER_TILE];
    float rr[HEADS_PER_TILE];
#pragma unroll
    for (int hh = 0; hh < HEADS_PER_TILE; ++hh) {
        const int f = feature0 + hh * 128;
        weight[hh] = norm_w;
        dst[hh] = nullptr;
        rotate[hh] = normed[hh] = false;
        rr[hh] = 1.0f;
        if (f >= features) continue;
        if (f < q_width) {
            normed[hh] = hp.q_weight != nullptr;
            rotate[hh] = hp.cos_table != nullptr;
            if (live) dst[hh] = hp.q_out + ((size_t)tok * hp.heads + f / 128) * 128;
        } else {
            const bool is_k = f < q_width + kv_width;
            const int g = (f - q_width - (is_k ? 0 : kv_width)) / 128;
            weight[hh] = norm_w + 128;
            normed[hh] = is_k && hp.k_weight != nullptr;
            rotate[hh] = is_k && hp.cos_table != nullptr;
            if (slot >= 0) {
                const int page = slot / hp.page_size, off = slot % hp.page_size;
                dst[hh] = hp.cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * hp.kv_heads + g) * hp.page_size + off) * 128;
            }
        }
        if (normed[hh]) {           // uniform over the warp: the loads below are warp-wide
            float p[32];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tcol + hh * 128 + 32 * c, r);
                tc::tmem_wait_ld();
#pragma unroll
                for (int l = 0; l < 8; ++l) {
                    const float x0 = __uint_as_float(r[4 * l]), x1 = __uint_as_float(r[4 * l + 1]);
                    const float x2 = __uint_as_float(r[4 * l + 2]), x3 = __uint_as_float(r[4 * l + 3]);
                    p[8 * c + l] = fmaf(x0, x0, fmaf(x1, x1, fmaf(x2, x2, x3 * x3)));
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < o; ++i) p[i] = p[i] + p[i + o];
            rr[hh] = 1.0f / sqrtf(p[0] / 128.0f + hp.eps);
        }
    }
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
        // values 32 half .. + 31 (a) and their partners 64 further on (b); the angles are the token's, the same
        // for every head, and read-only: asked for before the accumulators so that their latency is not in line
        float4 c4[8], s4[8];
        if (hp.cos_table) {
            const float4* cs = reinterpret_cast<const float4*>(hp.cos_table + (size_t)pos * 64 + 32 * half);
            const float4* sn = reinterpret_cast<const float4*>(hp.sin_table + (size_t)pos * 64 + 32 * half);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                c4[i] = __ldg(cs + i);
                s4[i] = __ldg(sn + i);
            }
        }
#pragma unroll
        for (int hh = 0; hh < HEADS_PER_TILE; ++hh) {
            if (feature0 + hh * 128 >= features) break;
            uint32_t a[32], b[32];
            tc::tmem_ld_32x32(tcol + hh * 128 + 32 * half, a);
            tc::tmem_ld_32x32(tcol + hh * 128 + 64 + 32 * half, b);
            tc::tmem_wait_ld();
            if (dst[hh] == nullptr) continue;
            const float* w = weight[hh];
#pragma unroll
            for (int j8 = 0; j8 < 32; j8 += 8) {
                float ya[8], yb[8];
#pragma unroll
                for (int j4 = 0; j4 < 8; j4 += 4) {
                    const float4 cq = c4[(j8 + j4) / 4], sq = s4[(j8 + j4) / 4];
                    const float cc[4] = {cq.x, cq.y, cq.z, cq.w}, ss[4] = {sq.x, sq.y, sq.z, sq.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = j8 + j4 + e;
                        float xa = __uint_as_float(a[j]), xb = __uint_as_float(b[j]);
                        if (normed[hh]) {
                            xa *= rr[hh] * w[32 * half + j];
                            xb *= rr[hh] * w[64 + 32 * half + j];
                        }
                        if (rotate[hh]) {
                            ya[j4 + e] = fmaf(-xb, ss[e], xa * cc[e]);
                            yb[j4 + e] = fmaf(xa, ss[e], xb * cc[e]);
                        } else {
                            ya[j4 + e] = xa;
                            yb[j4 + e] = xb;
                        }
                    }
                }
                *reinterpret_cast<uint4*>(dst[hh] + 32 * half + j8) =
                    make_uint4(pack2_bf16(ya[0], ya[1]), pack2_bf16(ya[2], ya[3]), pack2_bf16(ya[4], ya[5]),
                               pack2_bf16(ya[6], ya[7]));
                *reinterpret_cast<uint4*>(dst[hh] + 64 + 32 * half + j8) =
                    make_uint4(pack2_bf16(yb[0], yb[1]), pack2_bf16(yb[2], yb[3]), pack2_bf16(yb[4], yb[5]),
                               pack2_bf16(yb[6], yb[7]));
            }
        }
    }
}

}  // namespace
