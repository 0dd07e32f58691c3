// Pieces shared by the tiled bfloat16 attention kernels: warp-level matrix fragments over
// TMA-swizzled shared memory, and the online softmax bookkeeping.
//
// Keys and values reach shared memory page by page through TMA boxes of [page rows, 64 columns]
// with the 128-byte swizzle: the 16-byte chunk c of row r lies at chunk (c ^ (r & 7)), which lets
// ldmatrix read eight rows of one chunk column without bank conflicts.  A head of D columns is
// D / 64 such boxes side by side.
#pragma once
#include "tc_common.cuh"

namespace attn {

constexpr int BOX_COLS = 64;            // bfloat16 columns per box = one 128-byte swizzle row
constexpr float LOG2E = 1.4426950408889634f;

// Byte offset, inside a box whose base is 1024-byte aligned, of the 16-byte chunk `chunk` (0..7) of row `row`.
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// d (16x8, float32) += a (16x16 bfloat16, row) * b (16x8 bfloat16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace attn

// A cache [pages, 2, kv_heads, page_size, head_dim] seen as rows of head_dim bfloat16, in boxes of
// [page_size rows, 64 columns].  Row of (page, plane, head, slot) = ((page * 2 + plane) * kv_heads + head) * page_size + slot.
static inline int llmx_make_cache_map(CUtensorMap* map, const void* cache, uint64_t rows, uint64_t head_dim,
                                      uint32_t page_size) {
    return llmx_make_map_bf16_2d(map, cache, rows, head_dim, page_size, attn::BOX_COLS);
}
