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

// A cache [pages, 2, kv_heads, page_size, head_dim] (bfloat16) as a five-dimensional tensor
//   (column in a 64-wide half: 64) x (slot: page_size) x (half of the head: head_dim / 64) x (kv head) x (page * 2 + plane)
// so that one box {64, page_size, head_dim / 64, 1, 2} is everything one kv head needs of one page: its keys
// and its values.  In shared memory the box lies as [plane][half][slot][64 columns]: per plane and half one
// run of page_size rows of 128 bytes under the 128-byte swizzle.
static inline int llmx_make_cache_map(CUtensorMap* map, const void* cache, uint64_t pages, uint64_t kv_heads,
                                      uint32_t page_size, uint64_t head_dim) {
    llmx_encode_tiled_fn enc = llmx_encode_tiled();
    if (!enc) return 10003;
    const uint64_t halves = head_dim / attn::BOX_COLS;
    const cuuint64_t dims[5] = {(cuuint64_t)attn::BOX_COLS, page_size, halves, kv_heads, pages * 2};
    const cuuint64_t strides[4] = {head_dim * 2, (cuuint64_t)attn::BOX_COLS * 2, (cuuint64_t)page_size * head_dim * 2,
                                   kv_heads * page_size * head_dim * 2};
    const cuuint32_t box[5] = {(cuuint32_t)attn::BOX_COLS, page_size, (cuuint32_t)halves, 1, 2};
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 10003;
}
