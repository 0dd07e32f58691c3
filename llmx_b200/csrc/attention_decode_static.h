// llmx_attn_decode_static: split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in mxxm-t/llmx; it exists for callers of this library that
// are not allowed to allocate device memory at the time they call it: code that runs inside
// another framework's memory plan, a plugin whose host owns every byte of the device and hands
// out none, a real-time loop that may not touch the allocator, or a process whose memory pool
// is already carved up.  llmx_attn_decode needs a float workspace for the partial results of its
// key ranges, which such a caller would have to cudaMalloc; here that workspace is a fixed array
// inside the library's own device image.
//
// What to know before using it:
//   * Size limit.  The array holds LLMX_ATTN_DECODE_STATIC_FLOATS floats (16 MiB).  A call needs
//     total_rows * heads * splits * (head_dim + 2) of them when splits > 1 and none when
//     splits == 1; a call that needs more is refused with error 10004 and nothing is launched.
//     Every GPU on which the library is loaded holds these 16 MiB until the process exits.
//   * Set-up.  The first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current) and remembers it.  Make that first call
//     outside any stream capture.  The call performs no cudaMalloc, cudaFree or other
//     allocating routine, on the first call or later.
//   * Sharing.  Every call on a device uses the same array and finds in it whatever the last
//     call left.  Nothing in it has to start at zero: each launch writes every partial result
//     it later reads.  For the same reason two calls whose kernels may overlap on the GPU
//     (different streams, no dependency between them) race on the array and must not be made;
//     calls on one stream are safe.
//   * The caller still passes inputs and outputs: queries, the cache's tensor map (made on the
//     host by llmx_attn_cache_map, which allocates nothing either), block tables, the output.
//
// Arguments are those of llmx_attn_decode without the workspace and the device-side chunk
// pointer, plus `total_rows`, the number of rows of q/out (the partial results are indexed by row).
//   * `total_rows` is taken on trust.  The rows a request brings (row_start, row_count) lie in
//     device memory, where this host-side check cannot read them: the size test above uses
//     total_rows alone.  A caller that passes fewer rows than row_start + row_count reach makes
//     the kernel write partial results past what was checked, possibly past the array.  Pass the
//     true row count of q/out.
//
// The header is plain C as well as C++ (a C caller links against the same exported symbol).
#pragma once
#include <cuda_runtime.h>

#define LLMX_ATTN_DECODE_STATIC_FLOATS (4 * 1024 * 1024)
#define LLMX_ERR_TOO_LARGE 10004

#ifdef __cplusplus
extern "C" {
#endif

int llmx_attn_decode_static(const void* cache_map, const void* q, void* out, const int* req_list, int n_req,
                                       const int* row_start, const int* row_count, const int* history,
                                       const int* block_tables, int table_stride, int total_rows, int heads,
                                       int kv_heads, int head_dim, int page_size, int window, float scale, int splits,
                                       int chunk_keys, int max_rows, int* error_word, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
