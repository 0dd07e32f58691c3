// Plain paged attention: one block per (query row, head), any head width, any batch mix.
//
// The attention of the true 32-bit path, and the slow-but-general form of the
// bfloat16 path for shapes its tiled kernels refuse.  A row at position p attends the
// keys lo..p of its own request, lo = max(0, p - window + 1) (window <= 0: lo = 0);
// query head h reads kv head h / (heads / kv_heads).
//   s_t = dot(q, k_t) * scale;  m = max s;  e_t = exp(s_t - m);  l = sum e_t;  o = sum_t (e_t / l) v_t
// (src/backends/cpu/cpu_backend.hpp:980-1029), computed in the online form (m, l, acc)
// and divided at the end as the reference's device kernels do (f32.gpu:1640-1709).
// Each warp walks every fourth key in increasing order; the four partial states are
// merged in warp order, so the order of a row's sums depends on its own keys only.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 8;  // head widths up to 256

template <typename QT, typename KVT>
__global__ void __launch_bounds__(WARPS * 32)
attention_plain_kernel(const QT* __restrict__ q, const KVT* __restrict__ cache, QT* __restrict__ out,
                       const int* __restrict__ row_request, const int* __restrict__ positions,
                       const int* __restrict__ block_tables, int table_stride, int heads, int kv_heads, int head_dim,
                       int page_size, int window, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];  // WARPS * (head_dim + 2)
    const int row = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (heads / kv_heads);
    const int pos = positions[row];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_tables + (size_t)row_request[row] * table_stride;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const QT* qrow = q + ((size_t)row * heads + h) * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < head_dim ? to_float(qrow[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int t = lo + warp; t <= pos; t += WARPS) {
        const int page = table[t / page_size], off = t % page_size;
        const KVT* kp = cache + ((((size_t)page * 2 + 0) * kv_heads + g) * page_size + off) * head_dim;
        const KVT* vp = cache + ((((size_t)page * 2 + 1) * kv_heads + g) * page_size + off) * head_dim;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) s = fmaf(qv[i], to_float(kp[d]), s);
        }
        s = warp_sum(s) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) acc[i] = fmaf(e, to_float(vp[d]), acc[i] * corr);
        }
        m = m_new;
    }
    float* mine = smem + warp * (head_dim + 2);
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) mine[d] = acc[i];
    }
    if (lane == 0) {
        mine[head_dim] = m;
        mine[head_dim + 1] = l;
    }
    __syncthreads();
    if (warp == 0) {
        float mm = -INFINITY;
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, smem[w * (head_dim + 2) + head_dim]);
        float ll = 0.0f;
        float f[WARPS];
        for (int w = 0; w < WARPS; ++w) {
            const float mw = smem[w * (head_dim + 2) + head_dim];
            f[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
            ll += smem[w * (head_dim + 2) + head_dim + 1] * f[w];
        }
        QT* orow = out + ((size_t)row * heads + h) * head_dim;
        for (int d = lane; d < head_dim; d += 32) {
            float o = 0.0f;
            for (int w = 0; w < WARPS; ++w) o += smem[w * (head_dim + 2) + d] * f[w];
            orow[d] = from_float<QT>(o / ll);
        }
    }
}
}  // namespace

// q/out [rows, heads, head_dim] of `q_dtype`; the cache [pages, 2, kv_heads, page_size, head_dim] of `cache_dtype`
// (the two may differ: bfloat16 products over a float32 cache, or the reverse).
LLMX_EXPORT int llmx_attention_plain(const void* q, int q_dtype, const void* cache, int cache_dtype, void* out,
                                     const int* row_request, const int* positions, const int* block_tables,
                                     int table_stride, int rows, int heads, int kv_heads, int head_dim, int page_size,
                                     int window, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (head_dim <= 0 || head_dim > 32 * MAX_PER_LANE || heads % kv_heads || heads > 65535) return LLMX_ERR_UNSUPPORTED;
    dim3 grid(rows, heads);
    const size_t shmem = (size_t)WARPS * (head_dim + 2) * sizeof(float);
#define LLMX_PLAIN(QT, KVT)                                                                                            \
    launch_kernel(attention_plain_kernel<QT, KVT>, dim3(grid), dim3(WARPS * 32), shmem, stream, (const QT*)q,         \
                  (const KVT*)cache, (QT*)out, row_request, positions, block_tables, table_stride, heads, kv_heads,   \
                  head_dim, page_size, window, scale)
    if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_PLAIN(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_PLAIN(__nv_bfloat16, float);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_PLAIN(float, __nv_bfloat16);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_PLAIN(float, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_PLAIN
    return launch_status();
}
