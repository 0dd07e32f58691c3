// Row-wise kernels: embedding gather, RMSNorm, per-head norm + rotation + cache write, SwiGLU.
//
// All arithmetic is 32-bit: sums of squares, the reciprocal root, the rotation
// and the activation.  Only what is stored for a matrix product or in the cache
// is rounded to bfloat16 on the bfloat16 path.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: x[r, :] = table[ids[r], :] widened to 32-bit.
// Reference: llmx_gather (src/backends/gpu/kernels/f32.gpu:747-751).  Ids are checked
// on the host before the step; an id outside the table writes a zero row here.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                             int width, int table_rows) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int id = ids[r];
    float* dst = x + (size_t)r * width;
    if (id < 0 || id >= table_rows) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    const T* src = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_float(src[i]);
}

LLMX_EXPORT int llmx_embed(const void* table, int table_dtype, const int* ids, float* x, int rows, int width,
                           int table_rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (table_dtype == LLMX_BF16)
        launch_kernel(embed_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, x, width, table_rows);
    else
        launch_kernel(embed_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)table, ids, x, width, table_rows);
    return launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm: s = sum x_i^2; r = 1 / sqrt(s / n + eps); y_i = x_i * (r * w_i)
// (the grouping x * (r * w) is the reference's, src/backends/cpu/cpu_backend.hpp:1437-1459).
// `row_index` (optional) picks the source rows: y[i] = norm(x[row_index[i]]), which folds
// the head's row gather (src/model/arch/blocks.hpp:267-272) into its norm.
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, OutT* __restrict__ y,
                               const int* __restrict__ row_index, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[r] : r) * width;
    float s = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = src[i];
        s = fmaf(v, v, s);
    }
    s = block_sum(s, scratch);
    const float rr = 1.0f / sqrtf(s / (float)width + eps);
    OutT* dst = y + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_float<OutT>(src[i] * (rr * w[i]));
}

// The same for widths that are a multiple of 4 and at most 4 * VEC_MAX * blockDim: each thread keeps its
// values in registers (one read of the row, 16-byte loads all issued before the first is used).
constexpr int NORM_VEC_MAX = 8;

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = v;
}

// `zero` (optional): a float buffer of `zero_count` values (a multiple of 4, 16-byte aligned) that the launch
// clears with blocks of its own (those beyond `rows`): the output of the product that follows, when that product
// adds its pieces with atomics.
template <typename OutT>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, OutT* __restrict__ y,
                                   const int* __restrict__ row_index, int rows, int width, float eps,
                                   float* __restrict__ zero, long long zero_count) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (r >= rows) {
        // Blocks beyond the rows only clear: with a few rows, a few blocks would store for longer than the norm takes.
        float4* z = reinterpret_cast<float4*>(zero);
        const long long n4 = zero_count >> 2;
        const long long blocks = gridDim.x - rows;
        for (long long i = (long long)(r - rows) * blockDim.x + threadIdx.x; i < n4; i += blocks * blockDim.x)
            z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[r] : r) * width);
    const float4* wv = reinterpret_cast<const float4*>(w);
    const int n4 = width >> 2;
    float4 v[NORM_VEC_MAX];
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; ++k) {
        s = fmaf(v[k].x, v[k].x, s);
        s = fmaf(v[k].y, v[k].y, s);
        s = fmaf(v[k].z, v[k].z, s);
        s = fmaf(v[k].w, v[k].w, s);
    }
    s = block_sum(s, scratch);
    const float rr = 1.0f / sqrtf(s / (float)width + eps);
    OutT* dst = y + (size_t)r * width;
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            const float4 ww = wv[i];
            store4(dst + 4 * i, v[k].x * (rr * ww.x), v[k].y * (rr * ww.y), v[k].z * (rr * ww.z), v[k].w * (rr * ww.w));
        }
    }
}

LLMX_EXPORT int llmx_rmsnorm(const float* x, const float* w, void* y, int out_dtype, const int* row_index, int rows,
                             int width, float eps, float* zero, long long zero_count, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (zero && (zero_count % 4 || ((uintptr_t)zero & 15))) return LLMX_ERR_BAD_ARGUMENT;
    const bool aligned = width % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)w & 15) && !((uintptr_t)y & 15);
    if (aligned && width <= 4 * NORM_VEC_MAX * 256) {
        const int n4 = width / 4;
        // The block width depends on the row width alone, so a row's sum has one order whatever the batch.
        int threads = ((n4 + 3) / 4 + 31) / 32 * 32;
        threads = threads < 32 ? 32 : threads > 256 ? 256 : threads;
        // Clearing: blocks of their own, each about 16 KB (four 16-byte stores a thread), at most 1,024 of them.
        long long zero_blocks = zero ? (zero_count / 4 + 4 * threads - 1) / (4 * threads) : 0;
        zero_blocks = zero_blocks > 1024 ? 1024 : zero_blocks;
        const dim3 grid((unsigned)(rows + zero_blocks));
        if (out_dtype == LLMX_BF16)
            launch_kernel(rmsnorm_vec_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, x, w, (__nv_bfloat16*)y, row_index, rows, width, eps, zero, zero_count);
        else
            launch_kernel(rmsnorm_vec_kernel<float>, grid, dim3(threads), 0, stream, x, w, (float*)y, row_index, rows, width, eps, zero, zero_count);
        return launch_status();
    }
    if (zero && cudaMemsetAsync(zero, 0, (size_t)zero_count * sizeof(float), stream) != cudaSuccess) return launch_status();
    const int threads = width >= 1024 ? 256 : 128;
    if (out_dtype == LLMX_BF16)
        launch_kernel(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, w, (__nv_bfloat16*)y, row_index, width, eps);
    else
        launch_kernel(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, w, (float*)y, row_index, width, eps);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Per-head norm, rotation and cache write, one warp per (row, head).
//
// For a query head: RMSNorm over the head's D values with q_weight (skipped when null),
// rotate the first 2*rot_half values by the row's position, store to q_out.
// For a key head: the same with k_weight, stored to the key plane of the row's cache
// slot; the value head is stored raw to the value plane.
// Rotation pairs (i, i + rot_half), i < rot_half ("rotate half"):
//   a' = fma(-b, sin_i, a * cos_i);  b' = fma(a, sin_i, b * cos_i)
// (src/backends/cpu/cpu_backend.hpp:1461-1480, fused form f32.gpu:722-744).
// Cache layout: [page][plane][kv_head][slot][D]; `slots[row]` = page * page_size + slot,
// or negative to skip the write (a layer that reads another layer's cache).
// ---------------------------------------------------------------------------
template <typename QT, typename KVT>
__global__ void head_norm_rope_kernel(const float* __restrict__ qkv, int qkv_stride, int k_offset, int v_offset,
                                      const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                      float eps, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                      int rot_half, const int* __restrict__ positions, const int* __restrict__ slots,
                                      QT* __restrict__ q_out, KVT* __restrict__ cache, int rows, int heads, int kv_heads,
                                      int head_dim, int page_size) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_row = heads + kv_heads;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)rows * per_row) return;
    const int row = (int)(item / per_row), j = (int)(item % per_row);
    const bool is_q = j < heads;
    const int g = is_q ? 0 : j - heads;
    float* buf = smem + warp * head_dim;
    const float* src = qkv + (size_t)row * qkv_stride + (is_q ? j * head_dim : k_offset + g * head_dim);
    const float* weight = is_q ? q_weight : k_weight;

    int slot = 0;
    if (!is_q) {
        slot = slots[row];
        if (slot < 0) return;
    }
    float s = 0.0f;
    for (int d = lane; d < head_dim; d += 32) {
        const float v = src[d];
        buf[d] = v;
        s = fmaf(v, v, s);
    }
    if (weight) {
        s = warp_sum(s);
        const float rr = 1.0f / sqrtf(s / (float)head_dim + eps);
        __syncwarp();
        for (int d = lane; d < head_dim; d += 32) buf[d] = buf[d] * (rr * weight[d]);
    }
    __syncwarp();
    size_t key_base = 0, value_base = 0;
    if (!is_q) {
        const int page = slot / page_size, off = slot % page_size;
        key_base = ((((size_t)page * 2 + 0) * kv_heads + g) * page_size + off) * head_dim;
        value_base = ((((size_t)page * 2 + 1) * kv_heads + g) * page_size + off) * head_dim;
    }
    const float* cs = cos_table ? cos_table + (size_t)positions[row] * rot_half : nullptr;
    const float* sn = cos_table ? sin_table + (size_t)positions[row] * rot_half : nullptr;
    for (int d = lane; d < head_dim; d += 32) {
        float out;
        if (cs && d < 2 * rot_half) {
            const int i = d < rot_half ? d : d - rot_half;
            const float a = buf[i], b = buf[i + rot_half];
            out = d < rot_half ? fmaf(-b, sn[i], a * cs[i]) : fmaf(a, sn[i], b * cs[i]);
        } else {
            out = buf[d];
        }
        if (is_q) q_out[(size_t)row * heads * head_dim + j * head_dim + d] = from_float<QT>(out);
        else cache[key_base + d] = from_float<KVT>(out);
    }
    if (!is_q) {
        const float* vsrc = qkv + (size_t)row * qkv_stride + v_offset + g * head_dim;
        for (int d = lane; d < head_dim; d += 32) cache[value_base + d] = from_float<KVT>(vsrc[d]);
    }
}

// The same for the common shape -- a head of 128 values rotated whole (64 pairs) -- with each lane holding
// four consecutive values (16-byte loads, 8-byte stores); a pair's partner sits 16 lanes away.  A warp takes
// U consecutive (row, head) items of one row (U divides heads + kv_heads): their loads are all asked for
// before the first is used, and the row's position, cosines and sines are fetched once.
template <typename QT, typename KVT, int U>
__global__ void head_norm_rope_128_kernel(const float* __restrict__ qkv, int qkv_stride, int k_offset, int v_offset,
                                          const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                          float eps, const float* __restrict__ cos_table,
                                          const float* __restrict__ sin_table, const int* __restrict__ positions,
                                          const int* __restrict__ slots, QT* __restrict__ q_out, KVT* __restrict__ cache,
                                          int rows, int heads, int kv_heads, int page_size) {
    pdl_trigger();
    pdl_wait();
    constexpr int D = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_row = heads + kv_heads;
    // 32-bit arithmetic (the launcher sees to it that rows * per_row fits): a 64-bit division costs this
    // kernel, which is bound by the instructions it issues, a tenth of its time.
    const unsigned first = (blockIdx.x * (blockDim.x >> 5) + warp) * U;
    if (first >= (unsigned)rows * (unsigned)per_row) return;
    const int row = (int)(first / (unsigned)per_row), j0 = (int)(first - (unsigned)row * (unsigned)per_row);
    const float* row_src = qkv + (size_t)row * qkv_stride;
    const int slot = slots[row];
    float4 v[U], raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int j = j0 + u;
        const bool is_q = j < heads;
        const int g = is_q ? 0 : j - heads;
        v[u] = reinterpret_cast<const float4*>(row_src + (is_q ? j * D : k_offset + g * D))[lane];
        if (!is_q && slot >= 0) raw[u] = reinterpret_cast<const float4*>(row_src + v_offset + g * D)[lane];
    }
    float4 c = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cos_table) {
        // Lane l < 16 holds a = x[4l..4l+3], lane l + 16 holds b = x[64 + 4l ..]; both need cos/sin[4 (l % 16) ..].
        const size_t base = (size_t)positions[row] * 64 + 4 * (lane & 15);
        c = *reinterpret_cast<const float4*>(cos_table + base);
        sn = *reinterpret_cast<const float4*>(sin_table + base);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int j = j0 + u;
        const bool is_q = j < heads;
        const int g = is_q ? 0 : j - heads;
        if (!is_q && slot < 0) continue;
        const float* weight = is_q ? q_weight : k_weight;
        float4 x = v[u];
        if (weight) {
            float s = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, x.w * x.w)));
            s = warp_sum(s);
            const float rr = 1.0f / sqrtf(s / (float)D + eps);
            const float4 w4 = reinterpret_cast<const float4*>(weight)[lane];
            x.x *= rr * w4.x; x.y *= rr * w4.y; x.z *= rr * w4.z; x.w *= rr * w4.w;
        }
        if (cos_table) {
            float4 o;
            o.x = __shfl_xor_sync(0xffffffffu, x.x, 16); o.y = __shfl_xor_sync(0xffffffffu, x.y, 16);
            o.z = __shfl_xor_sync(0xffffffffu, x.z, 16); o.w = __shfl_xor_sync(0xffffffffu, x.w, 16);
            if (lane < 16) {        // a' = fma(-b, sin, a cos)
                x.x = fmaf(-o.x, sn.x, x.x * c.x); x.y = fmaf(-o.y, sn.y, x.y * c.y);
                x.z = fmaf(-o.z, sn.z, x.z * c.z); x.w = fmaf(-o.w, sn.w, x.w * c.w);
            } else {                // b' = fma(a, sin, b cos)
                x.x = fmaf(o.x, sn.x, x.x * c.x); x.y = fmaf(o.y, sn.y, x.y * c.y);
                x.z = fmaf(o.z, sn.z, x.z * c.z); x.w = fmaf(o.w, sn.w, x.w * c.w);
            }
        }
        if (is_q) {
            store4(q_out + ((size_t)row * heads + j) * D + 4 * lane, x.x, x.y, x.z, x.w);
        } else {
            const int page = slot / page_size, off = slot % page_size;
            const size_t key_base = ((((size_t)page * 2 + 0) * kv_heads + g) * page_size + off) * D;
            const size_t value_base = ((((size_t)page * 2 + 1) * kv_heads + g) * page_size + off) * D;
            store4(cache + key_base + 4 * lane, x.x, x.y, x.z, x.w);
            store4(cache + value_base + 4 * lane, raw[u].x, raw[u].y, raw[u].z, raw[u].w);
        }
    }
}

template <typename T, int U>
static void launch_head_norm_rope_128(const float* qkv, int qkv_stride, int k_offset, int v_offset, const float* q_weight,
                                      const float* k_weight, float eps, const float* cos_table, const float* sin_table,
                                      const int* positions, const int* slots, void* q_out, void* cache, int rows,
                                      int heads, int kv_heads, int page_size, cudaStream_t stream) {
    const int warps = 4;
    const long long groups = (long long)rows * (heads + kv_heads) / U;
    launch_kernel(head_norm_rope_128_kernel<T, T, U>, dim3((unsigned)((groups + warps - 1) / warps)), dim3(warps * 32), 0,
                  stream, qkv, qkv_stride, k_offset, v_offset, q_weight, k_weight, eps, cos_table, sin_table, positions,
                  slots, (T*)q_out, (T*)cache, rows, heads, kv_heads, page_size);
}

LLMX_EXPORT int llmx_head_norm_rope_kv(const float* qkv, int qkv_stride, int k_offset, int v_offset,
                                       const float* q_weight, const float* k_weight, float eps,
                                       const float* cos_table, const float* sin_table, int rot_half,
                                       const int* positions, const int* slots, void* q_out, int q_dtype, void* cache,
                                       int cache_dtype, int rows, int heads, int kv_heads, int head_dim,
                                       int page_size, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (head_dim <= 0 || rot_half < 0 || 2 * rot_half > head_dim) return LLMX_ERR_BAD_ARGUMENT;
    const int warps = 4;
    const long long items = (long long)rows * (heads + kv_heads);
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    const bool fast = q_dtype == cache_dtype && head_dim == 128 && (!cos_table || rot_half == 64) && qkv_stride % 4 == 0 && k_offset % 4 == 0 &&
                      v_offset % 4 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)q_out & 15) && !((uintptr_t)cache & 15) &&
                      !((uintptr_t)q_weight & 15) && !((uintptr_t)k_weight & 15) && !((uintptr_t)cos_table & 15) &&
                      !((uintptr_t)sin_table & 15);
    if (fast) {
        // Many rows: two items a warp (measured at 2,048 rows of 48 heads: one 24, two 20.5, four 22 us: more items
        // a warp cost registers, and with them resident warps); few rows: one item a warp keeps more warps busy.
        const int per_row = heads + kv_heads;
        if ((long long)rows * per_row >= (1ll << 31)) return LLMX_ERR_UNSUPPORTED;
        const int u = rows >= 64 && per_row % 2 == 0 ? 2 : 1;
#define LLMX_HNR(T, U) launch_head_norm_rope_128<T, U>(qkv, qkv_stride, k_offset, v_offset, q_weight, k_weight, eps, cos_table, \
                                                       sin_table, positions, slots, q_out, cache, rows, heads, kv_heads, page_size, stream)
        if (q_dtype == LLMX_BF16) {
            if (u == 2) LLMX_HNR(__nv_bfloat16, 2); else LLMX_HNR(__nv_bfloat16, 1);
        } else {
            if (u == 2) LLMX_HNR(float, 2); else LLMX_HNR(float, 1);
        }
#undef LLMX_HNR
        return launch_status();
    }
    const size_t shmem = (size_t)warps * head_dim * sizeof(float);
    // The general form takes queries and cache of different types (bfloat16 products over a float32 cache, or the reverse).
#define LLMX_HNR_ANY(QT, KVT)                                                                                           \
    launch_kernel(head_norm_rope_kernel<QT, KVT>, dim3(blocks), dim3(warps * 32), shmem, stream, qkv, qkv_stride,      \
                  k_offset, v_offset, q_weight, k_weight, eps, cos_table, sin_table, rot_half, positions, slots,       \
                  (QT*)q_out, (KVT*)cache, rows, heads, kv_heads, head_dim, page_size)
    if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_HNR_ANY(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_HNR_ANY(__nv_bfloat16, float);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_HNR_ANY(float, __nv_bfloat16);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_HNR_ANY(float, float);
    else return LLMX_ERR_BAD_ARGUMENT;
#undef LLMX_HNR_ANY
    return launch_status();
}

// ---------------------------------------------------------------------------
// SwiGLU: act = silu(g) * u, silu(g) = g / (1 + exp(-g))
// (src/backends/cpu/cpu_backend.hpp:1677; f32.gpu:596-631).  `gu` holds a row's gate
// values then its up values ([rows, 2 * width]).
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void swiglu_kernel(const float* __restrict__ gu, OutT* __restrict__ act, long long total, int width) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / width;
    const int c = (int)(i % width);
    const float g = gu[r * 2 * width + c], u = gu[r * 2 * width + width + c];
    act[i] = from_float<OutT>(g / (1.0f + expf(-g)) * u);
}

LLMX_EXPORT int llmx_swiglu(const float* gu, void* act, int out_dtype, int rows, int width, cudaStream_t stream) {
    const long long total = (long long)rows * width;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == LLMX_BF16) launch_kernel(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, gu, (__nv_bfloat16*)act, total, width);
    else launch_kernel(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, gu, (float*)act, total, width);
    return launch_status();
}
