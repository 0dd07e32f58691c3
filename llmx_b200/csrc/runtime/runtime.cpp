// The native runtime: parts, launch plans and the model's forward pass (see llmx_runtime.h).
//
// Host code only.  Kernels are called through `K`, a table of the kernel libraries' exported entry points.
// Intermediates of a step come from the step's workspace by bump allocation (a block gives its share back when
// it is done), so a forward pass allocates nothing; `llmx_model_workspace` walks the same code without
// launching to find how much a step needs.
#include "llmx_runtime.h"

#include <cuda_runtime.h>
#include <dirent.h>
#include <dlfcn.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#define LLMX_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;
int fail(int code, const std::string& what) {
    g_error = what;
    return code;
}

// ---------------------------------------------------------------------------------------------------------------
// The kernel table.  Signatures are those of the `extern "C"` entry points of the .cu files beside this folder.
// ---------------------------------------------------------------------------------------------------------------
typedef cudaStream_t S;
#define LLMX_KERNELS(X)                                                                                                  \
    X(llmx_embed, (const void*, int, const int*, float*, int, int, int, S))                                               \
    X(llmx_rmsnorm, (const float*, const float*, void*, int, const int*, int, int, float, float*, long long, S))          \
    X(llmx_head_norm_rope_kv, (const float*, int, int, int, const float*, const float*, float, const float*,              \
                               const float*, int, const int*, const int*, void*, int, void*, int, int, int, int, int,     \
                               int, S))                                                                                   \
    X(llmx_swiglu, (const float*, void*, int, int, int, S))                                                               \
    X(llmx_gemm_plain, (const void*, int, const void*, int, float*, int, int, int, int, S))                               \
    X(llmx_attention_plain, (const void*, int, const void*, int, void*, const int*, const int*, const int*, int, int,     \
                             int, int, int, int, int, float, S))                                                          \
    X(llmx_gemm_tc_weight_map, (void*, const void*, int, int))                                                            \
    X(llmx_gemm_tc_weight_map_box, (void*, const void*, int, int, int))                                                   \
    X(llmx_gemm_tc, (const void*, const void*, float*, int, int, int, int, int, int, int, int*, S))                       \
    X(llmx_gemm_tc_pair, (const void*, const void*, float*, int, int, int, int, int, int, int*, S))                       \
    X(llmx_gemm_tc_pair_swiglu, (const void*, const void*, void*, int, int, int, int*, S))                                \
    X(llmx_gemm_tc_pair_heads, (const void*, const void*, int, int, const float*, const float*, float, const float*,      \
                                const float*, const int*, const int*, void*, void*, int, int, int, int*, S))              \
    X(llmx_gemm_tc_swiglu, (const void*, const void*, void*, int, int, int, int, int*, S))                                \
    X(llmx_gemm_tc_heads, (const void*, const void*, int, int, int, const float*, const float*, float, const float*,      \
                           const float*, const int*, const int*, void*, void*, int, int, int, int*, S))                   \
    X(llmx_attn_cache_map, (void*, const void*, long long, int, int, int))                                                \
    X(llmx_attn_decode_fused, (const void*, const void*, void*, float*, const int*, int, const int*, const int*,          \
                               const int*, const int*, int, int, int, int, int, int, float, int, const int*, int, int,    \
                               int*, int*, S))                                                                            \
    X(llmx_attn_decode_qkv, (const void*, const float*, int, int, int, const float*, const float*, float, const float*,   \
                             const float*, const int*, void*, void*, float*, const int*, int, const int*, const int*,     \
                             const int*, const int*, int, int, int, int, int, int, float, int, const int*, int, int,      \
                             int*, int*, S))                                                                              \
    X(llmx_attn_decode_max_clusters, (int, int))                                                                          \
    X(llmx_attn_prefill_tc_cache_map, (void*, const void*, long long, int, int, int))                                     \
    X(llmx_attn_prefill_tc, (const void*, const void*, void*, int, const int*, int, const int*, const int*, const int*,   \
                             const int*, int, int, int, int, int, int, float, int, int, int, float*, int*, S))            \
    X(llmx_attn_prefill, (const void*, const void*, void*, const int*, int, const int*, const int*, const int*,           \
                          const int*, int, int, int, int, int, int, float, int, int*, S))                                 \
    X(llmx_sample, (const float*, int, int, const void*, int*, int, S))                                                   \
    X(llmx_penalize, (float*, int, const int*, const int*, const int*, const float*, const float*, const float*, int, S))

struct Kernels {
#define X(name, args) int(*name) args = nullptr;
    LLMX_KERNELS(X)
#undef X
} kern;

bool bind(const char* name, void* fn) {
#define X(kname, args)                                \
    if (!strcmp(name, #kname)) {                      \
        kern.kname = reinterpret_cast<int(*) args>(fn);  \
        return true;                                  \
    }
    LLMX_KERNELS(X)
#undef X
    return false;
}

long long g_launches = 0;
bool g_profile = false;
// Entry points a dry run would have called and found unbound: the caller binds them before the real run.
std::vector<const char*> g_missing;
void note_missing(const char* name) {
    for (const char* m : g_missing)
        if (!strcmp(m, name)) return;
    g_missing.push_back(name);
}
struct Timed { const char* name; cudaEvent_t a, b; };
std::vector<Timed> g_timed;
struct TimedResult { const char* name; float ms, idle; };
std::vector<TimedResult> g_results;

// ---------------------------------------------------------------------------------------------------------------
// The context of one forward pass: the step, its stream, the bump allocator over its workspace.
// ---------------------------------------------------------------------------------------------------------------
struct Ctx {
    const llmx_step* s;
    cudaStream_t stream;
    bool dry;                 // count the workspace, launch nothing
    size_t used = 0, peak = 0;
    int status = 0;

    Ctx(const llmx_step* step, bool dry_run) : s(step), stream((cudaStream_t)step->stream), dry(dry_run) {}

    void* alloc(size_t bytes) {
        const size_t at = (used + 255) & ~size_t(255);
        used = at + bytes;
        peak = std::max(peak, used);
        if (dry) return nullptr;
        if (used > s->workspace_bytes) {
            if (!status) status = fail(LLMX_RT_ERR_WORKSPACE, "the step's workspace is smaller than llmx_model_workspace says it must be");
            return nullptr;
        }
        return (char*)s->workspace + at;
    }
    template <typename T> T* alloc_n(size_t n) { return (T*)alloc(n * sizeof(T)); }
    const int* meta(int offset) const { return s->meta + offset; }
};

// A failure made on the host, for tests of what a failed step leaves behind: the nth call of one entry point from now
// returns an error without launching anything (the reference's tests fail an operation of their CPU backend the same
// way, tests/tiny_qwen.hpp:104-148).
std::string g_fail_name;
int g_fail_countdown = 0;

// Calls a kernel entry point: counted, timed when profiling is on, skipped on a dry run.
template <typename F, typename... A>
int call(Ctx& c, const char* name, F fn, int launches, A... args) {
    if (c.dry) {
        if (!fn) note_missing(name);
        return 0;
    }
    if (c.status) return c.status;
    if (!fn) return c.status = fail(LLMX_RT_ERR_UNBOUND, std::string("kernel ") + name + " is not bound (its library was not loaded)");
    if (g_fail_countdown > 0 && g_fail_name == name && --g_fail_countdown == 0)
        return c.status = fail(LLMX_RT_ERR_INJECTED, std::string(name) + ": a failure asked for by llmx_rt_fail_call (nothing was launched)");
    Timed t{name, nullptr, nullptr};
    if (g_profile) {
        cudaEventCreate(&t.a);
        cudaEventCreate(&t.b);
        cudaEventRecord(t.a, c.stream);
    }
    const int status = fn(args...);
    if (g_profile) {
        cudaEventRecord(t.b, c.stream);
        g_timed.push_back(t);
    }
    g_launches += launches;
    if (status) {
        char buf[160];
        const char* why = status == 10001 ? "bad argument" : status == 10002 ? "shape or type not supported by this kernel"
                        : status == 10003 ? "TMA descriptor could not be encoded" : status == 10004 ? "size beyond the stated maximum" : nullptr;
        if (why) snprintf(buf, sizeof buf, "%s: %s", name, why);
        else snprintf(buf, sizeof buf, "%s: CUDA error %d (%s)", name, status, cudaGetErrorString((cudaError_t)status));
        c.status = fail(status, buf);
    }
    return status;
}
#define CALL(c, fn, launches, ...) call(c, #fn, kern.fn, launches, __VA_ARGS__)

int g_sms = 0;
int sms() {
    if (!g_sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sms <= 0)
            g_sms = 148;
    }
    return g_sms;
}

inline int cdiv(int a, int b) { return (a + b - 1) / b; }
inline size_t elem(int dtype) { return dtype == LLMX_DT_BF16 ? 2 : 4; }

// ---------------------------------------------------------------------------------------------------------------
// Launch decisions of the tensor-core product.
// ---------------------------------------------------------------------------------------------------------------
constexpr int STREAM_K_MAX_ROWS = 64;         // at most this many tokens: few tiles, so (tile, k block) units are shared out over all blocks
constexpr int STREAM_K_MAX_TILES = 4 * 148;   // ... unless the weight alone makes plenty of tiles (the logits head)
constexpr int HEADS_MIN_ROWS = 256;           // from this many tokens on the q/k/v product finishes its heads itself

int gemm_schedule(int m, int n) { return m <= STREAM_K_MAX_ROWS && cdiv(n, 128) < STREAM_K_MAX_TILES ? 1 : 0; }

// schedule 0: whole tiles, 1: stream-K, 2: on pairs of SMs (there splits 0: only the last, partial round's tiles are cut)
struct GemmPlan { int schedule, token_tile, splits; };
// Which products of many tokens may run on pairs of SMs: a sum of PAIR_PLAIN, PAIR_GATED and PAIR_HEADS.
enum : int { PAIR_PLAIN = 1, PAIR_GATED = 2, PAIR_HEADS = 4, PAIR_ALL = 7 };
int g_pair_products = PAIR_ALL;
constexpr int PAIR_MIN_ROWS = 256;            // gated and q/k/v products: from this many tokens on

// Few tokens: stream-K.  Else whole tiles, and the token tile and the number of k ranges are chosen so that the
// tiles fill the SMs: with a few hundred tokens a [4096, 4096] weight makes 32 to 128 tiles, which would leave most
// of the 148 SMs idle, while two to four k ranges (added with atomics) fill them.  The estimate was fitted to
// timings of the layer's products at 96 to 2,048 tokens: a tile's time is its bytes over what one SM takes in
// (110 GB/s) or its multiply-adds at the SM's share of the tensor rate; atomics run beside the main loop at 500 G a
// second and show at the end of a block's last tile; a stored output that is added to in pieces must be cleared first.
// The same estimate serves the product on pairs of SMs (gemm_tc_pair.cu): a pair's tile is 256 weight rows, each block
// of the pair takes in its 128 weight rows and half the token tile, and the multiply-adds ran a tenth faster there.
GemmPlan gemm_plan_compute(int m, int n, int k, bool accumulate, int n_sms, bool pairs) {
    if (gemm_schedule(m, n) == 1) {
        // 33 to 64 tokens: a piece's write-out is 128 x 64 atomics, and stream-K cuts the tiles into about tiles +
        // blocks pieces.  Whole tiles with K in equal ranges make fewer pieces when they still fill the blocks that
        // run at once (two an SM).
        if (m > 32) {
            const int tiles = cdiv(n, 128), slots = 2 * n_sms;
            int splits = std::min(std::min(slots / std::max(tiles, 1), 8), cdiv(k, 64));
            if (splits >= 2 && tiles * splits * 4 >= slots * 3) return {0, 64, splits};
        }
        return {1, 0, 1};
    }
    if (m <= STREAM_K_MAX_ROWS) return {0, 0, 1};   // few tokens, plenty of weight tiles (the logits head): the narrowest token tile
    const int k_blocks = cdiv(k, 64);
    double best_t = -1;
    GemmPlan best = {0, 128, 1};
    for (int pair = 0; pair <= (pairs && n_sms >= 2 ? 1 : 0); ++pair) {
        const int units = pair ? n_sms / 2 : n_sms;                 // blocks, or pairs of blocks, that run at once
        const int n_tiles = cdiv(n, pair ? 256 : 128);
        for (int bn : {128, 256}) {
            if (bn == 256 && m <= 128) continue;
            const int m_tiles = cdiv(m, bn);
            for (int splits = 1; splits <= 4; ++splits) {
                if (splits > k_blocks) break;
                const long long tiles = (long long)n_tiles * m_tiles * splits;
                const long long waves = (tiles + units - 1) / units;
                const double kk = (double)cdiv(k_blocks, splits) * 64;
                const double per_tile = pair ? std::max(kk * (128 + bn / 2) * 2 / 110e3, 2.0 * 128 * bn * kk / 10.3e6)
                                             : std::max(kk * (128 + bn) * 2 / 110e3, 2.0 * 128 * bn * kk / 9.4e6);
                double t = waves * per_tile;
                if (splits > 1) {
                    t = std::max(t, (double)m * n * splits / 500e3) + std::min(bn, m) * 128 / 8e3;
                    if (!accumulate) t += (double)m * n * 4 / 5e6;
                }
                t *= 1.0 + 0.03 * (splits - 1);
                if (best_t < 0 || t < best_t) best_t = t, best = {pair ? 2 : 0, bn, splits};
            }
            if (pair) {
                // `splits` 0: whole tiles while they fill every pair, then the remaining tiles' K in `r` ranges (the
                // kernel's launcher chooses r the same way), so that the last round is not half empty.
                const long long tiles = (long long)n_tiles * m_tiles;
                const long long at_once = std::min<long long>(units, tiles * 8), left = tiles % at_once;
                long long best_cost = -1;
                int r_best = 1;
                for (int r = 1; left > 0 && r <= 8 && r <= k_blocks; ++r) {
                    const int per = cdiv(k_blocks, r);
                    if ((long long)(r - 1) * per >= k_blocks) continue;
                    const long long cost = (left * r + at_once - 1) / at_once * (r > 1 && per < 26 ? 26 : per);
                    if (best_cost < 0 || cost < best_cost) best_cost = cost, r_best = r;
                }
                if (r_best > 1) {
                    auto tile_time = [&](double kk) {
                        return std::max(kk * (128 + bn / 2) * 2 / 110e3, 2.0 * 128 * bn * kk / 10.3e6);
                    };
                    const long long rounds = (left * r_best + at_once - 1) / at_once;
                    double t = (double)(tiles / at_once) * tile_time(k_blocks * 64.0) + rounds * tile_time(std::max(cdiv(k_blocks, r_best), 26) * 64.0);
                    t += std::min(bn, m) * 128 / 8e3;
                    if (!accumulate) t += (double)m * n * 4 / 5e6;
                    t *= 1.03;
                    if (t < best_t) best_t = t, best = {2, bn, 0};
                }
            }
        }
    }
    return best;
}

GemmPlan gemm_plan(int m, int n, int k, bool accumulate) {
    static std::map<std::tuple<int, int, int, bool, bool>, GemmPlan> cache;
    const bool pairs = g_pair_products & PAIR_PLAIN;
    const auto key = std::make_tuple(m, n, k, accumulate, pairs);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    if (cache.size() > 65536) cache.clear();
    return cache[key] = gemm_plan_compute(m, n, k, accumulate, sms(), pairs);
}

// Weight rows per tile (128: one head, 256: two) of the q/k/v product that finishes its heads in the epilogue, or 0
// when the tokens are few: the plain product then fills the SMs by cutting k, and its float32 output goes through the
// per-head kernel.  Of the two tiles the one whose waves over the SMs take less time (a two-head tile takes about
// 1.55 times a one-head tile).
int heads_tile_compute(int m, int heads, int kv_heads, int n_sms) {
    if (m < HEADS_MIN_ROWS) return 0;
    const long long token_tiles = cdiv(m, 128), width = heads + 2 * kv_heads;
    const long long one = (token_tiles * width + n_sms - 1) / n_sms;
    const long long two = (token_tiles * ((width + 1) / 2) + n_sms - 1) / n_sms;
    return one * 1.0 <= two * 1.55 ? 128 : 256;
}

// ---------------------------------------------------------------------------------------------------------------
// Launch decisions of the attention kernels.
// ---------------------------------------------------------------------------------------------------------------
constexpr int ATTN_PAGE = 16;
constexpr int WAVE_BLOCKS = 148 * 2;      // decode blocks that run at once: two per SM
constexpr double CLUSTER_FILL = 0.92;     // of the clusters that fit at once, as many are planned for
constexpr int PREFILL_PART = 132;         // floats of one (row, head, key range) partial result of the tcgen05 prefill kernel
constexpr long long PREFILL_MAX_PARTIAL = 1ll << 26;

// Clusters of 2..16 decode blocks (head width 128) that a B200 runs at once: what is assumed where the device cannot be asked.
int b200_clusters(int size) {
    switch (size) {
        case 2: return 148; case 3: return 93; case 4: return 71; case 5: return 56; case 6: return 45;
        case 7: return 37; case 8: return 33; case 12: return 21; case 16: return 14; default: return 0;
    }
}

std::map<std::pair<int, int>, int> g_cluster_cache;
int max_clusters(int head_dim, int size) {
    auto& cache = g_cluster_cache;
    auto it = cache.find({head_dim, size});
    if (it != cache.end()) return it->second;
    int n = -1;
    if (kern.llmx_attn_decode_max_clusters) n = kern.llmx_attn_decode_max_clusters(head_dim, size);
    if (n < 0) return b200_clusters(size) * (head_dim == 64 ? 2 : 1);      // no device to ask: plan as for a B200
    return cache[{head_dim, size}] = n;
}

// (key ranges, keys per range) for requests that bring few rows.  Up to sixteen ranges of a (request, kv head) run as
// one thread-block cluster and meet in its shared memory; more would meet through memory and a counter, which costs
// about 4 us more a launch.  A cluster starts only when all its blocks find room in one part of the chip, so no more
// clusters are planned than the device runs at once (with a margin): a second round would double the kernel's time.
// Measured on a B200 (32 heads over 8; 1 to 16 requests, 512 to 32,768 keys): one range per 128 keys below 1,024 keys;
// then as many as fit, eight at most below 4,096 keys, sixteen from there on, twelve where sixteen do not fit only
// from 16,384 keys on.
void decode_schedule(int n_requests, int kv_heads, int max_context, int head_dim, const int* clusters, int* splits_out,
                     int* chunk_out) {
    auto fit = [&](int size) { return clusters ? clusters[size] : max_clusters(head_dim, size); };
    const int blocks = std::max(n_requests * kv_heads, 1);
    const int wave = WAVE_BLOCKS / blocks;
    int want;
    static const int small_sizes[] = {8, 6, 4, 3, 2, 0}, mid_sizes[] = {16, 8, 6, 4, 3, 2, 0}, big_sizes[] = {16, 12, 8, 6, 4, 3, 2, 0};
    const int* sizes;
    if (max_context < 1024) want = std::max(1, max_context / 128), sizes = small_sizes;
    else if (max_context < 4096) want = 8, sizes = small_sizes;
    else if (max_context < 16384) want = 16, sizes = mid_sizes;
    else want = 16, sizes = big_sizes;
    int splits = 1;
    if (fit(2) > 0) {
        for (const int* s = sizes; *s; ++s)
            if (*s <= want && blocks <= CLUSTER_FILL * fit(*s)) { splits = *s; break; }
    } else {                       // clusters turned off: ranges meet through memory, a wave of blocks at most
        splits = std::max(1, std::min(wave, max_context >= 16384 ? want : std::min(want, 8)));
    }
    const int chunk = cdiv(cdiv(max_context, 64), splits) * 64;
    *splits_out = std::max(1, chunk > 0 ? cdiv(max_context, chunk) : 1);
    *chunk_out = std::max(chunk, 64);
}

// (row tiles an item, key ranges) for the tcgen05 prefill kernel.  Its work items are (request, kv head, block of
// rows); a block of threads walks an item's key stages one after the other, so when items are fewer than the SMs the
// longest item is the kernel's time.  Two row tiles an item share their key stages and keep the tensor core busier
// (about 1.05 us a tile and stage of 128 keys against 1.9 us for a tile alone); cutting the keys into ranges makes
// more, shorter items at the price of the partial results' trip through memory and a second small kernel that adds
// the ranges up.  The cheapest combination wins (the estimates below are within a tenth of what was measured at 512
// rows after 4,096 keys, 256 after 8,192, and whole prompts of 1,024 to 8,192 tokens at 16, 32 and 64 heads over 8).
void prefill_shape(int n_requests, int kv_heads, int ratio, int max_rows, int max_context, int window, int n_sms, int* tiles_out,
                   int* splits_out) {
    const int per_tile = std::max(1, 128 / ratio);
    const int reach = window ? std::min(max_context, window + max_rows) : max_context;
    const int stages = cdiv(reach, 128);
    const int hist = std::max(max_context - max_rows, 0);
    double best_t = -1;
    int best_tiles = 2, best_splits = 1;
    const int tile_options[2] = {2, 1};
    const double rates[2] = {2.1, 1.9};           // us a key stage of an item of two tiles / of one
    const double item_cost = 4.0;                 // us an item costs a block beside its stages
    static const int split_options[] = {1, 2, 3, 4, 6, 8};
    for (int o = 0; o < 2; ++o) {
        const int tiles = tile_options[o], rows_per_item = tiles * per_tile;
        const int n_items = cdiv(max_rows, rows_per_item);
        // The items of a request are not equally long: item i's rows see the history and the rows up to its own (or
        // their window).  A block walks heavy and light items in turn, so many items share out evenly.
        long long sum = 0;
        int longest = 0;
        for (int i = 1; i <= n_items; ++i) {
            int keys = hist + std::min(i * rows_per_item, max_rows);
            if (window) keys = std::min(keys, window + rows_per_item);
            const int len = cdiv(keys, 128);
            sum += len;
            longest = std::max(longest, len);
        }
        const double total = (double)sum * kv_heads * n_requests;
        for (int splits : split_options) {
            if (splits > 1 && (stages < 8 * splits ||
                               (long long)max_rows * kv_heads * ratio * n_requests * splits * PREFILL_PART > PREFILL_MAX_PARTIAL))
                break;
            const long long units = (long long)n_items * kv_heads * n_requests * splits;
            const double unit_longest = cdiv(longest, splits);
            const double walk = units <= n_sms ? unit_longest : std::max(unit_longest, total / n_sms + 0.5 * unit_longest);
            // Ranges meet through memory: every (row, head, range) leaves 132 floats that the second kernel reads back
            // (4,096 rows x 32 heads x 2 ranges are 138 MB each way: 244 us with two ranges against 161 with one).
            const double meet = splits > 1 ? 4.0 + 2.0 * (double)max_rows * kv_heads * ratio * n_requests * splits * PREFILL_PART * 4 / 5e6 : 0.0;
            const double t = walk * rates[o] + item_cost * (double)((units + n_sms - 1) / n_sms) + meet;
            if (best_t < 0 || t < best_t - 1e-9) best_t = t, best_tiles = tiles, best_splits = splits;
        }
    }
    *tiles_out = best_tiles;
    *splits_out = best_splits;
}

bool tiled_attention_supported(int heads, int kv_heads, int head_dim, int page_size) {
    return (head_dim == 64 || head_dim == 128) && page_size == ATTN_PAGE && heads % kv_heads == 0 && heads / kv_heads <= 16;
}
bool tensor_core_prefill(int heads, int kv_heads, int head_dim, int page_size) {
    return head_dim == 128 && page_size == ATTN_PAGE && heads % kv_heads == 0 && heads / kv_heads <= 16;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// The cache's entries.
// ---------------------------------------------------------------------------------------------------------------
struct CacheEntry {
    int kind = 0;          // 0 none, 1 keys and values, 2 state
    int group = 0, dtype = 0, kv_heads = 0, page_size = 0, head_dim = 0;
    void* storage = nullptr;
    long long pages = 0, slots = 0, bytes_per_slot = 0;
    alignas(64) mutable unsigned char map[128];         // the decode / warp-level prefill kernels' TMA descriptor
    alignas(64) mutable unsigned char half_map[128];    // the tcgen05 prefill kernel's
    mutable bool have_map = false, have_half_map = false;
};
struct llmx_caches {
    std::vector<CacheEntry> entries;
};

// ---------------------------------------------------------------------------------------------------------------
// Plans.
// ---------------------------------------------------------------------------------------------------------------
struct AttnKey {
    int heads, kv_heads, head_dim, window;
    bool operator==(const AttnKey& o) const { return heads == o.heads && kv_heads == o.kv_heads && head_dim == o.head_dim && window == o.window; }
};
struct AttnPlan {
    AttnKey key;
    int max_rows = 1;                  // a request with at most this many rows runs the split-KV kernel
    std::vector<int> order;            // requests: those with few rows first, then the others
    int n_small = 0, n_large = 0, rows_small = 0, rows_large = 0;
    int ctx_small = 0, ctx_large = 0;
    int splits = 1, chunk = 64;        // key ranges of the split-KV kernel
    bool chunk_on_device = false;      // a recorded step: the keys per range are read from the plan's ints
    int tiles = 2, psplits = 1;        // item shape of the tcgen05 prefill kernel
    int offset = 0;                    // of this entry's ints within the plan's ints
};
struct llmx_plan {
    std::vector<AttnPlan> attn;
    std::vector<int> counts;
    int requests = 0, room = 0, typical_context = 0, ints = 0;
    int force_tiles = 0, force_splits = 0;
    const AttnPlan* find(const AttnKey& k) const {
        for (const AttnPlan& a : attn)
            if (a.key == k) return &a;
        return nullptr;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// Parts.
// ---------------------------------------------------------------------------------------------------------------
enum PartKind { PART_NORM, PART_MIXER, PART_FFN, PART_BLOCK, PART_EMBEDDING, PART_HEAD, PART_LINEAR };

struct llmx_part {
    PartKind kind;
    explicit llmx_part(PartKind k) : kind(k) {}
    virtual ~llmx_part() {}
    // The attention shapes below this part that want a launch plan.
    virtual void collect(std::vector<AttnKey>&) const {}
};

namespace {

struct Linear : llmx_part {
    const void* w;
    int dtype, N, K, flags;
    bool tensor_core;
    alignas(64) unsigned char map128[128];
    alignas(64) unsigned char head_map[2][128];
    bool have_map = false, have_head_map[2] = {false, false};

    explicit Linear(const llmx_linear_desc& d)
        : llmx_part(PART_LINEAR), w(d.weight), dtype(d.dtype), N(d.out_features), K(d.in_features), flags(d.flags) {
        tensor_core = dtype == LLMX_DT_BF16 && K % 8 == 0;
    }
    bool invariant() const { return flags & LLMX_FLAG_INVARIANT; }

    // Whether the product for this many rows adds its pieces into the output with atomics, which then must start
    // from zeros when the product is to be stored.
    bool adds_pieces(int rows) const {
        if (!tensor_core || invariant()) return false;
        const GemmPlan p = gemm_plan(rows, N, K, false);
        return p.schedule == 1 || p.splits != 1;
    }
    long long output_to_clear(int rows) const {
        if (!adds_pieces(rows) || ((long long)rows * N) % 4) return 0;
        return (long long)rows * N;
    }
    int ensure_map(Ctx& c) {
        if (have_map) return 0;
        if (c.dry) {
            if (!kern.llmx_gemm_tc_weight_map) note_missing("llmx_gemm_tc_weight_map");
            return 0;
        }
        if (!kern.llmx_gemm_tc_weight_map) return c.status = fail(LLMX_RT_ERR_UNBOUND, "kernel llmx_gemm_tc_weight_map is not bound");
        const int e = kern.llmx_gemm_tc_weight_map(map128, w, N, K);
        if (e) return c.status = fail(e, "gemm_tc weight map could not be made");
        have_map = true;
        return 0;
    }

    // out (+)= a W^T; a [rows, K] of the weight's type, out float32 [rows, N].  `cleared`: out already holds zeros.
    int forward(Ctx& c, const void* a, int rows, float* out, bool accumulate, bool cleared) {
        if (rows <= 0) return 0;
        if (!tensor_core) return CALL(c, llmx_gemm_plain, 1, a, dtype, w, dtype, out, rows, N, K, accumulate ? 1 : 0, c.stream);
        if (ensure_map(c)) return c.status;
        if (invariant())       // one schedule whatever the rows: whole tiles of 128 tokens, k in one piece
            return CALL(c, llmx_gemm_tc, 1, (const void*)map128, a, out, rows, N, K, accumulate ? 1 : 0, 1, 128, 0, c.s->error_word, c.stream);
        bool acc = accumulate || (cleared && adds_pieces(rows));
        const GemmPlan p = gemm_plan(rows, N, K, acc);
        if ((p.schedule == 1 || p.splits != 1) && !acc) {
            if (!c.dry && !c.status && cudaMemsetAsync(out, 0, (size_t)rows * N * sizeof(float), c.stream) != cudaSuccess)
                return c.status = fail(LLMX_RT_ERR_BAD_ARGUMENT, "clearing a product's output failed");
            acc = true;
        }
        if (p.schedule == 2)
            return CALL(c, llmx_gemm_tc_pair, 1, (const void*)map128, a, out, rows, N, K, acc ? 1 : 0, p.splits, p.token_tile,
                        c.s->error_word, c.stream);
        return CALL(c, llmx_gemm_tc, 1, (const void*)map128, a, out, rows, N, K, acc ? 1 : 0, p.splits, p.token_tile, p.schedule,
                    c.s->error_word, c.stream);
    }
    // Whether the gated form (both halves of a stacked gate/up weight in one kernel, silu(g) u written as bfloat16)
    // runs for this many rows: with few rows the product is spread over the SMs by k ranges, whose partial sums cannot
    // pass through the activation.
    bool fused_gate(int rows) const { return tensor_core && (invariant() || rows > STREAM_K_MAX_ROWS); }
    int gated(Ctx& c, const void* a, int rows, void* out) {
        if (ensure_map(c)) return c.status;
        if (!invariant() && (g_pair_products & PAIR_GATED) && rows >= PAIR_MIN_ROWS)
            return CALL(c, llmx_gemm_tc_pair_swiglu, 1, (const void*)map128, a, out, rows, N / 2, K, c.s->error_word, c.stream);
        return CALL(c, llmx_gemm_tc_swiglu, 1, (const void*)map128, a, out, rows, N / 2, K, invariant() ? 128 : 0, c.s->error_word, c.stream);
    }
    int ensure_head_map(Ctx& c, int tile) {
        const int i = tile == 256;
        if (have_head_map[i]) return 0;
        if (c.dry) {
            if (!kern.llmx_gemm_tc_weight_map_box) note_missing("llmx_gemm_tc_weight_map_box");
            return 0;
        }
        if (!kern.llmx_gemm_tc_weight_map_box) return c.status = fail(LLMX_RT_ERR_UNBOUND, "kernel llmx_gemm_tc_weight_map_box is not bound");
        const int e = kern.llmx_gemm_tc_weight_map_box(head_map[i], w, N, K, tile);
        if (e) return c.status = fail(e, "gemm_tc weight map could not be made");
        have_head_map[i] = true;
        return 0;
    }
};

struct Norm : llmx_part {
    const float* weight;
    int width, out_dtype;
    float eps;
    Norm(const float* w, int n, float e, int dt) : llmx_part(PART_NORM), weight(w), width(n), out_dtype(dt), eps(e) {}
    int forward(Ctx& c, const float* x, void* out, int dtype, const int* row_index, int rows, float* zero, long long zero_count) {
        return CALL(c, llmx_rmsnorm, 1, x, weight, out, dtype, row_index, rows, width, eps, zero, zero_count, c.stream);
    }
};

struct Mixer : llmx_part {
    int hidden;
    Mixer(int h) : llmx_part(PART_MIXER), hidden(h) {}
    virtual long long wants_cleared(Ctx&, int) { return 0; }
    virtual int act_dtype() const = 0;
    virtual int forward(Ctx&, const void* h, int rows, int cache_entry, float* residual, bool write_cache, float* cleared) = 0;
};
struct FeedForward : llmx_part {
    int hidden;
    FeedForward(int h) : llmx_part(PART_FFN), hidden(h) {}
    virtual long long wants_cleared(Ctx&, int) { return 0; }
    virtual int forward(Ctx&, const void* h, int rows, float* residual, float* cleared) = 0;
};
struct Block : llmx_part {
    Block() : llmx_part(PART_BLOCK) {}
    virtual int forward(Ctx&, float* x, int rows, int cache_entry, bool write_cache) = 0;
};

// ---- attention ------------------------------------------------------------------------------------------------
// For the rows of a step (src/model/arch/qwen3.hpp:272-295):
//     q, k, v = h Wq^T, h Wk^T, h Wv^T            (one product over the stacked weight)
//     q, k    = RMSNorm per head (optional), then rotated by position (optional)
//     k, v   -> the row's cache slot
//     o       = softmax(q K^T scale) V over the request's keys lo..p, causal; query head h reads kv head h / (H / G)
//     residual += o Wo^T
struct Attention : Mixer {
    llmx_attention_desc d;
    Linear qkv, o;
    int q_width, kv_width;

    explicit Attention(const llmx_attention_desc& desc) : Mixer(desc.hidden), d(desc), qkv(desc.qkv), o(desc.o) {
        q_width = d.heads * d.head_dim;
        kv_width = d.kv_heads * d.head_dim;
    }
    int act_dtype() const override { return qkv.dtype; }
    bool invariant() const { return d.flags & LLMX_FLAG_INVARIANT; }
    AttnKey key() const { return {d.heads, d.kv_heads, d.head_dim, d.window}; }
    void collect(std::vector<AttnKey>& out) const override {
        if (qkv.dtype != LLMX_DT_BF16 || invariant() || !tiled_attention_supported(d.heads, d.kv_heads, d.head_dim, ATTN_PAGE)) return;
        const AttnKey k = key();
        if (std::find(out.begin(), out.end(), k) == out.end()) out.push_back(k);
    }
    // The tiled bfloat16 kernels serve this entry: bfloat16 queries and cache, a head width and page size they take.
    bool tiled(const CacheEntry& e) const {
        return qkv.dtype == LLMX_DT_BF16 && e.dtype == LLMX_DT_BF16 && !invariant() &&
               tiled_attention_supported(d.heads, d.kv_heads, d.head_dim, e.page_size);
    }
    // Weight rows per tile when the q/k/v product can finish its heads itself for this many rows, else 0.
    int heads_tile(int rows) const {
        if (!qkv.tensor_core || invariant() || d.head_dim != 128 || (d.cos && d.rot_half != 64)) return 0;
        return heads_tile_compute(rows, d.heads, d.kv_heads, sms());
    }
    const AttnPlan* plan_of(Ctx& c) const { return c.s->plan ? c.s->plan->find(key()) : nullptr; }

    long long wants_cleared(Ctx& c, int rows) override {
        if (heads_tile(rows)) {
            const AttnPlan* p = plan_of(c);
            if (!(p && p->n_small > 0 && p->n_large == 0)) return 0;   // the product finishes its heads itself: no float32 output to clear
        }
        return qkv.output_to_clear(rows);
    }

    int ensure_maps(Ctx& c, const CacheEntry& e, bool half) {
        if (c.dry) {
            if (!half && !kern.llmx_attn_cache_map) note_missing("llmx_attn_cache_map");
            if (half && !kern.llmx_attn_prefill_tc_cache_map) note_missing("llmx_attn_prefill_tc_cache_map");
            return 0;
        }
        if (!half && !e.have_map) {
            if (!kern.llmx_attn_cache_map) return c.status = fail(LLMX_RT_ERR_UNBOUND, "kernel llmx_attn_cache_map is not bound");
            if (int err = kern.llmx_attn_cache_map(e.map, e.storage, e.pages, e.kv_heads, e.page_size, e.head_dim))
                return c.status = fail(err, "attention cache map could not be made");
            e.have_map = true;
        }
        if (half && !e.have_half_map) {
            if (!kern.llmx_attn_prefill_tc_cache_map) return c.status = fail(LLMX_RT_ERR_UNBOUND, "kernel llmx_attn_prefill_tc_cache_map is not bound");
            if (int err = kern.llmx_attn_prefill_tc_cache_map(e.half_map, e.storage, e.pages, e.kv_heads, e.page_size, e.head_dim))
                return c.status = fail(err, "attention cache map could not be made");
            e.have_half_map = true;
        }
        return 0;
    }

    // Which attention kernel runs for which rows: requests that bring one or a few rows run the split-KV decode
    // kernel, requests that bring a portion of a prompt the tiled prefill kernel (tcgen05 where the head width is
    // 128, else warp-level); both read the same pages.  Anything the tiled kernels do not take runs the plain
    // kernel (one block per row and head).
    int attend(Ctx& c, const void* q, const CacheEntry& e, void* out, int rows, int group) {
        const llmx_step& s = *c.s;
        const int* tables = c.meta(s.block_tables[group]);
        if (!tiled(e))
            return CALL(c, llmx_attention_plain, 1, q, qkv.dtype, (const void*)e.storage, e.dtype, out, c.meta(s.row_request),
                        c.meta(s.positions) + (size_t)d.position_stream * s.rows, tables, s.table_stride[group], rows, d.heads,
                        d.kv_heads, d.head_dim, e.page_size, d.window, d.scale, c.stream);
        const AttnPlan* p = plan_of(c);
        if (!p) return c.status = fail(LLMX_RT_ERR_BAD_ARGUMENT, "attention: the step carries no launch plan for this mixer (llmx_plan_make)");
        const int* list = c.meta(s.plan_offset + p->offset);
        if (p->n_small) {
            if (ensure_maps(c, e, false)) return c.status;
            float* partial = p->splits > 1 ? c.alloc_n<float>((size_t)rows * d.heads * p->splits * (d.head_dim + 2)) : nullptr;
            const bool counted = p->splits > 1 && p->n_small * d.kv_heads <= LLMX_COUNTERS && s.counters;
            CALL(c, llmx_attn_decode_fused, (p->splits > 1 && !counted ? 2 : 1), (const void*)e.map, q, out, partial, list, p->n_small,
                 c.meta(s.row_start), c.meta(s.row_count), c.meta(s.history), tables, s.table_stride[group], d.heads, d.kv_heads,
                 d.head_dim, e.page_size, d.window, d.scale, p->splits, p->chunk_on_device ? list + p->order.size() : nullptr,
                 p->chunk_on_device ? 64 : p->chunk, std::max(p->rows_small, 1), counted ? s.counters : nullptr, s.error_word, c.stream);
        }
        if (p->n_large && tensor_core_prefill(d.heads, d.kv_heads, d.head_dim, e.page_size)) {
            if (ensure_maps(c, e, true)) return c.status;
            float* partial = p->psplits > 1 ? c.alloc_n<float>((size_t)rows * d.heads * p->psplits * PREFILL_PART) : nullptr;
            CALL(c, llmx_attn_prefill_tc, p->psplits > 1 ? 2 : 1, (const void*)e.half_map, q, out, rows, list + p->n_small, p->n_large,
                 c.meta(s.row_start), c.meta(s.row_count), c.meta(s.history), tables, s.table_stride[group], d.heads, d.kv_heads,
                 d.head_dim, e.page_size, d.window, d.scale, p->rows_large, p->tiles, p->psplits, partial, s.error_word, c.stream);
        } else if (p->n_large) {
            if (ensure_maps(c, e, false)) return c.status;
            CALL(c, llmx_attn_prefill, 1, (const void*)e.map, q, out, list + p->n_small, p->n_large, c.meta(s.row_start),
                 c.meta(s.row_count), c.meta(s.history), tables, s.table_stride[group], d.heads, d.kv_heads, d.head_dim, e.page_size,
                 d.window, d.scale, p->rows_large, s.error_word, c.stream);
        }
        return c.status;
    }

    int forward(Ctx& c, const void* h, int rows, int cache_entry, float* residual, bool write_cache, float* cleared) override {
        const llmx_step& s = *c.s;
        if (!s.caches || cache_entry < 0 || cache_entry >= (int)s.caches->entries.size() || s.caches->entries[cache_entry].kind != 1)
            return c.status = fail(LLMX_RT_ERR_BAD_ARGUMENT, "attention: the cache entry is not one of keys and values");
        const CacheEntry& e = s.caches->entries[cache_entry];
        if (e.kv_heads != d.kv_heads || e.head_dim != d.head_dim)
            return c.status = fail(LLMX_RT_ERR_BAD_ARGUMENT, "attention: the cache entry's geometry is not this mixer's");
        if (d.position_stream < 0 || d.position_stream >= std::max(s.position_streams, 1))
            return c.status = fail(LLMX_RT_ERR_BAD_ARGUMENT, "attention: the step has no such position stream");
        const int g = e.group;
        const int act = qkv.dtype;
        const int* positions = c.meta(s.positions) + (size_t)d.position_stream * s.rows;
        const int* slots = c.meta(s.slots[g]);
        if (!write_cache) {        // a layer that reads another layer's cache computes its queries only
            int* none = c.alloc_n<int>(rows);
            if (!c.dry && !c.status) cudaMemsetAsync(none, 0xFF, (size_t)rows * sizeof(int), c.stream);
            slots = none;
        }
        void* o_buf = c.alloc((size_t)rows * q_width * elem(act));
        const AttnPlan* p = plan_of(c);
        const bool decoding_only = p && p->n_small > 0 && p->n_large == 0;
        const int tile = heads_tile(rows);
        if (tile && e.dtype == LLMX_DT_BF16 && e.page_size > 0 && !decoding_only) {
            // Many rows: the product norms, rotates and stores its heads in its own epilogue.
            void* q = c.alloc((size_t)rows * q_width * 2);
            if ((g_pair_products & PAIR_HEADS) && rows >= PAIR_MIN_ROWS) {
                if (qkv.ensure_map(c)) return c.status;
                CALL(c, llmx_gemm_tc_pair_heads, 1, (const void*)qkv.map128, h, rows, qkv.K, d.q_norm, d.k_norm, d.qk_norm_eps, d.cos, d.sin,
                     positions, slots, q, (void*)e.storage, d.heads, d.kv_heads, e.page_size, s.error_word, c.stream);
                attend(c, q, e, o_buf, rows, g);
                return o.forward(c, o_buf, rows, residual, true, false);
            }
            if (qkv.ensure_head_map(c, tile)) return c.status;
            CALL(c, llmx_gemm_tc_heads, 1, (const void*)qkv.head_map[tile == 256], h, rows, qkv.K, tile, d.q_norm, d.k_norm, d.qk_norm_eps,
                 d.cos, d.sin, positions, slots, q, (void*)e.storage, d.heads, d.kv_heads, e.page_size, s.error_word, c.stream);
            attend(c, q, e, o_buf, rows, g);
            return o.forward(c, o_buf, rows, residual, true, false);
        }
        float* qkv_out = cleared;
        if (!qkv_out) qkv_out = c.alloc_n<float>((size_t)rows * qkv.N);
        qkv.forward(c, h, rows, qkv_out, false, cleared != nullptr);
        if (!from_qkv(c, qkv_out, e, o_buf, rows, slots, g)) {
            if (c.status) return c.status;
            void* q = c.alloc((size_t)rows * q_width * elem(act));
            CALL(c, llmx_head_norm_rope_kv, 1, (const float*)qkv_out, qkv.N, q_width, q_width + kv_width, d.q_norm, d.k_norm,
                 d.qk_norm_eps, d.cos, d.sin, d.cos ? d.rot_half : 0, positions, slots, q, act, (void*)e.storage, e.dtype, rows, d.heads,
                 d.kv_heads, d.head_dim, e.page_size, c.stream);
            attend(c, q, e, o_buf, rows, g);
        }
        return o.forward(c, o_buf, rows, residual, true, false);
    }

    // A step of decoding rows only: the attention kernel norms and rotates its own queries, and the block whose key
    // range holds a new row stores that key and value (head width 128, rotated whole or not at all).  False, having
    // done nothing, when the step or the shapes do not qualify.
    bool from_qkv(Ctx& c, const float* qkv_out, const CacheEntry& e, void* o_buf, int rows, const int* slots, int g) {
        const llmx_step& s = *c.s;
        const AttnPlan* p = plan_of(c);
        const bool decoding_only = p && p->n_small > 0 && p->n_large == 0;
        if (!(decoding_only && tiled(e) && d.head_dim == 128 && (!d.cos || d.rot_half == 64) &&
              p->n_small * d.kv_heads <= LLMX_COUNTERS && s.counters))
            return false;
        if (ensure_maps(c, e, false)) return false;
        const int* list = c.meta(s.plan_offset + p->offset);
        float* partial = p->splits > 1 ? c.alloc_n<float>((size_t)rows * d.heads * p->splits * (d.head_dim + 2)) : nullptr;
        CALL(c, llmx_attn_decode_qkv, 1, (const void*)e.map, qkv_out, qkv.N, q_width, q_width + kv_width, d.q_norm,
             d.k_norm, d.qk_norm_eps, d.cos, d.sin, slots, (void*)e.storage, o_buf, partial, list, p->n_small, c.meta(s.row_start),
             c.meta(s.row_count), c.meta(s.history), c.meta(s.block_tables[g]), s.table_stride[g], d.heads, d.kv_heads,
             d.head_dim, e.page_size, d.window, d.scale, p->splits, p->chunk_on_device ? list + p->order.size() : nullptr,
             p->chunk_on_device ? 64 : p->chunk, std::max(p->rows_small, 1), s.counters, s.error_word, c.stream);
        return true;
    }
};

// ---- gated feed-forward ---------------------------------------------------------------------------------------
// residual += (silu(h Wg^T) * (h Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g)) in 32-bit (src/model/arch/blocks.hpp:101-106).
struct GatedMlp : FeedForward {
    llmx_mlp_desc d;
    Linear gate_up, down;
    explicit GatedMlp(const llmx_mlp_desc& desc) : FeedForward(desc.hidden), d(desc), gate_up(desc.gate_up), down(desc.down) {}
    long long wants_cleared(Ctx&, int rows) override { return gate_up.fused_gate(rows) ? 0 : gate_up.output_to_clear(rows); }
    int forward(Ctx& c, const void* h, int rows, float* residual, float* cleared) override {
        const int act = gate_up.dtype;
        void* a = c.alloc((size_t)rows * d.intermediate * elem(act));
        if (gate_up.fused_gate(rows)) {
            gate_up.gated(c, h, rows, a);
        } else {
            float* gu = cleared ? cleared : c.alloc_n<float>((size_t)rows * 2 * d.intermediate);
            gate_up.forward(c, h, rows, gu, false, cleared != nullptr);
            CALL(c, llmx_swiglu, 1, (const float*)gu, a, act, rows, d.intermediate, c.stream);
        }
        return down.forward(c, a, rows, residual, true, false);
    }
};

// ---- parts written elsewhere ----------------------------------------------------------------------------------
struct CallbackMixer : Mixer {
    llmx_callback fn; void* user;
    CallbackMixer(llmx_callback f, void* u, int hidden) : Mixer(hidden), fn(f), user(u) {}
    int act_dtype() const override { return -1; }
    int forward(Ctx& c, const void* h, int rows, int cache_entry, float* residual, bool write_cache, float*) override {
        if (c.dry || c.status) return c.status;
        const int e = fn(user, c.s, 1, const_cast<void*>(h), residual, rows, cache_entry, write_cache);
        return e ? (c.status = fail(LLMX_RT_ERR_CALLBACK, "a mixer's callback failed")) : 0;
    }
};
struct CallbackFfn : FeedForward {
    llmx_callback fn; void* user;
    CallbackFfn(llmx_callback f, void* u, int hidden) : FeedForward(hidden), fn(f), user(u) {}
    int forward(Ctx& c, const void* h, int rows, float* residual, float*) override {
        if (c.dry || c.status) return c.status;
        const int e = fn(user, c.s, 2, const_cast<void*>(h), residual, rows, -1, 0);
        return e ? (c.status = fail(LLMX_RT_ERR_CALLBACK, "a feed-forward's callback failed")) : 0;
    }
};
struct CallbackBlock : Block {
    llmx_callback fn; void* user;
    CallbackBlock(llmx_callback f, void* u) : fn(f), user(u) {}
    int forward(Ctx& c, float* x, int rows, int cache_entry, bool write_cache) override {
        if (c.dry || c.status) return c.status;
        const int e = fn(user, c.s, 0, nullptr, x, rows, cache_entry, write_cache);
        return e ? (c.status = fail(LLMX_RT_ERR_CALLBACK, "a block's callback failed")) : 0;
    }
};

// ---- x += mixer(norm(x)); x += ffn(norm(x)) ---------------------------------------------------------------------
struct PreNormBlock : Block {
    Norm *norm1, *norm2;
    Mixer* mixer;
    FeedForward* ffn;
    PreNormBlock(Norm* n1, Mixer* m, Norm* n2, FeedForward* f) : norm1(n1), norm2(n2), mixer(m), ffn(f) {}
    void collect(std::vector<AttnKey>& out) const override { mixer->collect(out); ffn->collect(out); }
    int forward(Ctx& c, float* x, int rows, int cache_entry, bool write_cache) override {
        const size_t mark = c.used;
        // A part may ask for a buffer to be zeroed before it runs; the norm in front of it does that in passing.
        long long n = mixer->wants_cleared(c, rows);
        float* cleared = n ? c.alloc_n<float>((size_t)n) : nullptr;
        void* h = c.alloc((size_t)rows * norm1->width * elem(norm1->out_dtype));
        norm1->forward(c, x, h, norm1->out_dtype, nullptr, rows, cleared, n);
        mixer->forward(c, h, rows, cache_entry, x, write_cache, cleared);
        c.used = mark;
        n = ffn->wants_cleared(c, rows);
        cleared = n ? c.alloc_n<float>((size_t)n) : nullptr;
        h = c.alloc((size_t)rows * norm2->width * elem(norm2->out_dtype));
        norm2->forward(c, x, h, norm2->out_dtype, nullptr, rows, cleared, n);
        ffn->forward(c, h, rows, x, cleared);
        c.used = mark;
        return c.status;
    }
};

struct Embedding : llmx_part {
    const void* table; int dtype, vocab, width;
    Embedding(const void* t, int dt, int v, int w) : llmx_part(PART_EMBEDDING), table(t), dtype(dt), vocab(v), width(w) {}
    int forward(Ctx& c, const int* ids, float* x, int rows) {
        return CALL(c, llmx_embed, 1, table, dtype, ids, x, rows, width, vocab, c.stream);
    }
};

// Logits for the rows that want them: gather, norm, product (src/model/arch/blocks.hpp:267-272).
struct Head : llmx_part {
    Norm* norm;
    Linear linear;
    Head(Norm* n, const llmx_linear_desc& w) : llmx_part(PART_HEAD), norm(n), linear(w) {}
    int forward(Ctx& c, const float* x, float* logits) {
        const int wanted = c.s->wanted;
        if (wanted <= 0) return 0;
        const size_t mark = c.used;
        void* h = c.alloc((size_t)wanted * norm->width * elem(linear.dtype));
        norm->forward(c, x, h, linear.dtype, c.meta(c.s->logit_rows), wanted, nullptr, 0);
        linear.forward(c, h, wanted, logits, false, false);
        c.used = mark;
        return c.status;
    }
};

template <typename T> T* as(llmx_part* p, PartKind kind) { return p && p->kind == kind ? static_cast<T*>(p) : nullptr; }

}  // namespace

struct llmx_model {
    Embedding* embedding;
    std::vector<Block*> blocks;
    std::vector<llmx_layer_step> order;
    Head* head;
    int hidden, vocab;

    int forward(Ctx& c, float* logits) {
        const int rows = c.s->rows;
        float* x = c.alloc_n<float>((size_t)rows * hidden);
        embedding->forward(c, c.meta(c.s->token_ids), x, rows);
        for (const llmx_layer_step& st : order) {
            blocks[st.block]->forward(c, x, rows, st.cache_entry, st.write_cache != 0);
            if (c.status) return c.status;
        }
        head->forward(c, x, logits);
        return c.status;
    }
};

// ===============================================================================================================
// The C interface.
// ===============================================================================================================
LLMX_API int llmx_rt_version(void) { return LLMX_RT_VERSION; }
LLMX_API const char* llmx_rt_last_error(void) { return g_error.c_str(); }
LLMX_API long long llmx_rt_launches(void) { return g_launches; }
LLMX_API void llmx_rt_count_launches(long long n) { g_launches += n; }

LLMX_API int llmx_rt_bind(const char* name, void* function) {
    if (!name || !function) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_rt_bind: a name and a function");
    if (!bind(name, function)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, std::string("llmx_rt_bind: the runtime calls no kernel named ") + name);
    return 0;
}

// A bound entry point by name, for the engine's own calls (the sampler's kernels); null when it is not bound, and the
// name is then noted as missing like a dry run's.
LLMX_API void* llmx_rt_kernel(const char* name) {
#define X(kname, args)                                                  \
    if (!strcmp(name, #kname)) {                                        \
        if (!kern.kname) note_missing(#kname);                          \
        return reinterpret_cast<void*>(kern.kname);                     \
    }
    LLMX_KERNELS(X)
#undef X
    return nullptr;
}

LLMX_API int llmx_rt_load_kernels(const char* folder) {
    DIR* dir = folder ? opendir(folder) : nullptr;
    if (!dir) return -fail(LLMX_RT_ERR_BAD_ARGUMENT, std::string("llmx_rt_load_kernels: cannot read ") + (folder ? folder : "(null)"));
    int bound = 0;
    while (dirent* ent = readdir(dir)) {
        const std::string name = ent->d_name;
        if (name.rfind("llmx_", 0) != 0 || name.size() < 4 || name.compare(name.size() - 3, 3, ".so") || name.rfind("llmx_runtime", 0) == 0)
            continue;
        void* lib = dlopen((std::string(folder) + "/" + name).c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!lib) continue;
#define X(kname, args)                                          \
        if (void* f = dlsym(lib, #kname)) {                     \
            kern.kname = reinterpret_cast<int(*) args>(f);      \
            ++bound;                                            \
        }
        LLMX_KERNELS(X)
#undef X
    }
    closedir(dir);
    return bound;
}

LLMX_API void llmx_rt_fail_call(const char* name, int nth) {
    g_fail_name = name ? name : "";
    g_fail_countdown = name && nth > 0 ? nth : 0;
}
LLMX_API int llmx_rt_missing(int i, const char** name) {
    if (i < 0 || i >= (int)g_missing.size()) return 0;
    *name = g_missing[i];
    return 1;
}
// What the runtime remembers about the device and the kernel libraries (the clusters that fit, chosen schedules).
LLMX_API void llmx_rt_reset_caches(void) {
    g_missing.clear();
    g_cluster_cache.clear();
}

LLMX_API int llmx_rt_pair_products(int on) {
    const int before = g_pair_products;
    g_pair_products = on & PAIR_ALL;
    return before;
}

LLMX_API int llmx_rt_profile(int on) {
    const bool before = g_profile;
    if (on && !g_profile) {
        g_timed.clear();
        g_results.clear();
    }
    if (!on && g_profile) {
        cudaDeviceSynchronize();
        g_results.clear();
        for (size_t i = 0; i < g_timed.size(); ++i) {
            TimedResult r{g_timed[i].name, 0.f, 0.f};
            cudaEventElapsedTime(&r.ms, g_timed[i].a, g_timed[i].b);
            if (i) {
                cudaEventElapsedTime(&r.idle, g_timed[i - 1].b, g_timed[i].a);
                r.idle = std::max(r.idle, 0.f);
            }
            g_results.push_back(r);
        }
        for (Timed& t : g_timed) {
            cudaEventDestroy(t.a);
            cudaEventDestroy(t.b);
        }
        g_timed.clear();
    }
    g_profile = on != 0;
    return before;
}
LLMX_API int llmx_rt_profile_read(int i, const char** name, float* ms, float* idle) {
    if (i < 0 || i >= (int)g_results.size()) return 0;
    *name = g_results[i].name;
    *ms = g_results[i].ms;
    *idle = g_results[i].idle;
    return 1;
}

LLMX_API void llmx_gemm_plan(int m, int n, int k, int accumulate, int n_sms, int* schedule, int* token_tile, int* splits) {
    const GemmPlan p = n_sms > 0 ? gemm_plan_compute(m, n, k, accumulate != 0, n_sms, g_pair_products & PAIR_PLAIN) : gemm_plan(m, n, k, accumulate != 0);
    *schedule = p.schedule, *token_tile = p.token_tile, *splits = p.splits;
}
LLMX_API int llmx_tiled_attention(int heads, int kv_heads, int head_dim, int page_size) {
    if (kv_heads <= 0 || heads <= 0 || !tiled_attention_supported(heads, kv_heads, head_dim, page_size)) return 0;
    return tensor_core_prefill(heads, kv_heads, head_dim, page_size) ? 2 : 1;
}
LLMX_API int llmx_heads_tile(int m, int heads, int kv_heads, int n_sms) { return heads_tile_compute(m, heads, kv_heads, n_sms > 0 ? n_sms : sms()); }
LLMX_API void llmx_decode_schedule(int n_requests, int kv_heads, int max_context, int head_dim, const int* clusters, int* splits, int* chunk) {
    decode_schedule(n_requests, kv_heads, max_context, head_dim, clusters, splits, chunk);
}
LLMX_API void llmx_prefill_shape(int n_requests, int kv_heads, int ratio, int max_rows, int max_context, int window, int n_sms, int* tiles,
                                 int* splits) {
    prefill_shape(n_requests, kv_heads, ratio, max_rows, max_context, window, n_sms > 0 ? n_sms : 148, tiles, splits);
}

// ---- caches ----
LLMX_API llmx_caches* llmx_caches_create(int entries) {
    if (entries < 0) return nullptr;
    llmx_caches* c = new llmx_caches;
    c->entries.resize(entries);
    return c;
}
LLMX_API void llmx_caches_destroy(llmx_caches* c) { delete c; }
LLMX_API int llmx_caches_set_kv(llmx_caches* c, int entry, int group, void* storage, int dtype, long long pages, int kv_heads, int page_size,
                                int head_dim) {
    if (!c || entry < 0 || entry >= (int)c->entries.size() || group < 0 || group >= LLMX_MAX_GROUPS || !storage || pages < 0 ||
        kv_heads <= 0 || page_size <= 0 || head_dim <= 0 || (dtype != LLMX_DT_F32 && dtype != LLMX_DT_BF16))
        return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_caches_set_kv: bad entry, group, storage or geometry");
    CacheEntry& e = c->entries[entry];
    e = CacheEntry();
    e.kind = 1, e.group = group, e.storage = storage, e.dtype = dtype, e.pages = pages, e.kv_heads = kv_heads, e.page_size = page_size,
    e.head_dim = head_dim;
    return 0;
}
LLMX_API int llmx_caches_set_state(llmx_caches* c, int entry, void* storage, long long slots, long long bytes_per_slot) {
    if (!c || entry < 0 || entry >= (int)c->entries.size() || !storage || slots < 0 || bytes_per_slot < 0)
        return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_caches_set_state: bad entry or storage");
    CacheEntry& e = c->entries[entry];
    e = CacheEntry();
    e.kind = 2, e.storage = storage, e.slots = slots, e.bytes_per_slot = bytes_per_slot;
    return 0;
}

// ---- plans ----
namespace {
void plan_attention(llmx_plan& plan, AttnPlan& a, const int* histories) {
    const int n = plan.requests;
    const int ratio = a.key.heads / a.key.kv_heads;
    a.max_rows = std::max(16 / ratio, 1);
    a.order.clear();
    a.n_small = a.n_large = a.rows_small = a.rows_large = a.ctx_small = a.ctx_large = 0;
    for (int r = 0; r < n; ++r)
        if (plan.counts[r] <= a.max_rows) a.order.push_back(r);
    a.n_small = (int)a.order.size();
    for (int r = 0; r < n; ++r)
        if (plan.counts[r] > a.max_rows) a.order.push_back(r);
    a.n_large = n - a.n_small;
    for (int r = 0; r < n; ++r) {
        const int c = plan.counts[r];
        const int ctx = plan.room > 0 ? plan.room : (histories ? histories[r] : 0) + c;
        // What a recorded step's grids must cover is its room; what its prompt portions are likely to meet (a matter
        // of speed only: the prefill kernels take any history under any item shape) is the context it was made at.
        const int likely = plan.room > 0 && plan.typical_context > 0 ? std::max(std::min(plan.typical_context, plan.room), c) : ctx;
        if (c <= a.max_rows) a.rows_small = std::max(a.rows_small, c), a.ctx_small = std::max(a.ctx_small, ctx);
        else a.rows_large = std::max(a.rows_large, c), a.ctx_large = std::max(a.ctx_large, likely);
    }
    a.chunk_on_device = plan.room > 0;
    if (a.n_small) decode_schedule(a.n_small, a.key.kv_heads, a.ctx_small, a.key.head_dim, nullptr, &a.splits, &a.chunk);
    if (a.n_large) {
        prefill_shape(a.n_large, a.key.kv_heads, ratio, a.rows_large, a.ctx_large, a.key.window, sms(), &a.tiles, &a.psplits);
        if (plan.force_tiles) a.tiles = plan.force_tiles;
        if (plan.force_splits) a.psplits = plan.force_splits;
    }
}
}  // namespace

LLMX_API llmx_plan* llmx_plan_make(const llmx_model* model, llmx_part* const* parts, int n_parts, const int* counts, const int* histories,
                                   int requests, int room, int typical_context) {
    if (requests <= 0 || !counts || (!histories && room <= 0)) {
        fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_plan_make: the rows each request brings, and histories or room");
        return nullptr;
    }
    std::vector<AttnKey> keys;
    if (model)
        for (const Block* b : model->blocks) b->collect(keys);
    for (int i = 0; i < n_parts; ++i)
        if (parts && parts[i]) parts[i]->collect(keys);
    llmx_plan* plan = new llmx_plan;
    plan->requests = requests, plan->room = room, plan->typical_context = typical_context;
    plan->counts.assign(counts, counts + requests);
    int at = 0;
    for (const AttnKey& k : keys) {
        AttnPlan a;
        a.key = k;
        a.offset = at;
        plan_attention(*plan, a, histories);
        at += (requests + 1 + 3) & ~3;
        plan->attn.push_back(a);
    }
    plan->ints = at;
    return plan;
}
LLMX_API int llmx_plan_ints(const llmx_plan* p) { return p ? p->ints : 0; }
LLMX_API void llmx_plan_free(llmx_plan* p) { delete p; }
LLMX_API void llmx_plan_force_prefill_shape(llmx_plan* p, int tiles, int splits) {
    if (!p) return;
    p->force_tiles = tiles, p->force_splits = splits;
    for (AttnPlan& a : p->attn) {
        if (tiles) a.tiles = tiles;
        if (splits) a.psplits = splits;
    }
}
LLMX_API void llmx_plan_force_decode(llmx_plan* p, int splits, int chunk) {
    if (!p || splits < 1 || chunk < 64 || chunk % 64) return;
    for (AttnPlan& a : p->attn) a.splits = splits, a.chunk = chunk;
}
LLMX_API int llmx_plan_fill(llmx_plan* p, const int* histories, int* out) {
    if (!p) return 0;
    if (!out || (p->room > 0 && !histories)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_plan_fill: histories and room for the ints");
    for (AttnPlan& a : p->attn) {
        int* at = out + a.offset;
        std::copy(a.order.begin(), a.order.end(), at);
        int chunk = a.chunk;
        if (p->room > 0) {          // the grid is the recording's; the keys per range follow the context at hand
            int ctx = 64;
            for (int r = 0; r < p->requests; ++r)
                if (p->counts[r] <= a.max_rows) ctx = std::max(ctx, histories[r] + p->counts[r]);
            chunk = std::max(64, cdiv(cdiv(ctx, 64), a.splits) * 64);
        }
        at[a.order.size()] = chunk;
    }
    return 0;
}
LLMX_API int llmx_plan_describe(const llmx_plan* p, int* out) {
    if (!p || p->attn.empty()) return 0;
    const AttnPlan& a = p->attn[0];
    out[0] = a.n_small, out[1] = a.n_large, out[2] = a.splits, out[3] = a.chunk, out[4] = a.tiles, out[5] = a.psplits, out[6] = a.rows_small,
    out[7] = a.rows_large;
    return 1;
}

// ---- parts ----
LLMX_API llmx_part* llmx_rmsnorm_create(const float* weight, int width, float eps, int out_dtype) {
    if (!weight || width <= 0) { fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_rmsnorm_create: a weight and a width"); return nullptr; }
    return new Norm(weight, width, eps, out_dtype);
}
namespace {
bool good(const llmx_linear_desc& d) {
    return d.weight && d.out_features > 0 && d.in_features > 0 && (d.dtype == LLMX_DT_F32 || d.dtype == LLMX_DT_BF16);
}
}
LLMX_API llmx_part* llmx_linear_create(const llmx_linear_desc* d) {
    if (!d || !good(*d)) { fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_linear_create: a weight, its shape and type"); return nullptr; }
    return new Linear(*d);
}
LLMX_API llmx_part* llmx_attention_create(const llmx_attention_desc* d) {
    if (!d || !good(d->qkv) || !good(d->o) || d->heads <= 0 || d->kv_heads <= 0 || d->heads % d->kv_heads || d->head_dim <= 0 ||
        d->qkv.out_features != (d->heads + 2 * d->kv_heads) * d->head_dim || d->qkv.in_features != d->hidden ||
        d->o.in_features != d->heads * d->head_dim || d->o.out_features != d->hidden || d->qkv.dtype != d->o.dtype ||
        (d->cos == nullptr) != (d->sin == nullptr) || (d->cos && (d->rot_half <= 0 || 2 * d->rot_half > d->head_dim)) || d->window < 0) {
        fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_attention_create: sizes and weights do not fit each other");
        return nullptr;
    }
    return new Attention(*d);
}
LLMX_API int llmx_attention_set_tables(llmx_part* p, const float* cos, const float* sin, int rot_half, int positions) {
    Attention* a = dynamic_cast<Attention*>(p);
    if (!a || (cos == nullptr) != (sin == nullptr) || (cos && (rot_half <= 0 || 2 * rot_half > a->d.head_dim)))
        return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_attention_set_tables: not an attention part, or tables that do not fit");
    a->d.cos = cos, a->d.sin = sin, a->d.rot_half = rot_half, a->d.table_positions = positions;
    return 0;
}
LLMX_API llmx_part* llmx_gated_mlp_create(const llmx_mlp_desc* d) {
    if (!d || !good(d->gate_up) || !good(d->down) || d->gate_up.out_features != 2 * d->intermediate || d->gate_up.in_features != d->hidden ||
        d->down.in_features != d->intermediate || d->down.out_features != d->hidden || d->gate_up.dtype != d->down.dtype) {
        fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_gated_mlp_create: sizes and weights do not fit each other");
        return nullptr;
    }
    return new GatedMlp(*d);
}
LLMX_API llmx_part* llmx_prenorm_block_create(llmx_part* n1, llmx_part* mixer, llmx_part* n2, llmx_part* ffn) {
    Norm *a = as<Norm>(n1, PART_NORM), *b = as<Norm>(n2, PART_NORM);
    Mixer* m = as<Mixer>(mixer, PART_MIXER);
    FeedForward* f = as<FeedForward>(ffn, PART_FFN);
    if (!a || !b || !m || !f) { fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_prenorm_block_create: two norms, a mixer and a feed-forward"); return nullptr; }
    return new PreNormBlock(a, m, b, f);
}
LLMX_API llmx_part* llmx_callback_create(int kind, llmx_callback fn, void* user, int hidden) {
    if (!fn) { fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_callback_create: a function"); return nullptr; }
    if (kind == 0) return new CallbackBlock(fn, user);
    if (kind == 1) return new CallbackMixer(fn, user, hidden);
    if (kind == 2) return new CallbackFfn(fn, user, hidden);
    fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_callback_create: kind 0 (block), 1 (mixer) or 2 (feed-forward)");
    return nullptr;
}
LLMX_API llmx_part* llmx_embedding_create(const void* table, int dtype, int vocab, int width) {
    if (!table || vocab <= 0 || width <= 0) { fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_embedding_create: a table and its shape"); return nullptr; }
    return new Embedding(table, dtype, vocab, width);
}
LLMX_API llmx_part* llmx_head_create(llmx_part* norm, const llmx_linear_desc* weight) {
    Norm* n = as<Norm>(norm, PART_NORM);
    if (!n || !weight || !good(*weight) || weight->in_features != n->width) {
        fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_head_create: a norm and a weight of its width");
        return nullptr;
    }
    return new Head(n, *weight);
}
LLMX_API void llmx_part_destroy(llmx_part* p) { delete p; }

namespace {
int finish(Ctx& c) { return c.status; }
bool good_step(const llmx_step* s) {
    if (!s || s->rows < 0 || s->requests < 0 || s->groups < 0 || s->groups > LLMX_MAX_GROUPS) {
        fail(LLMX_RT_ERR_BAD_ARGUMENT, "the step's description is malformed");
        return false;
    }
    return true;
}
}  // namespace

LLMX_API int llmx_norm_forward(llmx_part* p, const llmx_step* s, const float* x, void* out, int out_dtype, const int* row_index, int rows,
                               float* zero, long long zero_count) {
    Norm* n = as<Norm>(p, PART_NORM);
    if (!n || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_norm_forward: not a norm");
    Ctx c(s, false);
    n->forward(c, x, out, out_dtype, row_index, rows, zero, zero_count);
    return finish(c);
}
LLMX_API long long llmx_part_wants_cleared(llmx_part* p, const llmx_step* s, int rows) {
    if (!p || !good_step(s)) return 0;
    Ctx c(s, true);
    if (Mixer* m = as<Mixer>(p, PART_MIXER)) return m->wants_cleared(c, rows);
    if (FeedForward* f = as<FeedForward>(p, PART_FFN)) return f->wants_cleared(c, rows);
    return 0;
}
LLMX_API int llmx_mixer_forward(llmx_part* p, const llmx_step* s, const void* h, int rows, int cache_entry, float* residual, int write_cache,
                                float* cleared) {
    Mixer* m = as<Mixer>(p, PART_MIXER);
    if (!m || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_mixer_forward: not a mixer");
    Ctx c(s, false);
    m->forward(c, h, rows, cache_entry, residual, write_cache != 0, cleared);
    return finish(c);
}
LLMX_API int llmx_ffn_forward(llmx_part* p, const llmx_step* s, const void* h, int rows, float* residual, float* cleared) {
    FeedForward* f = as<FeedForward>(p, PART_FFN);
    if (!f || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_ffn_forward: not a feed-forward");
    Ctx c(s, false);
    f->forward(c, h, rows, residual, cleared);
    return finish(c);
}
LLMX_API int llmx_block_forward(llmx_part* p, const llmx_step* s, float* x, int rows, int cache_entry, int write_cache) {
    Block* b = as<Block>(p, PART_BLOCK);
    if (!b || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_block_forward: not a block");
    Ctx c(s, false);
    b->forward(c, x, rows, cache_entry, write_cache != 0);
    return finish(c);
}
LLMX_API int llmx_embedding_forward(llmx_part* p, const llmx_step* s, const int* ids, float* x, int rows) {
    Embedding* e = as<Embedding>(p, PART_EMBEDDING);
    if (!e || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_embedding_forward: not an embedding");
    Ctx c(s, false);
    e->forward(c, ids, x, rows);
    return finish(c);
}
LLMX_API int llmx_head_forward(llmx_part* p, const llmx_step* s, const float* x, float* logits) {
    Head* h = as<Head>(p, PART_HEAD);
    if (!h || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_head_forward: not a head");
    Ctx c(s, false);
    h->forward(c, x, logits);
    return finish(c);
}
LLMX_API int llmx_linear_forward(llmx_part* p, const llmx_step* s, const void* a, int rows, float* out, int accumulate, int cleared) {
    Linear* l = as<Linear>(p, PART_LINEAR);
    if (!l || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_linear_forward: not a linear part");
    Ctx c(s, false);
    l->forward(c, a, rows, out, accumulate != 0, cleared != 0);
    return finish(c);
}
LLMX_API int llmx_linear_gated(llmx_part* p, const llmx_step* s, const void* a, int rows, void* out) {
    Linear* l = as<Linear>(p, PART_LINEAR);
    if (!l || !good_step(s) || !l->tensor_core) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_linear_gated: not a tensor-core linear part");
    Ctx c(s, false);
    l->gated(c, a, rows, out);
    return finish(c);
}
LLMX_API int llmx_linear_adds_pieces(llmx_part* p, int rows) {
    Linear* l = as<Linear>(p, PART_LINEAR);
    return l && l->adds_pieces(rows) ? 1 : 0;
}
LLMX_API size_t llmx_part_workspace(llmx_part* p, const llmx_step* s, int rows, int cache_entry) {
    if (!p || !good_step(s)) return 0;
    Ctx c(s, true);
    if (Mixer* m = as<Mixer>(p, PART_MIXER)) m->forward(c, nullptr, rows, cache_entry, nullptr, true, nullptr);
    else if (FeedForward* f = as<FeedForward>(p, PART_FFN)) f->forward(c, nullptr, rows, nullptr, nullptr);
    else if (Block* b = as<Block>(p, PART_BLOCK)) b->forward(c, nullptr, rows, cache_entry, true);
    else if (Head* h = as<Head>(p, PART_HEAD)) h->forward(c, nullptr, nullptr);
    return c.peak + 256;
}

// ---- the attention dispatch alone (what a mixer runs once its queries are made) ----
namespace {
Attention bare_attention(int q_dtype, int heads, int kv_heads, int head_dim, int window, float scale) {
    llmx_attention_desc d = {};
    d.heads = heads, d.kv_heads = kv_heads, d.head_dim = head_dim, d.window = window, d.scale = scale;
    d.qkv.dtype = d.o.dtype = q_dtype;
    d.qkv.out_features = (heads + 2 * kv_heads) * head_dim;
    return Attention(d);
}
const CacheEntry* kv_entry(const llmx_step* s, int entry, int kv_heads, int head_dim) {
    if (!good_step(s) || !s->caches || entry < 0 || entry >= (int)s->caches->entries.size()) return nullptr;
    const CacheEntry& e = s->caches->entries[entry];
    return e.kind == 1 && e.kv_heads == kv_heads && e.head_dim == head_dim ? &e : nullptr;
}
}  // namespace
// An attention shape without weights: good for launch plans (llmx_plan_make) of callers that run the attention
// kernels on queries of their own.
LLMX_API llmx_part* llmx_attention_shape(int heads, int kv_heads, int head_dim, int window) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || head_dim <= 0 || window < 0) {
        fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_attention_shape: head counts, a head width and a window");
        return nullptr;
    }
    return new Attention(bare_attention(LLMX_DT_BF16, heads, kv_heads, head_dim, window, 1.0f));
}
// out = attention of the step's rows over cache entry `entry`; q/out [rows, heads * head_dim] of `q_dtype`.
LLMX_API int llmx_paged_attention(const llmx_step* s, const void* q, int q_dtype, int entry, void* out, int heads, int kv_heads, int head_dim,
                                  int window, float scale) {
    const CacheEntry* e = kv_entry(s, entry, kv_heads, head_dim);
    if (!e || heads <= 0 || heads % kv_heads) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_paged_attention: the entry and the head counts do not fit");
    Attention a = bare_attention(q_dtype, heads, kv_heads, head_dim, window, scale);
    Ctx c(s, false);
    a.attend(c, q, *e, out, s->rows, e->group);
    return c.status;
}
LLMX_API size_t llmx_paged_attention_workspace(const llmx_step* s, int entry, int heads, int kv_heads, int head_dim, int window) {
    const CacheEntry* e = kv_entry(s, entry, kv_heads, head_dim);
    if (!e) return 0;
    Attention a = bare_attention(LLMX_DT_BF16, heads, kv_heads, head_dim, window, 1.0f);
    Ctx c(s, true);
    a.attend(c, nullptr, *e, nullptr, s->rows, e->group);
    a.from_qkv(c, nullptr, *e, nullptr, s->rows, nullptr, e->group);
    return c.peak + 256;
}
// The decode kernel taking the q/k/v product's float32 output [rows, (heads + 2 kv_heads) * head_dim] as it is.
// Returns 0 when it ran, -1 when the step or the shapes do not qualify (nothing was done), else an error code.
LLMX_API int llmx_decode_from_qkv(const llmx_step* s, const float* qkv, int entry, const float* q_weight, const float* k_weight, float eps,
                                  const float* cos, const float* sin, int rot_half, void* out, int heads, int kv_heads, int head_dim, int window,
                                  float scale) {
    const CacheEntry* e = kv_entry(s, entry, kv_heads, head_dim);
    if (!e || heads <= 0 || heads % kv_heads) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_decode_from_qkv: the entry and the head counts do not fit");
    Attention a = bare_attention(LLMX_DT_BF16, heads, kv_heads, head_dim, window, scale);
    a.d.q_norm = q_weight, a.d.k_norm = k_weight, a.d.qk_norm_eps = eps, a.d.cos = cos, a.d.sin = sin, a.d.rot_half = rot_half;
    Ctx c(s, false);
    const bool ran = a.from_qkv(c, qkv, *e, out, s->rows, c.meta(s->slots[e->group]), e->group);
    return c.status ? c.status : ran ? 0 : -1;
}

// ---- the model ----
LLMX_API llmx_model* llmx_model_create(llmx_part* embedding, llmx_part* const* blocks, int n_blocks, const llmx_layer_step* order, int n_order,
                                       llmx_part* head, int hidden, int vocab) {
    Embedding* e = as<Embedding>(embedding, PART_EMBEDDING);
    Head* h = as<Head>(head, PART_HEAD);
    if (!e || !h || n_blocks < 0 || n_order < 0 || hidden <= 0 || vocab <= 0 || e->width != hidden || h->linear.N != vocab) {
        fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_model_create: an embedding, blocks, an order and a head that fit each other");
        return nullptr;
    }
    llmx_model* m = new llmx_model;
    m->embedding = e, m->head = h, m->hidden = hidden, m->vocab = vocab;
    for (int i = 0; i < n_blocks; ++i) {
        Block* b = as<Block>(blocks[i], PART_BLOCK);
        if (!b) {
            delete m;
            fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_model_create: a block is not a block");
            return nullptr;
        }
        m->blocks.push_back(b);
    }
    for (int i = 0; i < n_order; ++i) {
        if (order[i].block < 0 || order[i].block >= n_blocks) {
            delete m;
            fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_model_create: the order names a block the model does not have");
            return nullptr;
        }
        m->order.push_back(order[i]);
    }
    return m;
}
LLMX_API void llmx_model_destroy(llmx_model* m) { delete m; }
LLMX_API size_t llmx_model_workspace(const llmx_model* m, const llmx_step* s) {
    if (!m || !good_step(s)) return 0;
    Ctx c(s, true);
    const_cast<llmx_model*>(m)->forward(c, nullptr);
    return c.peak + 256;
}
LLMX_API int llmx_model_forward(llmx_model* m, const llmx_step* s, float* logits) {
    if (!m || !good_step(s)) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_model_forward: a model and a step");
    if (s->wanted > 0 && !logits) return fail(LLMX_RT_ERR_BAD_ARGUMENT, "llmx_model_forward: logits are wanted but there is nowhere to put them");
    Ctx c(s, false);
    m->forward(c, logits);
    return c.status;
}
