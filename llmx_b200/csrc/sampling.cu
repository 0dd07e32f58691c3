// Sampling on the device: greedy, temperature, top-k, top-p (nucleus), min-p and the penalties,
// with the meaning the reference's host sampler gives them (src/inference/sampler.hpp:258-378):
//
//   penalties    a seen token's logit v becomes v > 0 ? v / p : v * p (once), then presence +
//                frequency * count comes off it
//   temp <= 0    the largest score, ties to the lowest id (sampler.hpp:88-132)
//   otherwise    weight_i = exp((s_i - s_best) / temp) over the kept tokens;
//                top-k keeps the k best by (score descending, id ascending);
//                without top-p the draw walks the kept tokens in id order (min-p zeroes weights below it);
//                with top-p the nucleus is the shortest ranked prefix whose weight reaches
//                top_p * (kept weight), min-p then cuts its tail (never the best), and the draw
//                walks the nucleus best first.
//   the draw     target = r * weight of the walked set; the first token whose running sum exceeds it.
//
// `r` is the request's own uniform number, made on the host from its own generator, so a draw
// does not depend on what else is in the batch.  One block works on one row.  The top-k threshold is found by
// radix selection over the 32-bit order-preserving image of the score (counting tokens).  When the kept set
// then fits shared memory (top-k of at most 1,024, the usual case) it is gathered there, ranked, and
// the nucleus, min-p and the draw are one thread's walk over it with double sums, exactly the reference's
// walk; the vocabulary is read seven times in all (16-byte loads), where every later threshold used to be
// another radix selection over it (top-k 40, top-p 0.95 at 151,936 tokens: 670 us a draw before).  Without top-k
// (or a larger one) nothing is gathered: thresholds by radix selection over the vocabulary, summing weights.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int THREADS = 1024;
constexpr int KMAX = 1024;        // kept tokens a block gathers into shared memory
constexpr int TIES = 32;          // tokens with exactly the same score that are picked among without a second pass

// Calls f(id, score, in_range) for every id of the row, four consecutive ids a thread and round with 16-byte loads
// when the row allows.  Every thread of the block makes the same number of calls (ids past the end come with
// in_range false), so f may use warp-wide operations.
template <typename F>
__device__ __forceinline__ void scan_row(const float* __restrict__ row, int n, F&& f) {
    if ((((uintptr_t)row) & 15) == 0) {
        const int n4 = n >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int rounds = (n4 + THREADS - 1) / THREADS;
        // Eight loads of a thread are in flight before the first is used: one block must cover the latency of the
        // whole row by itself.
        constexpr int AHEAD = 8;
        for (int r0 = 0; r0 < rounds; r0 += AHEAD) {
            float4 v[AHEAD];
#pragma unroll
            for (int u = 0; u < AHEAD; ++u) {
                const int i = (r0 + u) * THREADS + threadIdx.x;
                v[u] = i < n4 ? __ldg(row4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < AHEAD; ++u) {
                if (r0 + u >= rounds) break;          // the same for every thread
                const int i = (r0 + u) * THREADS + threadIdx.x;
                const bool ok = i < n4;
                f(4 * i, v[u].x, ok);
                f(4 * i + 1, v[u].y, ok);
                f(4 * i + 2, v[u].z, ok);
                f(4 * i + 3, v[u].w, ok);
            }
        }
        if (n & 3) {
            const int id = 4 * n4 + threadIdx.x;
            const bool ok = id < n;
            f(id, ok ? row[id] : 0.0f, ok);
        }
    } else {
        const int rounds = (n + THREADS - 1) / THREADS;
#pragma unroll 4
        for (int r = 0; r < rounds; ++r) {
            const int id = r * THREADS + threadIdx.x;
            const bool ok = id < n;
            f(id, ok ? row[id] : 0.0f, ok);
        }
    }
}

struct RowParams {
    float temperature, top_p, min_p, r;
    int top_k, masked;
};

__device__ __forceinline__ uint32_t order_bits(float s) {
    s += 0.0f;  // -0 and +0 tie
    uint32_t b = __float_as_uint(s);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Shared {
    unsigned int count[256];
    double weight[256];
    double scan[THREADS];
    float best_score[32];
    int best_id[32];
    uint32_t u32[4];
    double f64[4];
    int i32[4];
};

// Which tokens take part: all but the masked one; then the top-k set; then the nucleus.
struct Sets {
    int skip;                 // masked id or -1
    bool has_topk;            // kept = bits > topk_bits || (bits == topk_bits && id <= topk_last_id)
    uint32_t topk_bits;
    int topk_last_id;
    bool has_nucleus;
    uint32_t nuc_bits;
    int nuc_last_id;
    bool has_minp;            // nucleus additionally needs weight >= min_p or to be the best
    float min_p;
    int best;
};

__device__ __forceinline__ bool in_kept(const Sets& s, int id, uint32_t bits) {
    if (id == s.skip) return false;
    if (!s.has_topk) return true;
    return bits > s.topk_bits || (bits == s.topk_bits && id <= s.topk_last_id);
}

__device__ __forceinline__ bool in_nucleus(const Sets& s, int id, uint32_t bits, float w) {
    if (!in_kept(s, id, bits)) return false;
    if (s.has_nucleus && !(bits > s.nuc_bits || (bits == s.nuc_bits && id <= s.nuc_last_id))) return false;
    if (s.has_minp && w < s.min_p && id != s.best) return false;
    return true;
}

// The id of the (nth + 1)-th token, in id order, with these bits among the tokens of a set
// (level 0: not masked, 1: kept, 2: nucleus).  Every thread returns the same id (-1 if there are fewer).
template <int LEVEL>
__device__ int nth_with_bits(const float* row, int n, uint32_t bits, int nth, const Sets& sets, float best_score,
                             float temp, Shared& sh) {
    __shared__ int found;
    __shared__ int base;
    __shared__ int n_hits;
    __shared__ int hit_list[TIES];
    if (threadIdx.x == 0) { found = -1; base = 0; n_hits = 0; }
    __syncthreads();
    // Scores are rarely equal bit for bit: one pass lists the few tokens that are, one thread picks among them.
    scan_row(row, n, [&](int id, float s, bool ok) {
        if (!ok) return;
        const uint32_t b = order_bits(s);
        if (b != bits) return;
        bool hit;
        if (LEVEL == 0) hit = id != sets.skip;
        else if (LEVEL == 1) hit = in_kept(sets, id, b);
        else hit = in_nucleus(sets, id, b, expf((s - best_score) / temp));
        if (hit) {
            const int slot = atomicAdd(&n_hits, 1);
            if (slot < TIES) hit_list[slot] = id;
        }
    });
    __syncthreads();
    if (n_hits <= TIES) {
        if (threadIdx.x == 0) {
            for (int i = 1; i < n_hits; ++i) {          // by id, ascending
                const int v = hit_list[i];
                int j = i - 1;
                for (; j >= 0 && hit_list[j] > v; --j) hit_list[j + 1] = hit_list[j];
                hit_list[j + 1] = v;
            }
            found = nth < n_hits ? hit_list[nth] : -1;
        }
        __syncthreads();
        const int id = found;
        __syncthreads();
        return id;
    }
    for (int start = 0; start < n; start += THREADS) {
        const int id = start + threadIdx.x;
        bool hit = false;
        if (id < n) {
            const float s = row[id];
            const uint32_t b = order_bits(s);
            if (b == bits) {
                if (LEVEL == 0) hit = id != sets.skip;
                else if (LEVEL == 1) hit = in_kept(sets, id, b);
                else hit = in_nucleus(sets, id, b, expf((s - best_score) / temp));
            }
        }
        // Rank of this hit among the block's hits in id order: ballot within the warp, warp totals through smem.
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (lane == 0) sh.count[warp] = __popc(ballot);
        __syncthreads();
        int before = base;
        for (int w = 0; w < warp; ++w) before += sh.count[w];
        before += __popc(ballot & ((1u << lane) - 1));
        if (hit && before == nth) found = id;
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < THREADS / 32; ++w) total += sh.count[w];
            base += total;
        }
        __syncthreads();
        if (found >= 0 || base > nth) break;
    }
    __syncthreads();
    return found;
}

// Radix selection by count: the bits of the k-th best token (k >= 1) among the tokens of level 0
// (not masked), and how many tokens with exactly those bits are among the k best.
__device__ void select_by_count(const float* row, int n, int k, const Sets& sets, Shared& sh, uint32_t& out_bits,
                                int& out_equal_taken) {
    uint32_t prefix = 0, mask = 0;
    int remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += THREADS) sh.count[i] = 0;
        __syncthreads();
        // Most scores share their leading bits: the lanes of a warp that fall into one bin add to it once.
        scan_row(row, n, [&](int id, float s, bool ok) {
            const uint32_t b = order_bits(s);
            const bool part = ok && id != sets.skip && (b & mask) == prefix;
            const unsigned who = __ballot_sync(0xffffffffu, part);
            if (part) {
                const unsigned bin = (b >> shift) & 255u;
                const unsigned peers = __match_any_sync(who, bin);
                if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&sh.count[bin], (unsigned)__popc(peers));
            }
        });
        __syncthreads();
        if (threadIdx.x == 0) {
            int acc = 0, bin = 255;
            for (; bin > 0; --bin) {
                if (acc + (int)sh.count[bin] >= remaining) break;
                acc += (int)sh.count[bin];
            }
            sh.u32[0] = (uint32_t)bin;
            sh.i32[0] = remaining - acc;
        }
        __syncthreads();
        prefix |= sh.u32[0] << shift;
        mask |= 255u << shift;
        remaining = sh.i32[0];
        __syncthreads();
    }
    out_bits = prefix;
    out_equal_taken = remaining;
}

// Radix selection by weight over the tokens of LEVEL, best first: the bits at which the running
// weight first reaches `goal` (strict: first exceeds it), the weight of the tokens above those
// bits, and how many tokens have exactly those bits.
template <int LEVEL>
__device__ void select_by_weight(const float* row, int n, double goal, bool strict, const Sets& sets, float best_score,
                                 float temp, Shared& sh, uint32_t& out_bits, double& out_above, int& out_equal_count) {
    uint32_t prefix = 0, mask = 0;
    double above = 0.0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += THREADS) { sh.count[i] = 0; sh.weight[i] = 0.0; }
        __syncthreads();
        for (int id = threadIdx.x; id < n; id += THREADS) {
            const float s = row[id];
            const uint32_t b = order_bits(s);
            if ((b & mask) != prefix) continue;
            const float w = expf((s - best_score) / temp);
            const bool in = LEVEL == 1 ? in_kept(sets, id, b) : in_nucleus(sets, id, b, w);
            if (!in) continue;
            const int bin = (b >> shift) & 255u;
            atomicAdd(&sh.count[bin], 1u);
            atomicAdd(&sh.weight[bin], (double)w);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            double acc = above;
            int bin = 255, last_nonempty = -1;
            for (; bin >= 0; --bin) {
                if (!sh.count[bin]) continue;
                last_nonempty = bin;
                const double next = acc + sh.weight[bin];
                if (strict ? (goal < next) : (next >= goal)) break;
                acc = next;
            }
            if (bin < 0) {               // rounding left the goal just out of reach: stop at the last tokens
                bin = last_nonempty < 0 ? 0 : last_nonempty;
                acc -= sh.weight[bin];
            }
            sh.u32[0] = (uint32_t)bin;
            sh.f64[0] = acc;
            sh.i32[0] = (int)sh.count[bin];
        }
        __syncthreads();
        prefix |= sh.u32[0] << shift;
        mask |= 255u << shift;
        above = sh.f64[0];
        out_equal_count = sh.i32[0];
        __syncthreads();
    }
    out_bits = prefix;
    out_above = above;
}

// Sum of the weights of LEVEL's tokens (min-p zeroing applied when asked), every thread gets the total.
template <int LEVEL>
__device__ double total_weight(const float* row, int n, const Sets& sets, float best_score, float temp, float zero_below,
                               Shared& sh) {
    double mine = 0.0;
    for (int id = threadIdx.x; id < n; id += THREADS) {
        const float s = row[id];
        const uint32_t b = order_bits(s);
        float w = expf((s - best_score) / temp);
        const bool in = LEVEL == 1 ? in_kept(sets, id, b) : in_nucleus(sets, id, b, w);
        if (!in) continue;
        if (w < zero_below) w = 0.0f;
        mine += (double)w;
    }
    sh.scan[threadIdx.x] = mine;
    __syncthreads();
    for (int o = THREADS / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh.scan[threadIdx.x] += sh.scan[threadIdx.x + o];
        __syncthreads();
    }
    const double total = sh.scan[0];
    __syncthreads();
    return total;
}

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int vocab,
                                                         const RowParams* __restrict__ params, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ Shared sh;
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const RowParams p = params[blockIdx.x];
    const int n = vocab;
    Sets sets;
    sets.skip = (p.masked >= 0 && p.masked < n && n > 1) ? p.masked : -1;
    sets.has_topk = sets.has_nucleus = sets.has_minp = false;
    sets.topk_bits = sets.nuc_bits = 0;
    sets.topk_last_id = sets.nuc_last_id = n;
    sets.min_p = 0.0f;

    // ---- the best token: largest score, ties to the lowest id; a NaN only as the first token taking part
    const int first = sets.skip == 0 ? 1 : 0;
    float bs = -INFINITY;
    int bi = first;
    scan_row(row, n, [&](int id, float s, bool ok) {
        if (ok && id != sets.skip && (s > bs || (s == bs && id < bi))) { bs = s; bi = id; }
    });
    for (int o = 16; o > 0; o >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, bs, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (os > bs || (os == bs && oi < bi)) { bs = os; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sh.best_score[threadIdx.x >> 5] = bs; sh.best_id[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < THREADS / 32; ++w)
            if (sh.best_score[w] > bs || (sh.best_score[w] == bs && sh.best_id[w] < bi)) { bs = sh.best_score[w]; bi = sh.best_id[w]; }
        if (isnan(row[first])) bi = first;
        sh.i32[1] = bi;
    }
    __syncthreads();
    const int best = sh.i32[1];
    const float best_score = row[best];
    sets.best = best;
    __syncthreads();
    if (!(p.temperature > 0.0f)) {
        if (threadIdx.x == 0) out[blockIdx.x] = best;
        return;
    }
    const float temp = p.temperature;
    const int m = sets.skip >= 0 ? n - 1 : n;
    const int keep = (p.top_k > 0 && p.top_k < m) ? p.top_k : m;

    // ---- top-k: the bits of the k-th best and the last id taken among its ties
    if (keep < m) {
        uint32_t bits;
        int taken;
        select_by_count(row, n, keep, sets, sh, bits, taken);
        const int last = nth_with_bits<0>(row, n, bits, taken - 1, sets, best_score, temp, sh);
        sets.has_topk = true;
        sets.topk_bits = bits;
        sets.topk_last_id = last < 0 ? n : last;
    }

    if (sets.has_topk && keep <= KMAX) {
        // ---- the kept tokens fit shared memory: gather them, put them in the order of the walk (ids ascending
        // without top-p, best first with it), and let one thread walk them as the reference's sampler does.
        __shared__ int c_id[KMAX], o_id[KMAX];
        __shared__ uint32_t c_bits[KMAX];
        __shared__ float c_w[KMAX], o_w[KMAX];
        __shared__ int n_kept;
        if (threadIdx.x == 0) n_kept = 0;
        __syncthreads();
        scan_row(row, n, [&](int id, float s, bool ok) {
            if (!ok) return;
            const uint32_t b = order_bits(s);
            if (!in_kept(sets, id, b)) return;
            const int slot = atomicAdd(&n_kept, 1);
            if (slot < KMAX) {
                c_id[slot] = id;
                c_bits[slot] = b;
                c_w[slot] = expf((s - best_score) / temp);
            }
        });
        __syncthreads();
        const int K = min(n_kept, KMAX);
        const bool ranked = p.top_p < 1.0f;
        for (int i = threadIdx.x; i < K; i += THREADS) {
            const int id = c_id[i];
            const uint32_t b = c_bits[i];
            int before = 0;
            for (int j = 0; j < K; ++j) {
                const bool first_j = ranked ? (c_bits[j] > b || (c_bits[j] == b && c_id[j] < id)) : c_id[j] < id;
                before += first_j ? 1 : 0;
            }
            o_id[before] = id;
            o_w[before] = c_w[i];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int pick = best;
            if (!ranked) {
                // id order: min-p zeroes the weights below it; the first token whose running sum exceeds the target
                const float cut = p.min_p > 0.0f ? p.min_p : 0.0f;
                double total = 0.0;
                for (int i = 0; i < K; ++i) total += (double)(o_w[i] < cut ? 0.0f : o_w[i]);
                const double target = (double)p.r * total;
                double acc = 0.0;
                for (int i = 0; i < K; ++i) {
                    acc += (double)(o_w[i] < cut ? 0.0f : o_w[i]);
                    if (target < acc) { pick = o_id[i]; break; }
                }
            } else {
                // best first: the nucleus is the shortest prefix whose weight reaches top_p of the kept weight; min-p
                // then cuts its tail (never the best); the draw walks what is left
                double kept_weight = 0.0;
                for (int i = 0; i < K; ++i) kept_weight += (double)o_w[i];
                const double goal = (double)p.top_p * kept_weight;
                int nucleus = K;
                double acc = 0.0;
                for (int i = 0; i < K; ++i) {
                    acc += (double)o_w[i];
                    if (acc >= goal) { nucleus = i + 1; break; }
                }
                const bool cut_tail = p.min_p > 0.0f;
                double nucleus_weight = 0.0;
                for (int i = 0; i < nucleus; ++i)
                    if (!(cut_tail && o_w[i] < p.min_p && o_id[i] != best)) nucleus_weight += (double)o_w[i];
                const double target = (double)p.r * nucleus_weight;
                acc = 0.0;
                int last = -1;
                for (int i = 0; i < nucleus; ++i) {
                    if (cut_tail && o_w[i] < p.min_p && o_id[i] != best) continue;
                    acc += (double)o_w[i];
                    last = o_id[i];
                    if (target < acc) break;
                }
                if (last >= 0) pick = last;
            }
            out[blockIdx.x] = pick;
        }
        return;
    }

    int chosen = best;
    if (p.top_p >= 1.0f) {
        // ---- id order: each thread owns a run of consecutive ids; runs are scanned, one thread walks its run
        const float cut = p.min_p > 0.0f ? p.min_p : 0.0f;
        const int seg = (n + THREADS - 1) / THREADS;
        const int lo = threadIdx.x * seg, hi = min(n, lo + seg);
        double mine = 0.0;
        for (int id = lo; id < hi; ++id) {
            const float s = row[id];
            if (!in_kept(sets, id, order_bits(s))) continue;
            float w = expf((s - best_score) / temp);
            if (w < cut) w = 0.0f;
            mine += (double)w;
        }
        sh.scan[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            double acc = 0.0;
            for (int t = 0; t < THREADS; ++t) { const double v = sh.scan[t]; sh.scan[t] = acc; acc += v; }
            sh.f64[1] = acc;
            sh.i32[2] = -1;
        }
        __syncthreads();
        const double target = (double)p.r * sh.f64[1];
        const double before = sh.scan[threadIdx.x];
        if (target >= before && target < before + mine) {
            double acc = before;
            for (int id = lo; id < hi; ++id) {
                const float s = row[id];
                if (!in_kept(sets, id, order_bits(s))) continue;
                float w = expf((s - best_score) / temp);
                if (w < cut) w = 0.0f;
                acc += (double)w;
                if (target < acc) { sh.i32[2] = id; break; }
            }
        }
        __syncthreads();
        if (sh.i32[2] >= 0) chosen = sh.i32[2];
    } else {
        // ---- rank order: nucleus by weight, min-p on its tail, then the draw best first
        const double kept_weight = total_weight<1>(row, n, sets, best_score, temp, 0.0f, sh);
        const double goal = (double)p.top_p * kept_weight;
        uint32_t bits;
        double above;
        int equal;
        select_by_weight<1>(row, n, goal, false, sets, best_score, temp, sh, bits, above, equal);
        {
            // Tokens with the threshold's bits all weigh the same; take as many as reach the goal (at least one).
            const float s_t = __uint_as_float((bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits);
            const double w_t = (double)expf((s_t - best_score) / temp);
            long long j = 1;
            if (w_t > 0.0 && above + w_t < goal) j = (long long)ceil((goal - above) / w_t);
            if (j < 1) j = 1;
            if (j > equal) j = equal;
            const int last = nth_with_bits<1>(row, n, bits, (int)j - 1, sets, best_score, temp, sh);
            sets.has_nucleus = true;
            sets.nuc_bits = bits;
            sets.nuc_last_id = last < 0 ? n : last;
        }
        if (p.min_p > 0.0f) { sets.has_minp = true; sets.min_p = p.min_p; }
        const double nucleus_weight = total_weight<2>(row, n, sets, best_score, temp, 0.0f, sh);
        const double target = (double)p.r * nucleus_weight;
        select_by_weight<2>(row, n, target, true, sets, best_score, temp, sh, bits, above, equal);
        {
            const float s_t = __uint_as_float((bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits);
            const double w_t = (double)expf((s_t - best_score) / temp);
            long long i = 0;
            if (w_t > 0.0 && target > above) i = (long long)floor((target - above) / w_t);
            if (i >= equal) i = equal - 1;
            if (i < 0) i = 0;
            const int id = nth_with_bits<2>(row, n, bits, (int)i, sets, best_score, temp, sh);
            if (id >= 0) chosen = id;
        }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = chosen;
}

// Greedy rows only: the largest score, ties to the lowest id, a NaN only as the first token taking part
// (src/inference/sampler.hpp:88-132), with 16-byte loads.  Used when no row of the batch draws.
__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int vocab,
                                                         const RowParams* __restrict__ params, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float best_score[32];
    __shared__ int best_id[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int masked = params[blockIdx.x].masked;
    const int skip = (masked >= 0 && masked < vocab && vocab > 1) ? masked : -1;
    const int first = skip == 0 ? 1 : 0;
    float bs = -INFINITY;
    int bi = first;
    const bool vec = (vocab % 4 == 0) && (((uintptr_t)row & 15) == 0);
    if (vec) {
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int i = threadIdx.x; i < vocab / 4; i += THREADS) {
            const float4 v = row4[i];
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int id = 4 * i + k;
                if (id != skip && (e[k] > bs || (e[k] == bs && id < bi))) { bs = e[k]; bi = id; }
            }
        }
    } else {
        for (int id = threadIdx.x; id < vocab; id += THREADS) {
            const float s = row[id];
            if (id != skip && (s > bs || (s == bs && id < bi))) { bs = s; bi = id; }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, bs, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (os > bs || (os == bs && oi < bi)) { bs = os; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { best_score[threadIdx.x >> 5] = bs; best_id[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < THREADS / 32; ++w)
            if (best_score[w] > bs || (best_score[w] == bs && best_id[w] < bi)) { bs = best_score[w]; bi = best_id[w]; }
        if (isnan(row[first])) bi = first;
        out[blockIdx.x] = bi;
    }
}

// One thread per (row, seen token): the repetition penalty, then the additive ones.
__global__ void penalty_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ row_of,
                               const int* __restrict__ token, const int* __restrict__ count,
                               const float* __restrict__ repetition, const float* __restrict__ presence,
                               const float* __restrict__ frequency, int items) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= items) return;
    const int r = row_of[i], t = token[i];
    if (t < 0 || t >= vocab) return;
    float* v = logits + (size_t)r * vocab + t;
    float s = *v;
    const float p = repetition[r];
    if (p > 0.0f && p != 1.0f) s = s > 0.0f ? s / p : s * p;
    if (presence[r] != 0.0f || frequency[r] != 0.0f) s -= presence[r] + frequency[r] * (float)count[i];
    *v = s;
}

}  // namespace

// params: rows x {temperature, top_p, min_p, r, top_k, masked} (24 bytes each) on the device.
// `all_greedy` != 0: every row has temperature <= 0 (the caller knows); the argmax kernel alone runs.
LLMX_EXPORT int llmx_sample(const float* logits, int rows, int vocab, const void* params, int* out, int all_greedy,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return LLMX_ERR_BAD_ARGUMENT;
    if (all_greedy) {
        launch_kernel(argmax_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, vocab, (const RowParams*)params, out);
        return launch_status();
    }
    launch_kernel(sample_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, vocab, (const RowParams*)params, out);
    return launch_status();
}

LLMX_EXPORT int llmx_penalize(float* logits, int vocab, const int* row_of, const int* token, const int* count,
                              const float* repetition, const float* presence, const float* frequency, int items,
                              cudaStream_t stream) {
    if (items <= 0) return 0;
    launch_kernel(penalty_kernel, dim3((items + 255) / 256), dim3(256), 0, stream, logits, vocab, row_of, token, count,
                  repetition, presence, frequency, items);
    return launch_status();
}
