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
// does not depend on what else is in the batch.  A row is the work of a thread-block cluster of up to eight blocks:
// each scans its slice of the vocabulary, their counts and sums meet in the first block's shared memory, which
// decides (one block alone issues instructions for 150,000 scores at about 25 us a pass, whatever its loads do).
// The top-k threshold is found by radix selection over the 32-bit order-preserving image of the score (counting
// tokens).  When the kept set then fits shared memory (top-k of at most 1,024, the usual case) it is gathered
// there, ranked, and the nucleus, min-p and the draw are one thread's walk over it with double sums, exactly the
// reference's walk.  Without top-k (or a larger one) nothing is gathered: thresholds by radix selection over the
// vocabulary, summing weights.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int THREADS = 1024;
constexpr int KMAX = 1024;        // kept tokens that are gathered into shared memory
constexpr int TIES = 32;          // tokens with exactly the same score that are picked among without a second pass
constexpr int MAX_CLUSTER = 8;    // blocks that share a row
constexpr int NO_ID = 0x7fffffff;
constexpr int STRIPES_BYTES = 256 * 32 * (8 + 4);

struct RowParams {
    float temperature, top_p, min_p, r;
    int top_k, masked;
};

__device__ __forceinline__ uint32_t order_bits(float s) {
    s += 0.0f;  // -0 and +0 tie
    uint32_t b = __float_as_uint(s);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// ---- the blocks of a row: a thread-block cluster.  Every block scans its slice of the vocabulary; what the blocks
// find meets in the shared memory of the cluster's first block (the leader), which decides and from which all read
// the decision back.  Nothing but the leader's shared memory is touched from outside its block, and the leader does
// not leave before every block has read what it wants of it (a cluster barrier before each exit that follows a read).
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_blocks() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of the leader's copy of a shared-memory location of this block.
__device__ __forceinline__ uint32_t on_leader(const void* local) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(a) : "r"((uint32_t)__cvta_generic_to_shared(local)));
    return a;
}
__device__ __forceinline__ void lead_add(const unsigned* p, unsigned v) {
    asm volatile("red.relaxed.cluster.shared::cluster.add.u32 [%0], %1;" ::"r"(on_leader(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void lead_add(const double* p, double v) {
    asm volatile("red.relaxed.cluster.shared::cluster.add.f64 [%0], %1;" ::"r"(on_leader(p)), "d"(v) : "memory");
}
__device__ __forceinline__ void lead_min(const int* p, int v) {
    asm volatile("red.relaxed.cluster.shared::cluster.min.s32 [%0], %1;" ::"r"(on_leader(p)), "r"(v) : "memory");
}
__device__ __forceinline__ int lead_take(const int* p) {       // the leader's counter before it is raised by one
    int old;
    asm volatile("atom.relaxed.cluster.shared::cluster.add.s32 %0, [%1], 1;" : "=r"(old) : "r"(on_leader(p)) : "memory");
    return old;
}
__device__ __forceinline__ int lead_reserve(const int* p, int n) {       // the leader's counter before it is raised by n
    int old;
    asm volatile("atom.relaxed.cluster.shared::cluster.add.s32 %0, [%1], %2;" : "=r"(old) : "r"(on_leader(p)), "r"(n) : "memory");
    return old;
}
__device__ __forceinline__ void lead_store(const int* p, int v) {
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(on_leader(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void lead_store(const uint32_t* p, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(on_leader(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void lead_store(const float* p, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(on_leader(p)), "f"(v) : "memory");
}
__device__ __forceinline__ void lead_store(const double* p, double v) {
    asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(on_leader(p)), "d"(v) : "memory");
}
__device__ __forceinline__ int lead_load(const int* p) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(on_leader(p)) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lead_load(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(on_leader(p)) : "memory");
    return v;
}
__device__ __forceinline__ double lead_load(const double* p) {
    double v;
    asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(on_leader(p)) : "memory");
    return v;
}

struct Shared {
    // each block's own
    unsigned int count[256];
    int min_id[256];              // a selection's last round: the lowest id of each bin
    double scan[THREADS];
    float best_score[32];
    int best_id[32];
    // the leader's copy is where the blocks meet
    unsigned int gcount[256];
    double gweight[256];
    int gmin_id[256];
    float part_score[MAX_CLUSTER];
    int part_id[MAX_CLUSTER];
    double part_total[MAX_CLUSTER];
    uint32_t u32[4];
    double f64[4];
    int i32[8];
    int n_hits, n_kept, walked;
    int hit_list[TIES];
    int c_id[KMAX], o_id[KMAX];
    uint32_t c_bits[KMAX], l_bits[KMAX];
    float c_w[KMAX], o_w[KMAX];
};

// One row as a block sees it: the row, the block's slice of ids [lo, hi) (lo a multiple of 4), its place in the cluster.
struct Row {
    const float* row;
    int n, lo, hi;
    uint32_t rank, blocks;
    Shared* sh;
    double* stripes;          // the block's own dynamic shared memory: sums [256 bins][32 lanes], then counts (select_by_weight)
};

// The leader's turn: once every block's contributions have landed, the leader's threads run `body`; when they are
// done every block may read what it left.  All threads of all blocks of the cluster call this.
template <typename Body>
__device__ __forceinline__ void leader_turn(const Row& c, Body&& body) {
    cluster_sync();
    if (c.rank == 0) body();
    cluster_sync();
}

// Calls f(id, score, in_range) for every id of the block's slice, four consecutive ids a thread and round with 16-byte
// loads when the row allows, AHEAD loads of a thread in flight before the first is used.  Every thread of the block
// makes the same number of calls (ids past the end come with in_range false), so f may use warp-wide operations.
template <int AHEAD = 8, typename F>
__device__ __forceinline__ void scan_slice(const Row& c, F&& f) {
    const float* __restrict__ row = c.row;
    if ((((uintptr_t)row) & 15) == 0) {
        const int first4 = c.lo >> 2, n4 = c.hi >> 2;              // whole groups of four within the slice
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int rounds = (n4 - first4 + THREADS - 1) / THREADS;
        for (int r0 = 0; r0 < rounds; r0 += AHEAD) {
            float4 v[AHEAD];
#pragma unroll
            for (int u = 0; u < AHEAD; ++u) {
                const int i = first4 + (r0 + u) * THREADS + threadIdx.x;
                v[u] = i < n4 ? __ldg(row4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < AHEAD; ++u) {
                if (r0 + u >= rounds) break;          // the same for every thread
                const int i = first4 + (r0 + u) * THREADS + threadIdx.x;
                const bool ok = i < n4;
                f(4 * i, v[u].x, ok);
                f(4 * i + 1, v[u].y, ok);
                f(4 * i + 2, v[u].z, ok);
                f(4 * i + 3, v[u].w, ok);
            }
        }
        if (c.hi & 3) {                               // the row's last one to three scores (the last slice only)
            const int id = 4 * n4 + threadIdx.x;
            const bool ok = id < c.hi;
            f(id, ok ? row[id] : 0.0f, ok);
        }
    } else {
        const int rounds = (c.hi - c.lo + THREADS - 1) / THREADS;
#pragma unroll 4
        for (int r = 0; r < rounds; ++r) {
            const int id = c.lo + r * THREADS + threadIdx.x;
            const bool ok = id < c.hi;
            f(id, ok ? row[id] : 0.0f, ok);
        }
    }
}

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

template <int LEVEL>
__device__ __forceinline__ bool in_level(const Sets& sets, int id, uint32_t b, float s, float best_score, float temp) {
    if (LEVEL == 0) return id != sets.skip;
    if (LEVEL == 1) return in_kept(sets, id, b);
    return in_nucleus(sets, id, b, expf((s - best_score) / temp));
}

// The bin a radix round stops at, found by the leader's first warp: bins are walked from 255 down, `acc` (starting at
// `above`) grows by each bin's amount, and the walk stops at the first bin where `reached(acc, acc + amount)` holds.
// A lane sums eight consecutive bins, a shuffle scan gives what lies above each lane, the one lane whose bins hold the
// stop walks them.  Returns the bin (or -1 when no bin stops the walk) and the amount above it; every lane of the
// warp gets both.
template <typename T, typename Amount, typename Reached>
__device__ __forceinline__ int find_bin(Amount&& amount, T above, Reached&& reached, T& out_above) {
    const int lane = threadIdx.x & 31;
    T mine = 0;
#pragma unroll
    for (int b = 0; b < 8; ++b) mine += amount(lane * 8 + b);
    // what the lanes above this one hold (lane 31 holds the highest bins)
    T higher = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T up = __shfl_down_sync(0xffffffffu, higher, o);
        if (lane + o < 32) higher += up;
    }
    higher = higher - mine + above;
    const bool here = reached(higher, higher + mine) ;
    const unsigned stops = __ballot_sync(0xffffffffu, here);
    if (!stops) {
        out_above = above;
        return -1;
    }
    const int owner = 31 - __clz(stops);              // the highest lane whose bins reach it
    int bin = -1;
    T acc = higher;
    if (lane == owner) {
        for (int b = 7; b >= 0; --b) {
            const T a = amount(lane * 8 + b);
            if (reached(acc, acc + a)) { bin = lane * 8 + b; break; }
            acc += a;
        }
    }
    bin = __shfl_sync(0xffffffffu, bin, owner);
    out_above = __shfl_sync(0xffffffffu, acc, owner);
    return bin;
}

// The id of the (nth + 1)-th token, in id order, with exactly these bits among the tokens of a set (level 0: not masked,
// 1: kept, 2: nucleus); -1 if there are fewer.  Scores are rarely equal bit for bit: one pass lists the few tokens that
// are and the leader picks among them; more ties than the list holds are walked by the leader alone, chunk by chunk.
// Every thread of the cluster returns the same id.
template <int LEVEL>
__device__ int nth_with_bits(const Row& c, uint32_t bits, int nth, const Sets& sets, float best_score, float temp) {
    Shared& sh = *c.sh;
    scan_slice(c, [&](int id, float s, bool ok) {
        if (!ok) return;
        const uint32_t b = order_bits(s);
        if (b != bits || !in_level<LEVEL>(sets, id, b, s, best_score, temp)) return;
        const int slot = lead_take(&sh.n_hits);
        if (slot < TIES) lead_store(&sh.hit_list[slot], id);
    });
    leader_turn(c, [&] {
        if (threadIdx.x == 0) {
            const int hits = sh.n_hits;
            sh.n_hits = 0;
            sh.i32[4] = hits;
            if (hits <= TIES) {
                for (int i = 1; i < hits; ++i) {          // by id, ascending
                    const int v = sh.hit_list[i];
                    int j = i - 1;
                    for (; j >= 0 && sh.hit_list[j] > v; --j) sh.hit_list[j + 1] = sh.hit_list[j];
                    sh.hit_list[j + 1] = v;
                }
                sh.i32[5] = nth < hits ? sh.hit_list[nth] : -1;
            }
        }
    });
    if (lead_load(&sh.i32[4]) <= TIES) return lead_load(&sh.i32[5]);
    leader_turn(c, [&] {
        // Rank of a hit among the row's hits in id order: ballot within the warp, warp totals through shared memory.
        int& found = sh.i32[6];
        int& base = sh.i32[7];
        if (threadIdx.x == 0) { found = -1; base = 0; }
        __syncthreads();
        for (int start = 0; start < c.n; start += THREADS) {
            const int id = start + threadIdx.x;
            bool hit = false;
            if (id < c.n) {
                const float s = c.row[id];
                const uint32_t b = order_bits(s);
                hit = b == bits && in_level<LEVEL>(sets, id, b, s, best_score, temp);
            }
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
        if (threadIdx.x == 0) sh.i32[5] = found;
    });
    return lead_load(&sh.i32[5]);
}

// Radix selection by count: the bits of the k-th best token (k >= 1) among the tokens that are not masked, how many
// tokens with exactly those bits are among the k best, and the lowest id with those bits (the last round notes each
// bin's, so that the usual case -- one token of the tie is taken -- needs no pass of its own).  A round: every block
// counts its slice's tokens by the next eight bits, adds its bins to the leader's, and the leader finds the bin that
// holds the k-th.
__device__ void select_by_count(const Row& c, int k, const Sets& sets, uint32_t& out_bits, int& out_equal_taken,
                                int& out_first_id) {
    Shared& sh = *c.sh;
    uint32_t prefix = 0, mask = 0;
    int remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += THREADS) { sh.count[i] = 0; sh.min_id[i] = NO_ID; }
        __syncthreads();
        // Most scores share their leading bits: a thread keeps the count of the bin it met last and adds it to the
        // block's bins only when the bin changes.
        int run_bin = -1;
        unsigned run = 0;
        scan_slice(c, [&](int id, float s, bool ok) {
            const uint32_t b = order_bits(s);
            if (!(ok && id != sets.skip && (b & mask) == prefix)) return;
            const int bin = (b >> shift) & 255u;
            if (shift == 0) atomicMin(&sh.min_id[bin], id);
            if (bin != run_bin) {
                if (run) atomicAdd(&sh.count[run_bin], run);
                run_bin = bin;
                run = 0;
            }
            ++run;
        });
        if (run) atomicAdd(&sh.count[run_bin], run);
        __syncthreads();
        if (threadIdx.x < 256 && sh.count[threadIdx.x]) {
            lead_add(&sh.gcount[threadIdx.x], sh.count[threadIdx.x]);
            if (shift == 0) lead_min(&sh.gmin_id[threadIdx.x], sh.min_id[threadIdx.x]);
        }
        leader_turn(c, [&] {
            if (threadIdx.x < 32) {
                int above = 0;
                int bin = find_bin<int>([&](int i) { return (int)sh.gcount[i]; }, 0,
                                        [&](int before, int after) { return after >= remaining && after > before; }, above);
                if (bin < 0) { bin = 0; above = 0; for (int i = 1; i < 256; ++i) above += (int)sh.gcount[i]; }
                if (threadIdx.x == 0) {
                    sh.u32[0] = (uint32_t)bin;
                    sh.i32[0] = remaining - above;
                    sh.i32[2] = sh.gmin_id[bin];
                }
            }
            __syncthreads();
            if (threadIdx.x < 256) { sh.gcount[threadIdx.x] = 0; sh.gmin_id[threadIdx.x] = NO_ID; }      // for the next round
        });
        prefix |= lead_load(&sh.u32[0]) << shift;
        mask |= 255u << shift;
        remaining = lead_load(&sh.i32[0]);
    }
    out_bits = prefix;
    out_equal_taken = remaining;
    const int first = lead_load(&sh.i32[2]);
    out_first_id = first == NO_ID ? -1 : first;
}

// Radix selection by weight over the tokens of LEVEL, best first.  The goal is `fraction` of the set's whole weight,
// which the first round's bins give; found are the bits at which the running weight first reaches the goal (strict:
// first exceeds it), the weight of the tokens above those bits, how many tokens have exactly those bits, and the
// lowest id among them (each bin's is noted in the last round).
template <int LEVEL>
__device__ void select_by_weight(const Row& c, double fraction, bool strict, const Sets& sets, float best_score, float temp,
                                 uint32_t& out_bits, double& out_goal, double& out_above, int& out_equal_count,
                                 int& out_first_id) {
    Shared& sh = *c.sh;
    uint32_t prefix = 0, mask = 0;
    double above = 0.0, goal = 0.0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += THREADS) sh.min_id[i] = NO_ID;
        unsigned* count_stripes = (unsigned*)(c.stripes + 256 * 32);
        for (int i = threadIdx.x; i < 256 * 32; i += THREADS) { c.stripes[i] = 0.0; count_stripes[i] = 0; }
        __syncthreads();
        // An addition of doubles to shared memory is a compare-and-swap loop, which the 32 lanes of a warp that meet in
        // one bin go through one after the other -- and the first rounds have a handful of bins for all tokens.  So a
        // bin's count and sum lie in 32 stripes, one a lane: lanes of a warp never meet, only warps do, and rarely at
        // the same moment.  The stripes are summed once the slice is scanned.  (Measured, 8 rows of 151,936 scores,
        // top-p alone: one word a bin with a few bins held back in registers 214 us a draw, stripes 95 us.)
        scan_slice<4>(c, [&](int id, float s, bool ok) {
            if (!ok) return;
            const uint32_t b = order_bits(s);
            if ((b & mask) != prefix) return;
            const float w = expf((s - best_score) / temp);
            const bool in = LEVEL == 1 ? in_kept(sets, id, b) : in_nucleus(sets, id, b, w);
            if (!in) return;
            const int bin = (b >> shift) & 255u;
            if (shift == 0) atomicMin(&sh.min_id[bin], id);
            const int at = bin * 32 + (threadIdx.x & 31);
            atomicAdd(&count_stripes[at], 1u);
            atomicAdd(&c.stripes[at], (double)w);
        });
        __syncthreads();
        if (threadIdx.x < 256) {
            double sum = 0.0;
            unsigned n = 0;
#pragma unroll 8
            for (int j = 0; j < 32; ++j) {           // lanes start apart: no bank is met twice
                const int at = threadIdx.x * 32 + ((j + threadIdx.x) & 31);
                sum += c.stripes[at];
                n += count_stripes[at];
            }
            if (n) {
                lead_add(&sh.gcount[threadIdx.x], n);
                lead_add(&sh.gweight[threadIdx.x], sum);
                if (shift == 0) lead_min(&sh.gmin_id[threadIdx.x], sh.min_id[threadIdx.x]);
            }
        }
        leader_turn(c, [&] {
            if (threadIdx.x < 32) {
                const int lane = threadIdx.x;
                auto amount = [&](int i) { return sh.gcount[i] ? sh.gweight[i] : 0.0; };
                double all = 0.0;                    // this round's bins together
#pragma unroll
                for (int b = 0; b < 8; ++b) all += amount(lane * 8 + b);
                for (int o = 16; o > 0; o >>= 1) all += __shfl_xor_sync(0xffffffffu, all, o);
                double goal_now = goal;
                if (shift == 24) {
                    goal_now = fraction * all;
                    if (lane == 0) sh.f64[2] = goal_now;
                }
                double acc = above;
                int bin = find_bin<double>(amount, above,
                                           [&](double before, double after) {
                                               return after > before && (strict ? (goal_now < after) : (after >= goal_now));
                                           }, acc);
                if (bin < 0) {
                    // Rounding left the goal just out of reach (or nothing weighs anything): stop at the last tokens,
                    // the lowest bin that holds any.
                    unsigned holds = 0;
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (sh.gcount[lane * 8 + b]) holds |= 1u << b;
                    const unsigned lanes = __ballot_sync(0xffffffffu, holds != 0);
                    if (!lanes) {
                        bin = 0;
                        acc = above;
                    } else {
                        const int owner = __ffs(lanes) - 1;
                        bin = owner * 8 + __ffs(__shfl_sync(0xffffffffu, holds, owner)) - 1;
                        acc = above + all - amount(bin);
                    }
                }
                if (lane == 0) {
                    sh.u32[0] = (uint32_t)bin;
                    sh.f64[0] = acc;
                    sh.i32[0] = (int)sh.gcount[bin];
                    sh.i32[2] = sh.gmin_id[bin];
                }
            }
            __syncthreads();
            if (threadIdx.x < 256) { sh.gcount[threadIdx.x] = 0; sh.gweight[threadIdx.x] = 0.0; sh.gmin_id[threadIdx.x] = NO_ID; }
        });
        prefix |= lead_load(&sh.u32[0]) << shift;
        mask |= 255u << shift;
        above = lead_load(&sh.f64[0]);
        if (shift == 24) goal = lead_load(&sh.f64[2]);
        out_equal_count = lead_load(&sh.i32[0]);
    }
    out_bits = prefix;
    out_goal = goal;
    out_above = above;
    const int first = lead_load(&sh.i32[2]);
    out_first_id = first == NO_ID ? -1 : first;
}

// The best token: largest score, ties to the lowest id; a NaN only as the first token taking part
// (src/inference/sampler.hpp:88-132).  Every thread of the cluster returns the same id.
__device__ int best_token(const Row& c, int skip) {
    Shared& sh = *c.sh;
    const int first = skip == 0 ? 1 : 0;
    float bs = -INFINITY;
    int bi = first;
    scan_slice(c, [&](int id, float s, bool ok) {
        if (ok && id != skip && (s > bs || (s == bs && id < bi))) { bs = s; bi = id; }
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
        lead_store(&sh.part_score[c.rank], bs);
        lead_store(&sh.part_id[c.rank], bi);
    }
    leader_turn(c, [&] {
        if (threadIdx.x == 0) {
            float s = sh.part_score[0];
            int i = sh.part_id[0];
            for (uint32_t b = 1; b < c.blocks; ++b)
                if (sh.part_score[b] > s || (sh.part_score[b] == s && sh.part_id[b] < i)) { s = sh.part_score[b]; i = sh.part_id[b]; }
            if (isnan(c.row[first])) i = first;
            sh.i32[1] = i;
        }
    });
    return lead_load(&sh.i32[1]);
}

__device__ __forceinline__ Row row_of_block(const float* logits, int vocab, Shared* sh, double* stripes) {
    Row c;
    c.row = logits + (size_t)blockIdx.y * vocab;
    c.n = vocab;
    c.rank = cluster_rank();
    c.blocks = cluster_blocks();
    const int per = (((vocab + (int)c.blocks - 1) / (int)c.blocks) + 3) & ~3;      // slices begin at multiples of four
    c.lo = min(vocab, (int)c.rank * per);
    c.hi = min(vocab, c.lo + per);
    c.sh = sh;
    c.stripes = stripes;
    return c;
}

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int vocab,
                                                         const RowParams* __restrict__ params, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ Shared sh;
    extern __shared__ double stripes[];       // STRIPES_BYTES
    const Row c = row_of_block(logits, vocab, &sh, stripes);
    const float* row = c.row;
    const RowParams p = params[blockIdx.y];
    const int n = vocab;
    // What the blocks meet in starts empty (only the leader's copy is ever used).
    for (int i = threadIdx.x; i < 256; i += THREADS) { sh.gcount[i] = 0; sh.gweight[i] = 0.0; sh.gmin_id[i] = NO_ID; }
    if (threadIdx.x == 0) { sh.n_hits = 0; sh.n_kept = 0; sh.walked = -1; }
    __syncthreads();
    cluster_sync();

    Sets sets;
    sets.skip = (p.masked >= 0 && p.masked < n && n > 1) ? p.masked : -1;
    sets.has_topk = sets.has_nucleus = sets.has_minp = false;
    sets.topk_bits = sets.nuc_bits = 0;
    sets.topk_last_id = sets.nuc_last_id = n;
    sets.min_p = 0.0f;

    const int best = best_token(c, sets.skip);
    const float best_score = row[best];
    sets.best = best;
    if (!(p.temperature > 0.0f)) {
        if (c.rank == 0 && threadIdx.x == 0) out[blockIdx.y] = best;
        cluster_sync();          // the other blocks have read the best token from the leader
        return;
    }
    const float temp = p.temperature;
    const int m = sets.skip >= 0 ? n - 1 : n;
    const int keep = (p.top_k > 0 && p.top_k < m) ? p.top_k : m;

    // ---- top-k: the bits of the k-th best and the last id taken among its ties
    if (keep < m) {
        uint32_t bits;
        int taken, first;
        select_by_count(c, keep, sets, bits, taken, first);
        const int last = taken == 1 ? first : nth_with_bits<0>(c, bits, taken - 1, sets, best_score, temp);
        sets.has_topk = true;
        sets.topk_bits = bits;
        sets.topk_last_id = last < 0 ? n : last;
    }

    if (sets.has_topk && keep <= KMAX) {
        // ---- the kept tokens fit shared memory: gather them in the leader's, put them in the order of the walk (ids
        // ascending without top-p, best first with it), and let one thread walk them as the reference's sampler does.
        // (each block lists its own first, in the lists that the leader orders them into later, then takes room for
        // all of them in the leader's lists at once: a thousand single additions to one counter of another block's
        // shared memory would take longer than everything else)
        __shared__ int n_mine, my_base;
        if (threadIdx.x == 0) n_mine = 0;
        __syncthreads();
        scan_slice(c, [&](int id, float s, bool ok) {
            if (!ok) return;
            const uint32_t b = order_bits(s);
            if (!in_kept(sets, id, b)) return;
            const int slot = atomicAdd(&n_mine, 1);
            if (slot < KMAX) {
                sh.o_id[slot] = id;
                sh.l_bits[slot] = b;
                sh.o_w[slot] = expf((s - best_score) / temp);
            }
        });
        __syncthreads();
        const int mine = min(n_mine, KMAX);
        if (threadIdx.x == 0) my_base = lead_reserve(&sh.n_kept, mine);
        __syncthreads();
        for (int i = threadIdx.x; i < mine; i += THREADS) {
            const int slot = my_base + i;
            if (slot < KMAX) {
                lead_store(&sh.c_id[slot], sh.o_id[i]);
                lead_store(&sh.c_bits[slot], sh.l_bits[i]);
                lead_store(&sh.c_w[slot], sh.o_w[i]);
            }
        }
        cluster_sync();
        if (c.rank != 0) return;
        const int K = min(sh.n_kept, KMAX);
        const bool ranked = p.top_p < 1.0f;
        for (int i = threadIdx.x; i < K; i += THREADS) {
            const int id = sh.c_id[i];
            const uint32_t b = sh.c_bits[i];
            int before = 0;
            for (int j = 0; j < K; ++j) {
                const bool first_j = ranked ? (sh.c_bits[j] > b || (sh.c_bits[j] == b && sh.c_id[j] < id)) : sh.c_id[j] < id;
                before += first_j ? 1 : 0;
            }
            sh.o_id[before] = id;
            sh.o_w[before] = sh.c_w[i];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const int* o_id = sh.o_id;
            const float* o_w = sh.o_w;
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
            out[blockIdx.y] = pick;
        }
        return;
    }

    int chosen = best;
    if (p.top_p >= 1.0f) {
        // ---- id order over the whole vocabulary: every thread of the cluster owns a run of consecutive ids; the runs'
        // weights are scanned (within the block, then over the blocks), one thread walks its run
        const float cut = p.min_p > 0.0f ? p.min_p : 0.0f;
        const int owners = (int)c.blocks * THREADS;
        const int seg = (n + owners - 1) / owners;
        const int lo = min(n, ((int)c.rank * THREADS + (int)threadIdx.x) * seg), hi = min(n, lo + seg);
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
            lead_store(&sh.part_total[c.rank], acc);
        }
        __syncthreads();
        cluster_sync();
        double before = sh.scan[threadIdx.x], total = 0.0;
        for (uint32_t b = 0; b < c.blocks; ++b) {
            const double t = lead_load(&sh.part_total[b]);
            if (b < c.rank) before += t;
            total += t;
        }
        const double target = (double)p.r * total;
        if (target >= before && target < before + mine) {
            double acc = before;
            for (int id = lo; id < hi; ++id) {
                const float s = row[id];
                if (!in_kept(sets, id, order_bits(s))) continue;
                float w = expf((s - best_score) / temp);
                if (w < cut) w = 0.0f;
                acc += (double)w;
                if (target < acc) { lead_store(&sh.walked, id); break; }
            }
        }
        cluster_sync();
        if (c.rank == 0 && threadIdx.x == 0) out[blockIdx.y] = sh.walked >= 0 ? sh.walked : best;
        return;
    }
    // ---- rank order over the whole vocabulary: nucleus by weight, min-p on its tail, then the draw best first
    uint32_t bits;
    double goal, above;
    int equal, first;
    select_by_weight<1>(c, (double)p.top_p, false, sets, best_score, temp, bits, goal, above, equal, first);
    {
        // Tokens with the threshold's bits all weigh the same; take as many as reach the goal (at least one).
        const float s_t = __uint_as_float((bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits);
        const double w_t = (double)expf((s_t - best_score) / temp);
        long long j = 1;
        if (w_t > 0.0 && above + w_t < goal) j = (long long)ceil((goal - above) / w_t);
        if (j < 1) j = 1;
        if (j > equal) j = equal;
        const int last = j == 1 ? first : nth_with_bits<1>(c, bits, (int)j - 1, sets, best_score, temp);
        sets.has_nucleus = true;
        sets.nuc_bits = bits;
        sets.nuc_last_id = last < 0 ? n : last;
    }
    if (p.min_p > 0.0f) { sets.has_minp = true; sets.min_p = p.min_p; }
    double target;
    select_by_weight<2>(c, (double)p.r, true, sets, best_score, temp, bits, target, above, equal, first);
    {
        const float s_t = __uint_as_float((bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits);
        const double w_t = (double)expf((s_t - best_score) / temp);
        long long i = 0;
        if (w_t > 0.0 && target > above) i = (long long)floor((target - above) / w_t);
        if (i >= equal) i = equal - 1;
        if (i < 0) i = 0;
        const int id = i == 0 ? first : nth_with_bits<2>(c, bits, (int)i, sets, best_score, temp);
        if (id >= 0) chosen = id;
    }
    if (c.rank == 0 && threadIdx.x == 0) out[blockIdx.y] = chosen;
    cluster_sync();              // the other blocks have read the last decision from the leader
}

// Greedy rows only: the best token of every row.  Used when no row of the batch draws.
__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int vocab,
                                                         const RowParams* __restrict__ params, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ Shared sh;
    const Row c = row_of_block(logits, vocab, &sh, nullptr);
    const int masked = params[blockIdx.y].masked;
    const int skip = (masked >= 0 && masked < vocab && vocab > 1) ? masked : -1;
    const int best = best_token(c, skip);
    if (c.rank == 0 && threadIdx.x == 0) out[blockIdx.y] = best;
    cluster_sync();              // the other blocks have read the best token from the leader
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

// A row's blocks: one for a small vocabulary, up to eight (a portable cluster) for a large one -- but no more than let
// all rows run at the same time (one block of 1,024 threads an SM; 15 clusters of eight, 35 of four, 74 of two on 148
// SMs): a second round of clusters costs more than the wider scan saves.  Measured at 151,936 scores, top-k 40 with
// top-p / top-p alone, us a draw: 16 rows 79 / 171 with eight blocks, 72 / 124 with four; 64 rows 166 / 408 with
// eight, 116 / 204 with two; 128 rows 280 / 726 with eight, 177 / 342 with one.
int blocks_for(int vocab, int rows) {
    int blocks = vocab >= 65536 ? 8 : vocab >= 16384 ? 4 : vocab >= 8192 ? 2 : 1;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    while (blocks > 1 && (long long)rows * blocks > (blocks == 8 ? sms * 13 / 16 : blocks == 4 ? sms * 15 / 16 : sms)) blocks >>= 1;
    return blocks;
}

template <typename K>
int launch_rows(K kernel, int dynamic_bytes, int rows, int vocab, const float* logits, const RowParams* params, int* out,
                cudaStream_t stream) {
    const int blocks = blocks_for(vocab, rows);
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)blocks, (unsigned)rows, 1);
    lc.blockDim = dim3(THREADS);
    lc.dynamicSmemBytes = (size_t)dynamic_bytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)blocks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = llmx_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&lc, kernel, logits, vocab, params, out);
    return launch_status();
}

}  // namespace

// params: rows x {temperature, top_p, min_p, r, top_k, masked} (24 bytes each) on the device.
// `all_greedy` != 0: every row has temperature <= 0 (the caller knows); the argmax kernel alone runs.
LLMX_EXPORT int llmx_sample(const float* logits, int rows, int vocab, const void* params, int* out, int all_greedy,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535) return LLMX_ERR_BAD_ARGUMENT;
    if (all_greedy) return launch_rows(argmax_kernel, 0, rows, vocab, logits, (const RowParams*)params, out, stream);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STRIPES_BYTES) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    return launch_rows(sample_kernel, STRIPES_BYTES, rows, vocab, logits, (const RowParams*)params, out, stream);
}

LLMX_EXPORT int llmx_penalize(float* logits, int vocab, const int* row_of, const int* token, const int* count,
                              const float* repetition, const float* presence, const float* frequency, int items,
                              cudaStream_t stream) {
    if (items <= 0) return 0;
    launch_kernel(penalty_kernel, dim3((items + 255) / 256), dim3(256), 0, stream, logits, vocab, row_of, token, count,
                  repetition, presence, frequency, items);
    return launch_status();
}
