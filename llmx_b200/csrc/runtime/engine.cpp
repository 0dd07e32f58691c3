// The native engine (see llmx_engine.h): cache bookkeeping, step metadata, scheduler, sampling state, all host code
// around the model runtime's forward pass.  The files a model is loaded from are read in loader.cpp.
#include "engine_internal.h"

#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <deque>
#include <map>
#include <set>

namespace llmx_engine_detail {

thread_local std::string g_error;
thread_local int g_code = 0;
int fail(int code, const std::string& what) {
    g_error = what;
    g_code = code;
    return code;
}

static void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw Failure{LLMX_ENGINE_ERR_DEVICE, std::string(what) + ": " + cudaGetErrorString(e)};
}

// ---------------------------------------------------------------------------------------------------------------
// Pages: a pool of page ids and one request's block table over it.  The protocol is the reference's
// (src/model/kv_cache.hpp:14-67 the pool, :71-179 a sequence): pages for a step are prepared before the step writes,
// committed once the whole step is enqueued, aborted when it fails, which returns exactly what the failed step took.
// A table of a group that keeps a window gives back the pages the window has passed at every commit.
// ---------------------------------------------------------------------------------------------------------------
PagePool::PagePool(long long pages) : refs_((size_t)std::max(pages, 0ll), 0) {
    for (long long p = (long long)refs_.size() - 1; p >= 0; --p) free_.push_back((int)p);     // lowest ids first
}
int PagePool::alloc() {
    if (free_.empty())
        throw Failure{LLMX_ENGINE_ERR_CACHE, "KV cache: all " + std::to_string(refs_.size()) +
                                                 " pages are in use; the run needs more tokens than the cache was made for"};
    const int page = free_.back();
    free_.pop_back();
    refs_[page] = 1;
    return page;
}
void PagePool::release(int page) {
    if (page < 0 || page >= (int)refs_.size() || refs_[page] == 0)
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "KV cache: page " + std::to_string(page) + " released twice"};
    if (--refs_[page] == 0) free_.push_back(page);
}
std::string PagePool::check() const {
    std::set<int> seen(free_.begin(), free_.end());
    if (seen.size() != free_.size()) return "a page is on the free list twice";
    for (int p = 0; p < (int)refs_.size(); ++p)
        if ((refs_[p] == 0) != (seen.count(p) > 0)) return "page " + std::to_string(p) + " is neither free nor held, or both";
    return "";
}

void BlockTable::prepare(int n) {
    if (pending) throw Failure{LLMX_ENGINE_ERR_REFUSED, "KV cache: a step is already in progress for this request"};
    const int need = pages_for(length + n);
    int taken = 0;
    try {
        while ((int)pages.size() < need) {
            pages.push_back(pool->alloc());
            ++taken;
        }
    } catch (const Failure&) {
        for (; taken > 0; --taken) {
            pool->release(pages.back());
            pages.pop_back();
        }
        throw;
    }
    pending = n;
}
void BlockTable::commit() {
    length += pending;
    pending = 0;
    if (window <= 0) return;
    const int lowest_needed = length - window + 1;
    if (lowest_needed <= 0) return;
    const int upto = std::min(lowest_needed / page_size, (int)pages.size());
    for (int i = first_live; i < upto; ++i) {
        pool->release(pages[i]);
        pages[i] = -1;
    }
    first_live = std::max(first_live, upto);
}
void BlockTable::shrink_to(int tokens) {
    const int keep = std::max(pages_for(tokens), first_live);
    while ((int)pages.size() > keep) {
        pool->release(pages.back());
        pages.pop_back();
    }
}
void BlockTable::abort() {
    shrink_to(length);
    pending = 0;
}
void BlockTable::truncate(int to) {
    length = std::min(length, to);
    pending = 0;
    shrink_to(length);
}
void BlockTable::free() {
    for (int i = first_live; i < (int)pages.size(); ++i) pool->release(pages[i]);
    pages.clear();
    length = pending = first_live = 0;
}

int StateSlots::take() {
    if (free_.empty()) throw Failure{LLMX_ENGINE_ERR_CACHE, "state slots: all " + std::to_string(held_.size()) + " are in use"};
    const int s = free_.back();
    free_.pop_back();
    held_[s] = true;
    return s;
}
void StateSlots::give_back(int s) {
    if (s < 0 || s >= (int)held_.size() || !held_[s])
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "state slot " + std::to_string(s) + " given back twice"};
    held_[s] = false;
    free_.push_back(s);
}

// ---------------------------------------------------------------------------------------------------------------
// The cache manager.  Entries with the same needs (kv heads, head width, window) form a group: one pool, one block
// table per request, page id p naming the same page in every member's storage
// [pages, 2, kv_heads, page_size, head_dim].  Groups with different needs have pools of their own, so a windowed
// group gives pages back while a full one keeps them.  State entries own [slots, bytes]; a live request holds two
// slots, the one its state lies in and a spare that a step writes; commit swaps them, so a failed step leaves the
// state as it was (the reference keeps checkpoints of its state slots to the same end, src/model/kv_cache.hpp:183-278).
// ---------------------------------------------------------------------------------------------------------------
Cache::Cache(const llmx_engine_desc& d, bool books_only) : page_size(d.page_size), max_requests(d.max_requests), kv_dtype(d.kv_dtype) {
    if (page_size <= 0) throw Failure{LLMX_ENGINE_ERR_REFUSED, "page_size must be positive"};
    entries.assign(d.entries, d.entries + d.n_entries);
    const long long window_tokens = d.window_kv_tokens > 0 ? d.window_kv_tokens : d.kv_tokens;
    entry_group.assign(entries.size(), -1);
    entry_member.assign(entries.size(), -1);
    bool has_state = false;
    for (size_t i = 0; i < entries.size(); ++i) {
        const llmx_cache_entry_desc& e = entries[i];
        if (e.kind == 2) has_state = true;
        if (e.kind != 1) continue;
        int g = -1;
        for (size_t k = 0; k < groups.size(); ++k)
            if (groups[k].kv_heads == e.kv_heads && groups[k].head_dim == e.head_dim && groups[k].window == e.window) g = (int)k;
        if (g < 0) {
            g = (int)groups.size();
            groups.emplace_back(e.kv_heads, e.head_dim, e.window, page_size, (e.window > 0 ? window_tokens : d.kv_tokens) / page_size);
        }
        entry_group[i] = g;
        entry_member[i] = (int)groups[g].members.size();
        groups[g].members.push_back((int)i);
    }
    if ((int)groups.size() > LLMX_MAX_GROUPS)
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "a model may have " + std::to_string(LLMX_MAX_GROUPS) + " cache groups at most"};
    slots = StateSlots(has_state ? 2 * max_requests : 0);
    state_storage.assign(entries.size(), nullptr);
    if (books_only) return;
    // Storage, zero-filled: a kernel may load (and mask) slots of a page that were never written.
    views = llmx_caches_create((int)entries.size());
    const size_t elem = kv_dtype == LLMX_DT_BF16 ? 2 : 4;
    for (size_t g = 0; g < groups.size(); ++g) {
        Group& gr = groups[g];
        gr.member_bytes = (size_t)gr.pool.pages() * 2 * gr.kv_heads * page_size * gr.head_dim * elem;
        const size_t bytes = std::max<size_t>(gr.member_bytes * gr.members.size(), 256);
        cuda_check(cudaMalloc(&gr.storage, bytes), "allocating the cache");
        cuda_check(cudaMemset(gr.storage, 0, bytes), "clearing the cache");
        for (size_t m = 0; m < gr.members.size(); ++m)
            if (llmx_caches_set_kv(views, gr.members[m], (int)g, (char*)gr.storage + m * gr.member_bytes, kv_dtype, gr.pool.pages(),
                                   gr.kv_heads, page_size, gr.head_dim))
                throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("cache entry: ") + llmx_rt_last_error()};
    }
    for (size_t i = 0; i < entries.size(); ++i) {
        if (entries[i].kind != 2) continue;
        const size_t bytes = std::max<size_t>((size_t)slots.count() * (size_t)entries[i].state_bytes, 256);
        cuda_check(cudaMalloc(&state_storage[i], bytes), "allocating state slots");
        cuda_check(cudaMemset(state_storage[i], 0, bytes), "clearing state slots");
        if (llmx_caches_set_state(views, (int)i, state_storage[i], slots.count(), entries[i].state_bytes))
            throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("cache entry: ") + llmx_rt_last_error()};
    }
}
Cache::~Cache() {
    if (views) llmx_caches_destroy(views);
    for (Group& g : groups)
        if (g.storage) cudaFree(g.storage);
    for (void* s : state_storage)
        if (s) cudaFree(s);
}
RequestCache& Cache::new_request(long long id) {
    if (live.count(id)) throw Failure{LLMX_ENGINE_ERR_REFUSED, "request " + std::to_string(id) + " is already live"};
    RequestCache rc;
    for (Group& g : groups) rc.tables.emplace_back(&g.pool, page_size, g.window);
    if (slots.count()) {
        rc.state_slot = slots.take();
        try {
            rc.state_slot_out = slots.take();
        } catch (const Failure&) {
            slots.give_back(rc.state_slot);
            throw;
        }
    }
    return live.emplace(id, std::move(rc)).first->second;
}
void Cache::free_request(long long id) {
    auto it = live.find(id);
    if (it == live.end()) return;
    RequestCache& rc = it->second;
    for (BlockTable& t : rc.tables) t.free();
    if (rc.state_slot >= 0) slots.give_back(rc.state_slot);
    if (rc.state_slot_out >= 0) slots.give_back(rc.state_slot_out);
    live.erase(it);
}
void RequestCache::prepare(int n) {
    size_t done = 0;
    try {
        for (; done < tables.size(); ++done) tables[done].prepare(n);
    } catch (const Failure&) {
        for (size_t i = 0; i < done; ++i) tables[i].abort();
        throw;
    }
    pending = n;
}
void RequestCache::commit() {
    for (BlockTable& t : tables) t.commit();
    if (pending) std::swap(state_slot, state_slot_out);
    length += pending;
    pending = 0;
}
void RequestCache::abort() {
    for (BlockTable& t : tables) t.abort();
    pending = 0;
}
void RequestCache::truncate(int to) {
    if (pending) throw Failure{LLMX_ENGINE_ERR_REFUSED, "KV cache: a step is in progress for this request"};
    if (to < 0 || to > length)
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "cannot truncate a request of " + std::to_string(length) + " tokens to " + std::to_string(to)};
    if (to == length) return;
    if (state_slot >= 0) throw Failure{LLMX_ENGINE_ERR_REFUSED, "a request whose layers keep fixed-size state cannot be rolled back"};
    for (const BlockTable& t : tables)
        if (t.window > 0 && to < t.first_live * t.page_size)
            throw Failure{LLMX_ENGINE_ERR_REFUSED, "KV cache: cannot roll back into pages the window has given back"};
    for (BlockTable& t : tables) t.truncate(to);
    length = to;
}
// Pages a request of `tokens` positions holds at most, per group: a windowed group holds its window, the page the
// window starts in and the portion being written, never more than the whole history.
std::vector<long long> Cache::pages_needed(long long tokens, long long step_tokens) const {
    std::vector<long long> out;
    for (const Group& g : groups) {
        long long held = tokens;
        if (g.window > 0) held = std::min(tokens, (long long)g.window + page_size + std::max(step_tokens, 1ll) + page_size);
        out.push_back((held + page_size - 1) / page_size);
    }
    return out;
}
std::string Cache::check() const {
    for (size_t g = 0; g < groups.size(); ++g) {
        const std::string bad = groups[g].pool.check();
        if (!bad.empty()) return "group " + std::to_string(g) + ": " + bad;
        std::map<int, int> held;
        for (const auto& kv : live) {
            const BlockTable& t = kv.second.tables[g];
            for (int i = t.first_live; i < (int)t.pages.size(); ++i) ++held[t.pages[i]];
        }
        for (int p = 0; p < groups[g].pool.pages(); ++p) {
            const auto it = held.find(p);
            const int n = it == held.end() ? 0 : it->second;
            if (groups[g].pool.refs(p) != n)
                return "group " + std::to_string(g) + " page " + std::to_string(p) + ": the pool counts " +
                       std::to_string(groups[g].pool.refs(p)) + " holders, requests hold " + std::to_string(n);
        }
    }
    return slots.check();
}
std::string StateSlots::check() const {
    std::set<int> seen(free_.begin(), free_.end());
    if (seen.size() != free_.size()) return "a state slot is free twice";
    for (int s = 0; s < (int)held_.size(); ++s)
        if (held_[s] == (seen.count(s) > 0)) return "state slot " + std::to_string(s) + " is both held and free, or neither";
    return "";
}

// ---------------------------------------------------------------------------------------------------------------
// The scheduler: which requests run in the next step, and with which tokens.  Pure bookkeeping.  The policy follows the
// reference's server scheduler (docs/SERVER.md:46-58, :136-243; src/server/policy.hpp:153-158, :207-256):
//   admission    first come, first served; at most max_requests running; a request is admitted when every cache group
//                can hold what it reserves; admission stops at the first request that does not fit (no overtaking).
//   reservation  full: prompt + max_tokens, so a running request never runs out of pages; prompt only: the prompt and
//                a page of growth, and when pages then run out while decoding,
//   pages out    the request admitted last is paused: its pages are given back and it returns to the head of the line,
//                to recompute its prompt and what it has generated when it is admitted again (its sampling state is
//                kept, so its reply continues as if nothing had happened).  A request that cannot fit even alone ends
//                with reason "cache".
//   a step       decoding requests first, one token each; then portions of prompts, in admission order, until the
//                step's token budget is spent; the portion that ends a prompt wants logits.
//   finishing    a drawn end-of-sequence id ends the reply (the id is not part of it) unless ignore_eos; reaching
//                max_tokens ends it with reason "length".
// ---------------------------------------------------------------------------------------------------------------
void Scheduler::add(const std::shared_ptr<Request>& r) {
    if (r->prompt.empty()) throw Failure{LLMX_ENGINE_ERR_REFUSED, "generate: empty prompt"};
    if ((long long)r->prompt.size() + r->params.max_tokens > max_positions)
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "request " + std::to_string(r->id) + ": prompt of " + std::to_string(r->prompt.size()) +
                                                   " tokens plus max_tokens " + std::to_string(r->params.max_tokens) +
                                                   " exceeds the context length of " + std::to_string(max_positions)};
    const std::vector<long long> alone = cache->pages_needed((long long)r->prompt.size() + r->params.max_tokens, max_batch_tokens);
    for (size_t g = 0; g < alone.size(); ++g)
        if (alone[g] > cache->groups[g].pool.pages())
            throw Failure{LLMX_ENGINE_ERR_REFUSED, "request " + std::to_string(r->id) + " needs " + std::to_string(alone[g]) +
                                                       " pages of group " + std::to_string(g) + "; the cache has " +
                                                       std::to_string(cache->groups[g].pool.pages())};
    if (max_queue > 0 && (int)waiting.size() >= max_queue) throw Failure{LLMX_ENGINE_ERR_REFUSED, "the queue is full"};
    waiting.push_back(r);
}
std::vector<long long> Scheduler::reservation(const Request& r) const {
    if (!reserve_prompt_only) return cache->pages_needed((long long)r.prompt.size() + r.params.max_tokens, max_batch_tokens);
    return cache->pages_needed((long long)r.tokens() + cache->page_size, max_batch_tokens);      // in hand plus a page of growth
}
bool Scheduler::fits(const std::vector<long long>& extra) const {
    for (size_t g = 0; g < extra.size(); ++g) {
        long long total = extra[g];
        for (const auto& kv : reserved) total += kv.second[g];
        if (total > cache->groups[g].pool.pages()) return false;
    }
    return true;
}
void Scheduler::admit() {
    while (!waiting.empty() && (int)running.size() < max_requests) {
        std::shared_ptr<Request> r = waiting.front();
        const std::vector<long long> need = reservation(*r);
        if (!fits(need)) break;                          // no overtaking
        waiting.pop_front();
        reserved[r->id] = need;
        r->state = Request::RUNNING;
        r->fed = 0;
        ++r->admissions;
        if (r->order < 0) r->order = admission++;
        running.push_back(r);
        std::stable_sort(running.begin(), running.end(), [](const auto& a, const auto& b) { return a->order < b->order; });
    }
}
void Scheduler::pause_latest() {
    auto it = std::max_element(running.begin(), running.end(), [](const auto& a, const auto& b) { return a->order < b->order; });
    std::shared_ptr<Request> victim = *it;
    running.erase(it);
    reserved.erase(victim->id);
    victim->state = Request::WAITING;
    victim->fed = 0;
    waiting.push_front(victim);
    to_release.push_back(victim->id);
    ++preemptions;
}
void Scheduler::finish(const std::shared_ptr<Request>& r, int reason) {
    r->state = Request::FINISHED;
    r->finished = reason;
    to_release.push_back(r->id);
}
// Under prompt-only reservation: every running request has room for its next tokens, or someone is paused.
void Scheduler::grow(std::vector<std::shared_ptr<Request>>& ended) {
    if (!reserve_prompt_only) return;
    while (!running.empty()) {
        std::shared_ptr<Request> short_one;
        for (const auto& r : running) {              // kept in admission order
            const std::vector<long long> want = cache->pages_needed(std::min<long long>(r->tokens() + 1, max_positions), max_batch_tokens);
            std::vector<long long>& have = reserved[r->id];
            bool lacks = false;
            for (size_t g = 0; g < want.size(); ++g) lacks = lacks || want[g] > have[g];
            if (!lacks) continue;
            const std::vector<long long> grown =
                cache->pages_needed(std::min<long long>(r->tokens() + cache->page_size, max_positions), max_batch_tokens);
            std::vector<long long> extra(grown.size());
            for (size_t g = 0; g < grown.size(); ++g) extra[g] = std::max(grown[g] - have[g], 0ll);
            if (fits(extra)) {
                for (size_t g = 0; g < grown.size(); ++g) have[g] = std::max(grown[g], have[g]);
            } else {
                short_one = r;
                break;
            }
        }
        if (!short_one) return;
        if (running.size() == 1) {                   // alone and still short: it can never go on
            std::shared_ptr<Request> r = running.back();
            running.pop_back();
            reserved.erase(r->id);
            finish(r, 3);
            ended.push_back(r);
            return;
        }
        pause_latest();
    }
}
std::vector<Planned> Scheduler::plan(std::vector<std::shared_ptr<Request>>& ended) {
    grow(ended);
    admit();
    std::vector<Planned> entries;
    long long budget = max_batch_tokens;
    for (const auto& r : running)                    // decoding requests first
        if (r->decoding() && budget > 0) {
            entries.push_back(Planned{r, {r->output.back()}, true});
            --budget;
        }
    for (const auto& r : running) {                  // then portions of prompts, in admission order
        if (r->decoding() || budget <= 0) continue;
        const long long total = r->tokens(), todo = total - r->fed;
        if (todo <= 0) continue;
        const long long n = std::min(todo, budget);
        Planned p{r, {}, n == todo};
        for (long long i = r->fed; i < r->fed + n; ++i) p.tokens.push_back(r->token_at(i));
        entries.push_back(std::move(p));
        budget -= n;
    }
    return entries;
}
// Books a step; `drawn[i]` is the token drawn for the i-th entry that wanted logits.  Returns the (request, token,
// finished) records of those entries.
std::vector<llmx_step_result> Scheduler::complete(const std::vector<Planned>& entries, const std::vector<int>& drawn) {
    std::vector<llmx_step_result> out;
    size_t k = 0;
    for (const Planned& e : entries) {
        Request& r = *e.request;
        r.fed += (long long)e.tokens.size();
        if (!e.want_last) continue;
        const int token = drawn[k++];
        bool stop = false;
        if (!r.params.ignore_eos) {
            stop = std::find(eos_ids.begin(), eos_ids.end(), token) != eos_ids.end() ||
                   std::find(r.stop_ids.begin(), r.stop_ids.end(), token) != r.stop_ids.end();
        }
        int reason = 0;
        if (stop) {
            reason = 1;
        } else {
            r.output.push_back(token);
            r.sampling.saw(token);
            if ((int)r.output.size() >= r.params.max_tokens) reason = 2;
        }
        if (reason) {
            running.erase(std::find(running.begin(), running.end(), e.request));
            reserved.erase(r.id);
            finish(e.request, reason);
        }
        out.push_back(llmx_step_result{r.id, stop ? -1 : token, reason});
    }
    return out;
}

// ---------------------------------------------------------------------------------------------------------------
// Sampling state: each request has its own xorshift64 generator (src/inference/sampler.hpp:21-32) seeded from its
// settings and its own count of the tokens it has generated.  A draw uses one uniform number of the request's
// generator, so what a request generates does not depend on what it was batched with.  The logits never leave the
// device: the kernels of sampling.cu pick the ids there and only those are copied back.
// ---------------------------------------------------------------------------------------------------------------
unsigned long long XorShift64::next() {
    unsigned long long x = state;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    return state = x;
}
float XorShift64::unit() { return (float)((double)(next() >> 40) * (1.0 / 16777216.0)); }

static void check_sampling(const llmx_sampling& p) {
    auto bad = [](const char* what) { throw Failure{LLMX_ENGINE_ERR_REFUSED, what}; };
    if (p.max_tokens < 1) bad("max_tokens must be an integer of at least 1");
    if (!std::isfinite(p.temp) || p.temp < 0) bad("temp must be a finite number of at least 0");
    if (p.top_k < 0) bad("top_k must be an integer of at least 0");
    if (!std::isfinite(p.top_p) || p.top_p < 0 || p.top_p > 1) bad("top_p must lie in 0..1");
    if (!std::isfinite(p.min_p) || p.min_p < 0 || p.min_p > 1) bad("min_p must lie in 0..1");
    if (!std::isfinite(p.penalty) || p.penalty < 1) bad("penalty must be at least 1");
    if (!std::isfinite(p.presence_penalty) || p.presence_penalty < -2 || p.presence_penalty > 2) bad("presence_penalty must lie in -2..2");
    if (!std::isfinite(p.frequency_penalty) || p.frequency_penalty < -2 || p.frequency_penalty > 2) bad("frequency_penalty must lie in -2..2");
    if (p.n_stop < 0 || (p.n_stop > 0 && !p.stop_ids)) bad("stop_ids: a count and no ids");
}

// ---------------------------------------------------------------------------------------------------------------
// The engine.
// ---------------------------------------------------------------------------------------------------------------
void DeviceBuffer::ensure(size_t want, cudaStream_t stream) {
    if (want <= bytes) return;
    if (ptr) {
        cuda_check(cudaStreamSynchronize(stream), "waiting before a buffer grows");
        cudaFree(ptr);
        ptr = nullptr;
        bytes = 0;
    }
    const size_t size = std::max<size_t>((want + (want >> 2) + 255) & ~size_t(255), 4096);
    cuda_check(cudaMalloc(&ptr, size), "allocating a device buffer");
    bytes = size;
}
DeviceBuffer::~DeviceBuffer() {
    if (ptr) cudaFree(ptr);
}

}  // namespace llmx_engine_detail

using namespace llmx_engine_detail;

llmx_engine::llmx_engine(llmx_model* m, const llmx_engine_desc& d, std::unique_ptr<LoadedModel> own)
    : owned(std::move(own)), model(m), vocab(d.vocab), max_positions(d.max_positions),
      position_streams(std::max(d.position_streams, 1)), device(d.device), books_only(m == nullptr && d.device < 0) {
    if (!model && !books_only) throw Failure{LLMX_ENGINE_ERR_REFUSED, "an engine needs a model"};
    if (d.vocab <= 0 || d.max_positions <= 0 || d.max_requests <= 0 || d.n_entries < 0 || d.kv_tokens < 0)
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "an engine needs a vocabulary, a context length and room for at least one request"};
    if (d.kv_dtype != LLMX_DT_BF16 && d.kv_dtype != LLMX_DT_F32) throw Failure{LLMX_ENGINE_ERR_REFUSED, "the cache holds bfloat16 or float32"};
    if (!books_only) {
        cuda_check(cudaSetDevice(device), "choosing the device");
        cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "creating the engine's stream");
    }
    cache.reset(new Cache(d, books_only));
    sched.cache = cache.get();
    sched.max_positions = max_positions;
    sched.max_batch_tokens = d.max_batch_tokens > 0 ? d.max_batch_tokens : 2048;
    sched.max_requests = d.max_requests;
    sched.max_queue = d.max_queue;
    sched.reserve_prompt_only = d.reserve_prompt_only != 0;
    sched.eos_ids.assign(d.eos_ids, d.eos_ids + (d.eos_ids ? d.n_eos : 0));
    if (books_only) return;
    cuda_check(cudaMalloc(&error_word, sizeof(int)), "allocating the error word");
    cuda_check(cudaMemset(error_word, 0, sizeof(int)), "clearing the error word");
    cuda_check(cudaMalloc(&counters, LLMX_COUNTERS * sizeof(int)), "allocating the counters");
    cuda_check(cudaMemset(counters, 0, LLMX_COUNTERS * sizeof(int)), "clearing the counters");
    for (Pinned& p : ring) cuda_check(cudaEventCreateWithFlags(&p.done, cudaEventDisableTiming), "creating an event");
}
llmx_engine::~llmx_engine() {
    if (books_only) return;
    if (stream) cudaStreamSynchronize(stream);
    for (Pinned& p : ring) {
        if (p.host) cudaFreeHost(p.host);
        if (p.done) cudaEventDestroy(p.done);
    }
    recordings.clear();
    if (error_word) cudaFree(error_word);
    if (counters) cudaFree(counters);
    cache.reset();
    if (host_ids) cudaFreeHost(host_ids);
    if (sample_host) cudaFreeHost(sample_host);
    if (stream) cudaStreamDestroy(stream);
}

int* llmx_engine::pinned(size_t ints) {
    ring_at = (ring_at + 1) % (int)(sizeof ring / sizeof ring[0]);
    Pinned& p = ring[ring_at];
    if (p.used) cuda_check(cudaEventSynchronize(p.done), "waiting for a step's metadata copy");
    if (p.ints < ints) {
        if (p.host) cudaFreeHost(p.host);
        p.host = nullptr;
        const size_t n = std::max<size_t>(ints + (ints >> 1), 4096);
        cuda_check(cudaMallocHost((void**)&p.host, n * sizeof(int)), "allocating pinned memory");
        p.ints = n;
    }
    return p.host;
}

void llmx_engine::sync_and_check() {
    int word = 0;
    cuda_check(cudaMemcpyAsync(&word, error_word, sizeof(int), cudaMemcpyDeviceToHost, stream), "reading the error word");
    cuda_check(cudaStreamSynchronize(stream), "waiting for the step");
    if (word) {
        cudaMemsetAsync(error_word, 0, sizeof(int), stream);
        throw Failure{LLMX_ENGINE_ERR_DEVICE, "a kernel gave up a bounded wait (code " + std::to_string(word) + ")"};
    }
}

// Where a step's metadata lies in its one int32 buffer (sections padded to 16 bytes): token ids [rows], positions
// [streams, rows], the request of each row, first row / row count / history / state slots read of each request, the rows
// whose logits are wanted, state slots written, then for every cache group its block tables [requests, max_pages] and the
// rows' cache slots, then the ints of the launch plan.  Fills the offsets of `s`; returns the total.
size_t llmx_engine::layout(llmx_step& s, const std::vector<int>& counts, int wanted, const std::vector<int>& max_pages, int plan_ints) const {
    const int n_req = (int)counts.size(), n_groups = (int)cache->groups.size();
    int rows = 0;
    for (int c : counts) rows += c;
    size_t at = 0;
    auto section = [&](size_t n) {
        const size_t off = at;
        at += (std::max<size_t>(n, 1) + 3) & ~size_t(3);
        return (int)off;
    };
    s.rows = rows, s.requests = n_req, s.wanted = wanted, s.groups = n_groups, s.position_streams = position_streams;
    s.token_ids = section(rows);
    s.positions = section((size_t)position_streams * rows);
    s.row_request = section(rows);
    s.row_start = section(n_req);
    s.row_count = section(n_req);
    s.history = section(n_req);
    s.state_slots = section(n_req);
    s.logit_rows = section(wanted);
    s.state_slots_out = section(n_req);
    for (int g = 0; g < n_groups; ++g) {
        s.block_tables[g] = section((size_t)n_req * max_pages[g]);
        s.table_stride[g] = max_pages[g];
        s.slots[g] = section(rows);
        s.page_size[g] = cache->page_size;
    }
    s.plan_offset = section(plan_ints);
    s.caches = cache->views;
    s.error_word = error_word;
    s.counters = counters;
    s.stream = stream;
    return at;
}

void llmx_engine::fill_meta(int* buf, const llmx_step& s, size_t total, const std::vector<Batch>& batch,
                            const std::vector<RequestCache*>& caches, const std::vector<int>& histories) const {
    memset(buf, 0, total * sizeof(int));
    const int n_groups = (int)cache->groups.size(), rows = s.rows, ps = cache->page_size;
    int k = 0, a = 0;
    for (int r = 0; r < s.requests; ++r) {
        const int n = (int)batch[r].tokens.size();
        for (int i = 0; i < n; ++i) {
            buf[s.token_ids + a + i] = batch[r].tokens[i];
            for (int st = 0; st < position_streams; ++st) buf[s.positions + (size_t)st * rows + a + i] = histories[r] + i;
            buf[s.row_request + a + i] = r;
        }
        buf[s.row_start + r] = a;
        buf[s.row_count + r] = n;
        buf[s.history + r] = histories[r];
        buf[s.state_slots + r] = caches[r]->state_slot;
        buf[s.state_slots_out + r] = caches[r]->state_slot_out;
        for (int w : batch[r].want) buf[s.logit_rows + k++] = a + w;
        for (int g = 0; g < n_groups; ++g) {
            const std::vector<int>& pg = caches[r]->tables[g].pages;
            for (size_t p = 0; p < pg.size(); ++p) buf[s.block_tables[g] + (size_t)r * s.table_stride[g] + p] = pg[p];
            // A released page (-1) is never addressed: the window keeps queries above it.
            for (int i = 0; i < n; ++i) {
                const int pos = histories[r] + i;
                buf[s.slots[g] + a + i] = pg[pos / ps] * ps + pos % ps;
            }
        }
        a += n;
    }
}

// Recorded steps.  The kernels a step launches, their grids and the buffers they use depend on how many rows each
// request brings, on which rows' logits are wanted and on how much context the block tables have room for -- not on the
// requests' histories, tokens or pages, which the kernels read from the step's metadata on the device.  A recording
// holds the CUDA graph of one such shape, made once the shape has come a few times (a scheduler that cuts prompts
// into portions of its token budget, and every decode step of the same requests, bring the same shape again and again),
// and the static metadata buffer, workspace and logits it uses; a step of that shape is then one copy and one launch.
// What the model's parts decide on the host from a shape is decided once, for the recording's room; every run only
// refills the plan's ints (llmx_plan_fill).
Recording::~Recording() {
    if (exec) cudaGraphExecDestroy(exec);
    if (plan) llmx_plan_free(plan);
}
static int room_for(int context, int max_positions) {
    return std::min((context / 2048 + 2) * 2048, std::max(max_positions, 1));       // at least 2,048 tokens ahead, so recordings change rarely
}
Recording* llmx_engine::recording_for(const std::vector<Batch>& batch, const std::vector<int>& counts, int context) {
    if (!record_steps) return nullptr;
    const int room = room_for(context, max_positions);
    std::vector<int> key = {room, (int)batch.size()};
    bool decode = true;
    for (size_t r = 0; r < batch.size(); ++r) {
        key.push_back(counts[r]);
        key.push_back((int)batch[r].want.size());
        key.insert(key.end(), batch[r].want.begin(), batch[r].want.end());
        decode = decode && counts[r] == 1;
    }
    auto it = recordings.find(key);
    if (it != recordings.end()) return it->second.get();
    int& seen = shapes_seen[key];
    if (seen < (decode ? 4 : 16)) {            // making a recording costs about as much as ten to twenty plain steps save
        if (shapes_seen.size() > 4096) shapes_seen.clear();
        else ++seen;
        return nullptr;
    }
    shapes_seen.erase(key);
    std::unique_ptr<Recording> rec(new Recording);
    rec->room = room;
    const int n_groups = (int)cache->groups.size();
    std::vector<int> max_pages(n_groups);
    for (int g = 0; g < n_groups; ++g) max_pages[g] = std::max(1, (room + cache->page_size - 1) / cache->page_size);
    rec->plan = llmx_plan_make(model, nullptr, 0, counts.data(), nullptr, (int)counts.size(), room, context);
    if (!rec->plan) throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("launch plan: ") + llmx_rt_last_error()};
    int wanted = 0;
    for (const Batch& b : batch) wanted += (int)b.want.size();
    llmx_step& s = rec->step;
    rec->total = layout(s, counts, wanted, max_pages, llmx_plan_ints(rec->plan));
    s.room = room;
    s.plan = rec->plan;
    rec->meta.ensure(rec->total * sizeof(int), stream);
    cuda_check(cudaMemsetAsync(rec->meta.ptr, 0, rec->total * sizeof(int), stream), "clearing a recording's metadata");
    s.meta = (const int*)rec->meta.ptr;
    const size_t need = llmx_model_workspace(model, &s);
    const char* missing = nullptr;
    if (llmx_rt_missing(0, &missing)) return nullptr;       // a plain step binds what is missing first
    rec->workspace.ensure(need, stream);
    s.workspace = rec->workspace.ptr, s.workspace_bytes = rec->workspace.bytes;
    rec->logits.ensure((size_t)std::max(wanted, 1) * vocab * sizeof(float), stream);
    // Keep the number of recordings bounded (the least recently used goes) before this one is made.
    while (recordings.size() >= 24) {
        auto oldest = recordings.begin();
        for (auto j = recordings.begin(); j != recordings.end(); ++j)
            if (j->second->last_use < oldest->second->last_use) oldest = j;
        cuda_check(cudaStreamSynchronize(stream), "waiting before a recording goes");
        recordings.erase(oldest);
    }
    const long long before = llmx_rt_launches();
    cuda_check(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "beginning a recording");
    const int err = llmx_model_forward(model, &s, (float*)rec->logits.ptr);
    cudaGraph_t graph = nullptr;
    const cudaError_t ended = cudaStreamEndCapture(stream, &graph);
    if (err || ended != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        record_steps = false;                               // this model's steps are not recorded; plain steps go on
        return nullptr;
    }
    rec->launches = llmx_rt_launches() - before;
    const cudaError_t made = cudaGraphInstantiate(&rec->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (made != cudaSuccess) {
        cudaGetLastError();
        record_steps = false;
        return nullptr;
    }
    Recording* out = rec.get();
    recordings[key] = std::move(rec);
    return out;
}

// One batch through the model: validate, reserve pages (all or none), lay out the metadata, copy it once, run the
// layers, commit.  Anything that fails before the commit leaves every request as it was.
void llmx_engine::run(const std::vector<Batch>& batch) {
    if (batch.empty()) throw Failure{LLMX_ENGINE_ERR_REFUSED, "a step needs at least one entry"};
    std::set<long long> seen;
    int fresh = 0;
    for (const Batch& b : batch) {
        const std::string who = "request " + std::to_string(b.request);
        if (!seen.insert(b.request).second) throw Failure{LLMX_ENGINE_ERR_REFUSED, who + " appears twice in one step"};
        if (b.tokens.empty()) throw Failure{LLMX_ENGINE_ERR_REFUSED, who + ": an entry without tokens"};
        for (int t : b.tokens)
            if (t < 0 || t >= vocab)
                throw Failure{LLMX_ENGINE_ERR_REFUSED, who + ": token id " + std::to_string(t) + " is outside the vocabulary of " + std::to_string(vocab)};
        const auto it = cache->live.find(b.request);
        const long long have = it == cache->live.end() ? 0 : it->second.length;
        if (it == cache->live.end()) ++fresh;
        if (have + (long long)b.tokens.size() > max_positions)
            throw Failure{LLMX_ENGINE_ERR_REFUSED, who + ": context length of " + std::to_string(max_positions) + " exceeded"};
        for (int w : b.want)
            if (w < 0 || w >= (int)b.tokens.size())
                throw Failure{LLMX_ENGINE_ERR_REFUSED, who + ": wanted place " + std::to_string(w) + " is not among its " +
                                                           std::to_string(b.tokens.size()) + " tokens"};
    }
    if ((int)cache->live.size() + fresh > cache->max_requests)
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "more than " + std::to_string(cache->max_requests) + " live requests"};

    std::vector<long long> created;
    std::vector<RequestCache*> caches, prepared;
    llmx_plan* plan = nullptr;
    try {
        for (const Batch& b : batch) {
            auto it = cache->live.find(b.request);
            if (it == cache->live.end()) {
                caches.push_back(&cache->new_request(b.request));
                created.push_back(b.request);
            } else {
                caches.push_back(&it->second);
            }
        }
        // (a map's elements do not move when others are added)
        for (size_t i = 0; i < batch.size(); ++i) {
            caches[i]->prepare((int)batch[i].tokens.size());
            prepared.push_back(caches[i]);
        }
        if (books_only) {          // the books alone: the pages are reserved, nothing runs
            for (RequestCache* rc : caches) rc->commit();
            ++steps;
            return;
        }

        // ---- the metadata: one int32 buffer, sections padded to 16 bytes (the layout of llmx_step) ----
        const int n_req = (int)batch.size(), n_groups = (int)cache->groups.size();
        std::vector<int> counts(n_req), histories(n_req);
        int wanted = 0, context = 0;
        for (int r = 0; r < n_req; ++r) {
            counts[r] = (int)batch[r].tokens.size();
            histories[r] = caches[r]->length;
            wanted += (int)batch[r].want.size();
            context = std::max(context, histories[r] + counts[r]);
        }
        Recording* rec = recording_for(batch, counts, context);
        if (rec) {
            // A shape that keeps coming: its metadata into the recording's static buffer, one copy, one graph launch.
            int* buf = pinned(rec->total);
            fill_meta(buf, rec->step, rec->total, batch, caches, histories);
            if (llmx_plan_ints(rec->plan) && llmx_plan_fill(rec->plan, histories.data(), buf + rec->step.plan_offset))
                throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("launch plan: ") + llmx_rt_last_error()};
            cuda_check(cudaMemcpyAsync(rec->meta.ptr, buf, rec->total * sizeof(int), cudaMemcpyHostToDevice, stream), "copying the step's metadata");
            cuda_check(cudaEventRecord(ring[ring_at].done, stream), "recording the copy");
            ring[ring_at].used = true;
            last_h2d_bytes = (long long)(rec->total * sizeof(int));
            cuda_check(cudaGraphLaunch(rec->exec, stream), "replaying a recorded step");
            llmx_rt_count_launches(rec->launches);
            rec->last_use = ++use_clock;
            cur_logits = (float*)rec->logits.ptr;
            ++replays;
        } else {
            plan = llmx_plan_make(model, nullptr, 0, counts.data(), histories.data(), n_req, 0, 0);
            if (!plan) throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("launch plan: ") + llmx_rt_last_error()};
            std::vector<int> max_pages(n_groups, 1);
            for (int g = 0; g < n_groups; ++g)
                for (RequestCache* rc : caches) max_pages[g] = std::max(max_pages[g], (int)rc->tables[g].pages.size());
            llmx_step s = {};
            const size_t total = layout(s, counts, wanted, max_pages, llmx_plan_ints(plan));
            int* buf = pinned(total);
            fill_meta(buf, s, total, batch, caches, histories);
            if (llmx_plan_ints(plan) && llmx_plan_fill(plan, histories.data(), buf + s.plan_offset))
                throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("launch plan: ") + llmx_rt_last_error()};
            meta.ensure(total * sizeof(int), stream);
            cuda_check(cudaMemcpyAsync(meta.ptr, buf, total * sizeof(int), cudaMemcpyHostToDevice, stream), "copying the step's metadata");
            cuda_check(cudaEventRecord(ring[ring_at].done, stream), "recording the copy");
            ring[ring_at].used = true;
            last_h2d_bytes = (long long)(total * sizeof(int));
            s.meta = (const int*)meta.ptr;
            s.plan = plan;
            const size_t need = llmx_model_workspace(model, &s);
            const char* missing = nullptr;
            if (llmx_rt_missing(0, &missing))
                throw Failure{LLMX_ENGINE_ERR_UNBOUND, std::string("kernel ") + (missing ? missing : "?") + " is not bound (its library was not loaded)"};
            workspace.ensure(need, stream);
            s.workspace = workspace.ptr, s.workspace_bytes = workspace.bytes;
            logits.ensure((size_t)std::max(wanted, 1) * vocab * sizeof(float), stream);
            if (int err = llmx_model_forward(model, &s, (float*)logits.ptr))
                throw Failure{err == LLMX_RT_ERR_UNBOUND ? (int)LLMX_ENGINE_ERR_UNBOUND : (int)LLMX_ENGINE_ERR_DEVICE,
                              std::string("forward: ") + llmx_rt_last_error()};
            cur_logits = (float*)logits.ptr;
        }
        last_wanted = wanted;
    } catch (...) {
        if (plan) llmx_plan_free(plan);
        for (RequestCache* rc : prepared) rc->abort();
        for (long long id : created) cache->free_request(id);
        throw;
    }
    llmx_plan_free(plan);
    for (RequestCache* rc : caches) rc->commit();
    ++steps;
}

// One token per row of the last step's logits, row i drawn for states[i].
std::vector<int> llmx_engine::draw(const std::vector<Request*>& who) {
    const int rows = (int)who.size();
    if (rows == 0) return {};
    typedef int (*sample_fn)(const float*, int, int, const void*, int*, int, cudaStream_t);
    typedef int (*penalize_fn)(float*, int, const int*, const int*, const int*, const float*, const float*, const float*, int, cudaStream_t);
    const sample_fn sample = (sample_fn)llmx_rt_kernel("llmx_sample");
    const penalize_fn penalize = (penalize_fn)llmx_rt_kernel("llmx_penalize");
    if (!sample || !penalize) throw Failure{LLMX_ENGINE_ERR_UNBOUND, "kernel llmx_sample is not bound (its library was not loaded)"};
    // Penalties first, in place: the logits are this step's own.
    std::vector<int> row_of, token, count;
    for (int r = 0; r < rows; ++r)
        if (who[r]->sampling.penalized())
            for (const auto& kv : who[r]->sampling.counts) {
                row_of.push_back(r);
                token.push_back(kv.first);
                count.push_back(kv.second);
            }
    struct Row { float temp, top_p, min_p, u; int top_k, masked; };
    const size_t items = row_of.size();
    const size_t bytes = items * 3 * sizeof(int) + (size_t)rows * 3 * sizeof(float) + (size_t)rows * sizeof(Row) + (size_t)rows * sizeof(int) + 64;
    sample_buf.ensure(bytes, stream);
    // Pinned staging, so that the settings' copy and the draw are enqueued behind the step without waiting for it
    // (every call ends with a synchronisation, after which the buffer is free again).
    if (sample_host_bytes < bytes) {
        if (sample_host) cudaFreeHost(sample_host);
        sample_host = nullptr;
        cuda_check(cudaMallocHost((void**)&sample_host, std::max<size_t>(bytes + (bytes >> 1), 4096)), "allocating pinned memory");
        sample_host_bytes = std::max<size_t>(bytes + (bytes >> 1), 4096);
    }
    char* h = sample_host;
    int* h_items = (int*)h;
    float* h_pen = (float*)(h_items + 3 * items);
    Row* h_rows = (Row*)(h_pen + 3 * rows);
    if (items) {
        memcpy(h_items, row_of.data(), items * sizeof(int));
        memcpy(h_items + items, token.data(), items * sizeof(int));
        memcpy(h_items + 2 * items, count.data(), items * sizeof(int));
    }
    bool all_greedy = true;
    std::vector<unsigned long long> generators(rows);      // a draw that fails leaves the requests' generators as they were
    for (int r = 0; r < rows; ++r) generators[r] = who[r]->sampling.rng.state;
    try {
        for (int r = 0; r < rows; ++r) {
            const llmx_sampling& p = who[r]->params;
            h_pen[r] = p.penalty, h_pen[rows + r] = p.presence_penalty, h_pen[2 * rows + r] = p.frequency_penalty;
            const bool greedy = p.temp <= 0.0f;
            all_greedy = all_greedy && greedy;
            h_rows[r] = Row{p.temp, p.top_p, p.min_p, greedy ? 0.0f : who[r]->sampling.rng.unit(), p.top_k, who[r]->sampling.masked};
        }
        char* d = (char*)sample_buf.ptr;
        cuda_check(cudaMemcpyAsync(d, h, (char*)(h_rows + rows) - h, cudaMemcpyHostToDevice, stream), "copying the sampling settings");
        int* d_items = (int*)d;
        float* d_pen = (float*)(d_items + 3 * items);
        Row* d_rows = (Row*)(d_pen + 3 * rows);
        int* d_out = (int*)(d_rows + rows);
        if (items)
            if (int err = penalize(cur_logits, vocab, d_items, d_items + items, d_items + 2 * items, d_pen, d_pen + rows,
                                   d_pen + 2 * rows, (int)items, stream))
                throw Failure{LLMX_ENGINE_ERR_DEVICE, "penalize: error " + std::to_string(err)};
        if (int err = sample(cur_logits, rows, vocab, d_rows, d_out, all_greedy ? 1 : 0, stream))
            throw Failure{LLMX_ENGINE_ERR_DEVICE, "sample: error " + std::to_string(err)};
        if (host_ids_n < (size_t)rows) {
            if (host_ids) cudaFreeHost(host_ids);
            host_ids = nullptr;
            cuda_check(cudaMallocHost((void**)&host_ids, (size_t)std::max(rows, 64) * sizeof(int)), "allocating pinned memory");
            host_ids_n = (size_t)std::max(rows, 64);
        }
        cuda_check(cudaMemcpyAsync(host_ids, d_out, (size_t)rows * sizeof(int), cudaMemcpyDeviceToHost, stream), "reading the drawn ids");
        sync_and_check();
    } catch (...) {
        for (int r = 0; r < rows; ++r) who[r]->sampling.rng.state = generators[r];
        throw;
    }
    return std::vector<int>(host_ids, host_ids + rows);
}

// ===============================================================================================================
// The C interface.
// ===============================================================================================================
#define LLMX_API extern "C" __attribute__((visibility("default")))

template <typename F>
static int guarded(F&& f) {
    try {
        return f();
    } catch (const Failure& e) {
        return fail(e.code, e.what);
    } catch (const std::exception& e) {
        return fail(LLMX_ENGINE_ERR_REFUSED, e.what());
    }
}

LLMX_API const char* llmx_engine_last_error(void) { return g_error.c_str(); }
LLMX_API int llmx_engine_last_code(void) { return g_code; }

LLMX_API void llmx_sampling_defaults(llmx_sampling* p) {
    *p = llmx_sampling{64, 0.8f, 40, 0.95f, 0.0f, 1.0f, 0.0f, 0.0f, 0ull, 0, nullptr, 0};
}
LLMX_API void llmx_sampling_greedy(llmx_sampling* p, int max_tokens) {
    *p = llmx_sampling{max_tokens, 0.0f, 0, 1.0f, 0.0f, 1.0f, 0.0f, 0.0f, 0ull, 0, nullptr, 0};
}

LLMX_API llmx_engine* llmx_engine_create(llmx_model* model, const llmx_engine_desc* desc) {
    llmx_engine* e = nullptr;
    const int err = guarded([&] {
        if (!desc) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_create: no description"};
        e = new llmx_engine(model, *desc, nullptr);
        return 0;
    });
    return err ? nullptr : e;
}
LLMX_API void llmx_engine_destroy(llmx_engine* e) { delete e; }

LLMX_API int llmx_engine_forward(llmx_engine* e, const llmx_entry* entries, int n, float* out, const float** device_logits) {
    return guarded([&] {
        if (!e || (n > 0 && !entries)) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_forward: an engine and entries"};
        if (!e->books_only) cuda_check(cudaSetDevice(e->device), "choosing the device");
        std::vector<Batch> batch;
        for (int i = 0; i < n; ++i) {
            Batch b;
            b.request = entries[i].request;
            if (entries[i].n_tokens > 0) b.tokens.assign(entries[i].tokens, entries[i].tokens + entries[i].n_tokens);
            if (entries[i].n_want > 0) b.want.assign(entries[i].want, entries[i].want + entries[i].n_want);
            batch.push_back(std::move(b));
        }
        e->run(batch);
        if (e->books_only) return 0;
        if (out && e->last_wanted > 0)
            cuda_check(cudaMemcpyAsync(out, e->cur_logits, (size_t)e->last_wanted * e->vocab * sizeof(float), cudaMemcpyDeviceToHost, e->stream),
                       "reading the logits");
        e->sync_and_check();
        if (device_logits) *device_logits = e->last_wanted > 0 ? (const float*)e->cur_logits : nullptr;
        return 0;
    });
}
LLMX_API int llmx_engine_end(llmx_engine* e, long long request) {
    return guarded([&] {
        e->cache->free_request(request);
        return 0;
    });
}
LLMX_API int llmx_engine_truncate(llmx_engine* e, long long request, int length) {
    return guarded([&] {
        auto it = e->cache->live.find(request);
        if (it == e->cache->live.end()) throw Failure{LLMX_ENGINE_ERR_REFUSED, "request " + std::to_string(request) + " is not live"};
        it->second.truncate(length);
        return 0;
    });
}
LLMX_API int llmx_engine_length(llmx_engine* e, long long request) {
    const auto it = e->cache->live.find(request);
    return it == e->cache->live.end() ? 0 : it->second.length;
}

LLMX_API long long llmx_engine_add_request(llmx_engine* e, const int* ids, int n, const llmx_sampling* sampling) {
    long long id = -1;
    const int err = guarded([&] {
        if (!e || !sampling || (n > 0 && !ids)) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_add_request: an engine, ids and settings"};
        check_sampling(*sampling);
        auto r = std::make_shared<Request>();
        r->id = e->next_id;
        r->prompt.assign(ids, ids + std::max(n, 0));
        for (int t : r->prompt)
            if (t < 0 || t >= e->vocab)
                throw Failure{LLMX_ENGINE_ERR_REFUSED, "token id " + std::to_string(t) + " is outside the vocabulary of " + std::to_string(e->vocab)};
        r->params = *sampling;
        r->stop_ids.assign(sampling->stop_ids, sampling->stop_ids + (sampling->stop_ids ? sampling->n_stop : 0));
        r->params.stop_ids = nullptr;
        r->sampling.init(*sampling, e->sched.eos_ids.empty() ? -1 : e->sched.eos_ids[0]);
        e->sched.add(r);
        e->requests[r->id] = r;
        id = e->next_id++;
        return 0;
    });
    return err ? -(long long)err : id;
}

// The first half of a step: give back what is to be given back, plan, and say which requests ended without running.
// Leaves the planned entries in `planned`; returns false when there is nothing to run.
bool llmx_engine::begin_step(std::vector<llmx_step_result>& early) {
    auto release = [&] {
        for (long long id : sched.to_release) cache->free_request(id);
        sched.to_release.clear();
    };
    release();
    std::vector<std::shared_ptr<Request>> ended;
    planned = sched.plan(ended);
    release();
    for (const auto& r : ended) early.push_back(llmx_step_result{r->id, -1, r->finished});
    if (planned.empty() && !sched.idle() && ended.empty())
        throw Failure{LLMX_ENGINE_ERR_REFUSED, "the scheduler planned an empty step while requests are waiting"};
    return !planned.empty();
}
// The planned entries through the model (or, for the books alone, through the cache's books); who wants a token.
std::vector<Request*> llmx_engine::run_planned() {
    std::vector<Batch> batch;
    std::vector<Request*> wanting;
    for (const Planned& p : planned) {
        Batch b;
        b.request = p.request->id;
        b.tokens = p.tokens;
        if (p.want_last) {
            b.want.push_back((int)p.tokens.size() - 1);
            wanting.push_back(p.request.get());
        }
        batch.push_back(std::move(b));
    }
    // The sampler's kernels must be there before the step changes anything.
    if (!books_only && !wanting.empty() && (!llmx_rt_kernel("llmx_sample") || !llmx_rt_kernel("llmx_penalize")))
        throw Failure{LLMX_ENGINE_ERR_UNBOUND, "kernel llmx_sample is not bound (its library was not loaded)"};
    run(batch);
    return wanting;
}
// The second half: book the tokens drawn for the entries that wanted one.
std::vector<llmx_step_result> llmx_engine::finish_step(const std::vector<int>& drawn) {
    std::vector<llmx_step_result> out = sched.complete(planned, drawn);
    planned.clear();
    for (long long id : sched.to_release) cache->free_request(id);
    sched.to_release.clear();
    return out;
}

LLMX_API int llmx_engine_step(llmx_engine* e, llmx_step_result* out, int capacity) {
    int written = 0;
    const int err = guarded([&] {
        if (!e || (capacity > 0 && !out)) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_step: an engine and room for results"};
        if (e->books_only) throw Failure{LLMX_ENGINE_ERR_REFUSED, "an engine of books alone runs nothing: llmx_engine_plan and llmx_engine_book"};
        if (!e->planned.empty()) throw Failure{LLMX_ENGINE_ERR_REFUSED, "a planned step is waiting for llmx_engine_book"};
        cuda_check(cudaSetDevice(e->device), "choosing the device");
        std::vector<llmx_step_result> results;
        if (e->begin_step(results)) {
            // What the cache held before the step: a failure that shows only after the step's rows were committed (a
            // kernel that gave up a wait, a draw that could not run) takes the rows back, so that every request is
            // as it was and the same step can be planned again.
            std::vector<std::pair<long long, int>> before;       // request, committed tokens (-1: not in the cache yet)
            for (const Planned& p : e->planned) {
                const auto it = e->cache->live.find(p.request->id);
                before.emplace_back(p.request->id, it == e->cache->live.end() ? -1 : it->second.length);
            }
            bool ran = false;
            try {
                const std::vector<Request*> wanting = e->run_planned();
                ran = true;
                const std::vector<int> drawn = e->draw(wanting);
                if (wanting.empty()) e->sync_and_check();
                for (const llmx_step_result& r : e->finish_step(drawn)) results.push_back(r);
            } catch (...) {
                if (ran)
                    for (const auto& b : before) {
                        const auto it = e->cache->live.find(b.first);
                        if (it == e->cache->live.end()) continue;
                        try {
                            if (b.second < 0) e->cache->free_request(b.first);
                            else it->second.truncate(b.second);
                        } catch (const Failure&) {
                            // fixed-size state or a window that has moved on cannot be taken back: the step's failure is what is reported
                        }
                    }
                e->planned.clear();
                throw;
            }
        }
        for (const llmx_step_result& r : results)
            if (written < capacity) out[written++] = r;
        return 0;
    });
    return err ? -err : written;
}

// The two halves of a step for a caller that draws the tokens itself.  llmx_engine_plan plans a step, reserves its
// pages and (with a model) runs it; it writes the planned entries and returns their number (0: nothing to run; requests
// that ended without running are then reported by llmx_engine_book).  llmx_engine_book takes one token for every entry
// that wanted one, in order, and books them.  An engine created without a model and with device < 0 keeps the books
// alone: the scheduler's decisions and the cache's pages can be followed without a GPU.
LLMX_API int llmx_engine_plan(llmx_engine* e, llmx_planned_entry* out, int capacity) {
    int written = 0;
    const int err = guarded([&] {
        if (!e || (capacity > 0 && !out)) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_plan: an engine and room for entries"};
        if (!e->planned.empty()) throw Failure{LLMX_ENGINE_ERR_REFUSED, "a planned step is waiting for llmx_engine_book"};
        if (!e->books_only) cuda_check(cudaSetDevice(e->device), "choosing the device");
        e->early.clear();
        if (!e->begin_step(e->early)) return 0;
        try {
            e->run_planned();
        } catch (...) {
            e->planned.clear();
            throw;
        }
        for (const Planned& p : e->planned)
            if (written < capacity)
                out[written++] = llmx_planned_entry{p.request->id, (int)p.tokens.size(), p.tokens.empty() ? -1 : p.tokens[0], p.want_last ? 1 : 0};
        return 0;
    });
    return err ? -err : written;
}
// The logits of the step that ran last ([wanted, vocab] float32): copied to `out` (host, may be null); `device` (may be
// null) receives the device buffer, valid until the next step.  Returns the number of wanted places.
LLMX_API int llmx_engine_last_logits(llmx_engine* e, float* out, const float** device) {
    int wanted = 0;
    const int err = guarded([&] {
        if (!e || e->books_only) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_last_logits: an engine with a model"};
        wanted = e->last_wanted;
        if (out && wanted > 0)
            cuda_check(cudaMemcpyAsync(out, e->cur_logits, (size_t)wanted * e->vocab * sizeof(float), cudaMemcpyDeviceToHost, e->stream),
                       "reading the logits");
        e->sync_and_check();
        if (device) *device = wanted > 0 ? (const float*)e->cur_logits : nullptr;
        return 0;
    });
    return err ? -err : wanted;
}
LLMX_API int llmx_engine_book(llmx_engine* e, const int* drawn, int n, llmx_step_result* out, int capacity) {
    int written = 0;
    const int err = guarded([&] {
        if (!e || (n > 0 && !drawn) || (capacity > 0 && !out)) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_book: an engine, tokens and room for results"};
        std::vector<llmx_step_result> results = e->early;
        e->early.clear();
        if (!e->planned.empty()) {
            int wanting = 0;
            for (const Planned& p : e->planned) wanting += p.want_last ? 1 : 0;
            if (wanting != n)
                throw Failure{LLMX_ENGINE_ERR_REFUSED, "the planned step wants " + std::to_string(wanting) + " tokens, " + std::to_string(n) + " were given"};
            for (const llmx_step_result& r : e->finish_step(std::vector<int>(drawn, drawn + n))) results.push_back(r);
        } else if (n) {
            throw Failure{LLMX_ENGINE_ERR_REFUSED, "no planned step is waiting for tokens"};
        }
        for (const llmx_step_result& r : results)
            if (written < capacity) out[written++] = r;
        return 0;
    });
    return err ? -err : written;
}
LLMX_API int llmx_engine_idle(llmx_engine* e) { return e->sched.idle() ? 1 : 0; }

LLMX_API int llmx_engine_output(llmx_engine* e, long long request, int* tokens, int capacity, int* finished) {
    const auto it = e->requests.find(request);
    if (it == e->requests.end()) return -fail(LLMX_ENGINE_ERR_REFUSED, "no such request: " + std::to_string(request));
    const Request& r = *it->second;
    const int n = std::min((int)r.output.size(), std::max(capacity, 0));
    if (tokens) memcpy(tokens, r.output.data(), (size_t)n * sizeof(int));
    if (finished) *finished = r.finished;
    return n;
}
LLMX_API int llmx_engine_forget(llmx_engine* e, long long request) {
    const auto it = e->requests.find(request);
    if (it == e->requests.end() || it->second->state != Request::FINISHED)
        return fail(LLMX_ENGINE_ERR_REFUSED, "only a finished request's record can be forgotten");
    e->requests.erase(it);
    return 0;
}

LLMX_API int llmx_engine_groups(llmx_engine* e) { return (int)e->cache->groups.size(); }
LLMX_API int llmx_engine_pages(llmx_engine* e, int group, long long* total, long long* free_pages) {
    if (group < 0 || group >= (int)e->cache->groups.size()) return fail(LLMX_ENGINE_ERR_REFUSED, "no such cache group");
    if (total) *total = e->cache->groups[group].pool.pages();
    if (free_pages) *free_pages = e->cache->groups[group].pool.free_pages();
    return 0;
}
LLMX_API int llmx_engine_held_pages(llmx_engine* e, long long request, int group) {
    const auto it = e->cache->live.find(request);
    if (it == e->cache->live.end() || group < 0 || group >= (int)it->second.tables.size()) return 0;
    const BlockTable& t = it->second.tables[group];
    return (int)t.pages.size() - t.first_live;
}
LLMX_API int llmx_engine_check(llmx_engine* e) {
    const std::string bad = e->cache->check();
    return bad.empty() ? 0 : fail(LLMX_ENGINE_ERR_REFUSED, bad);
}
LLMX_API long long llmx_engine_preemptions(llmx_engine* e) { return e->sched.preemptions; }
LLMX_API long long llmx_engine_steps(llmx_engine* e) { return e->steps; }
LLMX_API long long llmx_engine_replays(llmx_engine* e) { return e->replays; }
LLMX_API void llmx_engine_record_steps(llmx_engine* e, int on) { e->record_steps = on != 0; }
LLMX_API long long llmx_engine_last_h2d_bytes(llmx_engine* e) { return e->last_h2d_bytes; }
LLMX_API int llmx_engine_vocab(llmx_engine* e) { return e->vocab; }
LLMX_API int llmx_engine_max_positions(llmx_engine* e) { return e->max_positions; }
