// What the native engine's translation units share (engine.cpp: bookkeeping and steps; loader.cpp: files and models).
#pragma once
#include "llmx_engine.h"

#include <cuda_runtime.h>

#include <deque>
#include <map>
#include <memory>
#include <string>
#include <vector>

// A bound kernel entry point by name (null when its library is not loaded; the name is then noted as missing).
extern "C" void* llmx_rt_kernel(const char* name);

namespace llmx_engine_detail {

struct Failure {
    int code;
    std::string what;
};
extern thread_local std::string g_error;
int fail(int code, const std::string& what);

// ---- pages -----------------------------------------------------------------------------------------------------
class PagePool {
public:
    explicit PagePool(long long pages = 0);
    int alloc();
    void release(int page);
    int pages() const { return (int)refs_.size(); }
    int free_pages() const { return (int)free_.size(); }
    int refs(int page) const { return refs_[page]; }
    std::string check() const;

private:
    std::vector<int> refs_;
    std::vector<int> free_;        // LIFO; lowest ids are handed out first from a fresh pool
};

// One request's pages in one group: logical page number -> page id.  window 0 keeps every key; W keeps, for a query at
// position p, the keys p-W+1..p, so once `length` tokens are committed the pages wholly below length-W+1 are given back
// (their entries become -1 and are never read again).
struct BlockTable {
    PagePool* pool;
    int page_size, window;
    std::vector<int> pages;
    int length = 0, pending = 0, first_live = 0;
    BlockTable(PagePool* p, int ps, int w) : pool(p), page_size(ps), window(w) {}
    int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
    void prepare(int n);       // positions [length, length + n) become addressable; on exhaustion what this call took goes back
    void commit();
    void abort();
    void truncate(int to);
    void free();

private:
    void shrink_to(int tokens);
};

class StateSlots {
public:
    explicit StateSlots(int n = 0) : held_((size_t)n, false) {
        for (int s = n - 1; s >= 0; --s) free_.push_back(s);
    }
    int take();
    void give_back(int slot);
    int count() const { return (int)held_.size(); }
    std::string check() const;

private:
    std::vector<bool> held_;
    std::vector<int> free_;
};

struct Group {
    int kv_heads, head_dim, window, page_size;
    PagePool pool;
    std::vector<int> members;      // cache entry indices, in storage order
    void* storage = nullptr;       // [members, pages, 2, kv_heads, page_size, head_dim]
    size_t member_bytes = 0;
    Group(int kvh, int d, int w, int ps, long long pages) : kv_heads(kvh), head_dim(d), window(w), page_size(ps), pool(pages) {}
};

struct RequestCache {
    std::vector<BlockTable> tables;
    int state_slot = -1, state_slot_out = -1;      // where the request's state lies / where a step leaves it (swapped at commit)
    int length = 0, pending = 0;
    void prepare(int n);       // room for n more tokens in every group, or in none
    void commit();
    void abort();
    void truncate(int to);
};

struct Cache {
    int page_size, max_requests, kv_dtype;
    std::vector<llmx_cache_entry_desc> entries;
    std::vector<int> entry_group, entry_member;
    std::vector<Group> groups;
    StateSlots slots;
    std::vector<void*> state_storage;
    std::map<long long, RequestCache> live;
    llmx_caches* views = nullptr;

    Cache(const llmx_engine_desc&, bool books_only);      // books_only: no device storage
    ~Cache();
    Cache(const Cache&) = delete;
    RequestCache& new_request(long long id);
    void free_request(long long id);
    std::vector<long long> pages_needed(long long tokens, long long step_tokens) const;
    std::string check() const;
};

// ---- sampling state -----------------------------------------------------------------------------------------------
struct XorShift64 {
    unsigned long long state = 0x9E3779B97F4A7C15ull;
    unsigned long long next();
    float unit();              // uniform in [0, 1): the top 24 bits
};
struct SamplingState {
    XorShift64 rng;
    std::map<int, int> counts; // of the tokens the request has generated (kept only when a penalty is on)
    int masked = -1;           // the id that is never drawn (ignore_eos)
    bool penalties = false;
    void init(const llmx_sampling& p, int eos_id) {
        if (p.seed) rng.state = p.seed;
        masked = p.ignore_eos ? eos_id : -1;
        penalties = (p.penalty > 0 && p.penalty != 1.0f) || p.presence_penalty != 0.0f || p.frequency_penalty != 0.0f;
    }
    bool penalized() const { return penalties; }
    void saw(int token) {
        if (penalties) ++counts[token];
    }
};

// ---- the scheduler ------------------------------------------------------------------------------------------------
struct Request {
    enum State { WAITING, RUNNING, FINISHED };
    long long id = 0;
    std::vector<int> prompt, output, stop_ids;
    llmx_sampling params{};
    long long fed = 0;         // tokens of prompt + output that are in the cache
    State state = WAITING;
    int finished = 0;          // 1 end of sequence, 2 max_tokens, 3 the cache cannot hold it
    int admissions = 0;
    long long order = -1;      // first admission number
    SamplingState sampling;
    long long tokens() const { return (long long)prompt.size() + (long long)output.size(); }
    int token_at(long long i) const { return i < (long long)prompt.size() ? prompt[(size_t)i] : output[(size_t)(i - (long long)prompt.size())]; }
    bool decoding() const { return !output.empty() && fed == tokens() - 1; }      // everything but the last drawn token is in the cache
};
struct Planned {
    std::shared_ptr<Request> request;
    std::vector<int> tokens;
    bool want_last;
};
struct Scheduler {
    Cache* cache = nullptr;
    long long max_positions = 0, max_batch_tokens = 2048;
    int max_requests = 16, max_queue = 0;
    bool reserve_prompt_only = false;
    std::vector<int> eos_ids;
    std::deque<std::shared_ptr<Request>> waiting;
    std::vector<std::shared_ptr<Request>> running;
    std::map<long long, std::vector<long long>> reserved;
    std::vector<long long> to_release;     // requests whose cache is to be given back before the next step
    long long admission = 0, preemptions = 0;

    void add(const std::shared_ptr<Request>&);
    bool idle() const { return waiting.empty() && running.empty(); }
    std::vector<Planned> plan(std::vector<std::shared_ptr<Request>>& ended);
    std::vector<llmx_step_result> complete(const std::vector<Planned>&, const std::vector<int>& drawn);

private:
    std::vector<long long> reservation(const Request&) const;
    bool fits(const std::vector<long long>& extra) const;
    void admit();
    void pause_latest();
    void grow(std::vector<std::shared_ptr<Request>>& ended);
    void finish(const std::shared_ptr<Request>&, int reason);
};

// ---- device memory the engine owns ---------------------------------------------------------------------------------
struct DeviceBuffer {
    void* ptr = nullptr;
    size_t bytes = 0;
    void ensure(size_t want, cudaStream_t stream);     // grows (never shrinks); waits for the stream before it frees
    ~DeviceBuffer();
};

// A model the engine loaded itself: the parts, the weights' device memory, what the configuration says.
struct LoadedModel {
    virtual ~LoadedModel() {}
    llmx_model* model = nullptr;
    llmx_engine_desc desc{};
    std::vector<llmx_cache_entry_desc> entries;
    std::vector<int> eos_ids;
};

struct Batch {
    long long request;
    std::vector<int> tokens, want;
};

// The CUDA graph of one step shape and what it reads and writes (see engine.cpp, "Recorded steps").
struct Recording {
    int room = 0;
    llmx_step step{};
    size_t total = 0;
    llmx_plan* plan = nullptr;
    DeviceBuffer meta, workspace, logits;
    cudaGraphExec_t exec = nullptr;
    long long launches = 0, last_use = 0;
    ~Recording();
};

}  // namespace llmx_engine_detail

struct llmx_engine {
    std::unique_ptr<llmx_engine_detail::LoadedModel> owned;
    llmx_model* model;
    int vocab, max_positions, position_streams, device;
    bool books_only;           // no model and no device: the cache's and the scheduler's books alone
    cudaStream_t stream = nullptr;
    std::unique_ptr<llmx_engine_detail::Cache> cache;
    llmx_engine_detail::Scheduler sched;
    std::map<long long, std::shared_ptr<llmx_engine_detail::Request>> requests;
    long long next_id = 0, steps = 0, last_h2d_bytes = 0;
    int last_wanted = 0;
    float* cur_logits = nullptr;       // the logits of the step that ran last (the engine's buffer or a recording's)
    bool record_steps = true;
    std::map<std::vector<int>, std::unique_ptr<llmx_engine_detail::Recording>> recordings;
    std::map<std::vector<int>, int> shapes_seen;
    long long use_clock = 0, replays = 0;
    int* error_word = nullptr;
    int* counters = nullptr;
    llmx_engine_detail::DeviceBuffer meta, workspace, logits, sample_buf;
    struct Pinned { int* host = nullptr; size_t ints = 0; cudaEvent_t done = nullptr; bool used = false; } ring[4];
    int ring_at = 0;
    int* host_ids = nullptr;
    size_t host_ids_n = 0;
    char* sample_host = nullptr;       // pinned staging of a draw's settings
    size_t sample_host_bytes = 0;

    llmx_engine(llmx_model*, const llmx_engine_desc&, std::unique_ptr<llmx_engine_detail::LoadedModel>);
    ~llmx_engine();
    llmx_engine(const llmx_engine&) = delete;
    int* pinned(size_t ints);
    std::vector<llmx_engine_detail::Planned> planned;      // a step that is planned and not yet booked
    std::vector<llmx_step_result> early;                    // requests that ended while it was planned
    bool begin_step(std::vector<llmx_step_result>& early_results);
    std::vector<llmx_engine_detail::Request*> run_planned();
    std::vector<llmx_step_result> finish_step(const std::vector<int>& drawn);
    void run(const std::vector<llmx_engine_detail::Batch>&);
    size_t layout(llmx_step&, const std::vector<int>& counts, int wanted, const std::vector<int>& max_pages, int plan_ints) const;
    void fill_meta(int* buf, const llmx_step&, size_t total, const std::vector<llmx_engine_detail::Batch>&,
                   const std::vector<llmx_engine_detail::RequestCache*>&, const std::vector<int>& histories) const;
    llmx_engine_detail::Recording* recording_for(const std::vector<llmx_engine_detail::Batch>&, const std::vector<int>& counts, int context);
    std::vector<int> draw(const std::vector<llmx_engine_detail::Request*>&);
    void sync_and_check();
};
