// llmx_b200 native engine: everything between a request's tokens and its next token, as host code.
//
// The model runtime (llmx_runtime.h) runs one step's rows through the layers.  This library is what stands around it:
// the cache's bookkeeping (pages, block tables, groups of layers with pools of their own, slots of fixed-size state),
// the step's metadata, the scheduler (admission, portions of prompts under a token budget, decoding, what happens
// when pages run out), the sampler's state and draws, and the files (config.json, safetensors) a model is loaded
// from.  It is the counterpart of the reference's header-only entry points: `infer::load_model`
// (src/inference/load.hpp:74-94), `Model::make_sequence / forward / step / reset` (src/model/runtime.hpp:1006-1387)
// and `infer::generate` (src/inference/generate.hpp:19-124), with the server scheduler's policy
// (src/server/policy.hpp:153-256) for many requests at once.
//
//   llmx_engine_load(dir)                   ->  an engine that owns its model, weights and cache
//   llmx_engine_create(model, desc)         ->  an engine over a model the caller built (llmx_model_create)
//   llmx_engine_add_request(ids, sampling)  ->  id
//   llmx_engine_step()                      ->  [(id, token, finished)]: plan a step, run it, draw, book
//   llmx_engine_forward(entries)            ->  logits at the wanted places (the low level: the caller schedules)
//
// Every function returns 0 (or a count, or an id) on success and a negative or LLMX_ENGINE_ERR_* code on failure;
// `llmx_engine_last_error` gives the text for the calling thread.  A step that fails leaves every request as it was.
// The engine runs on its own CUDA stream and synchronises where a result goes to the host.
//
// Threads: an engine is one caller's at a time -- its functions take no lock, so calls on the same engine from several
// threads must be serialised by the caller (a server puts its step loop on one thread and hands requests to it).
// Different engines may be used from different threads; the error text is kept per thread.
#pragma once
#include "llmx_runtime.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { LLMX_ENGINE_ERR_REFUSED = 20001,      // a request or a batch the engine does not take (the text says why)
       LLMX_ENGINE_ERR_CACHE = 20002,        // the pages do not suffice
       LLMX_ENGINE_ERR_FILE = 20003,         // a file that cannot be read or does not say what it must
       LLMX_ENGINE_ERR_WEIGHTS = 20004,      // tensors missing, unexpected or of the wrong shape (all listed)
       LLMX_ENGINE_ERR_DEVICE = 20005,       // a CUDA call failed, or a kernel gave up a bounded wait
       LLMX_ENGINE_ERR_UNBOUND = LLMX_RT_ERR_UNBOUND };   // a kernel library is not loaded (llmx_rt_missing names what)

typedef struct llmx_engine llmx_engine;

// What a cache entry (a layer's share of the cache) needs: nothing, keys and values, or a tensor of fixed size.
typedef struct llmx_cache_entry_desc {
    int kind;                   // 0 none, 1 keys and values, 2 fixed-size state
    int kv_heads, head_dim;     // kind 1
    int window;                 // kind 1: 0 keeps every key, W the last W
    long long state_bytes;      // kind 2: bytes per request
} llmx_cache_entry_desc;

typedef struct llmx_engine_desc {
    int vocab, max_positions, position_streams;
    int page_size;
    long long kv_tokens;            // tokens the pool of every group that keeps all keys is made for
    long long window_kv_tokens;     // ... of groups that keep a window (0: as many)
    int max_requests;               // live requests
    int kv_dtype;                   // LLMX_DT_*
    const llmx_cache_entry_desc* entries;
    int n_entries;
    const int* eos_ids;
    int n_eos;
    // the scheduler
    int max_batch_tokens;           // the most tokens one step holds (0: 2,048)
    int max_queue;                  // waiting requests at most (0: no limit)
    int reserve_prompt_only;        // 0: a request reserves prompt + max_tokens; 1: its prompt and a page of growth
    int device;
} llmx_engine_desc;

// Options of llmx_engine_load.
typedef struct llmx_engine_options {
    int dtype;                      // LLMX_DT_BF16 (the serving path) or LLMX_DT_F32 (everything in true 32-bit)
    int kv_dtype;                   // -1: as dtype
    int page_size;                  // 0: 16
    long long kv_tokens;            // 0: 8192
    long long window_kv_tokens;
    int max_requests;               // 0: 16
    int max_batch_tokens, max_queue, reserve_prompt_only;
    int invariant;                  // schedules chosen by sizes alone (LLMX_FLAG_INVARIANT)
    int device;
    const char* kernel_dir;         // folder of built kernel libraries to bind (null: the caller has bound them)
} llmx_engine_options;

typedef struct llmx_sampling {
    int max_tokens;                 // tokens generated at most (>= 1)
    float temp;                     // 0: greedy
    int top_k;                      // 0 keeps every token
    float top_p, min_p;
    float penalty, presence_penalty, frequency_penalty;
    unsigned long long seed;        // 0 keeps the generator's fixed default state
    int ignore_eos;
    const int* stop_ids;            // extra ids that end a reply
    int n_stop;
} llmx_sampling;
void llmx_sampling_defaults(llmx_sampling*);      // the reference's: 64 tokens, temp 0.8, top-k 40, top-p 0.95
void llmx_sampling_greedy(llmx_sampling*, int max_tokens);

llmx_engine* llmx_engine_create(llmx_model* model, const llmx_engine_desc*);    // the model stays the caller's
// A folder with config.json and model.safetensors (or several *.safetensors files); the model class is chosen by
// config.json.  (A folder of random weights for a configuration and a seed is written by the Python package's
// `llmx_b200.weights.write_random_model`; this loader reads it like any other.)
llmx_engine* llmx_engine_load(const char* model_dir, const llmx_engine_options*);
void llmx_engine_destroy(llmx_engine*);
const char* llmx_engine_last_error(void);
int llmx_engine_last_code(void);            // the code of the calling thread's last failure (for calls that return a pointer)

// ---- the low level: the caller says which requests bring which tokens ------------------------------------------
typedef struct llmx_entry {
    long long request;              // any id; a request is live from its first entry to llmx_engine_end
    const int* tokens;
    int n_tokens;
    const int* want;                // places among these tokens whose logits are wanted
    int n_want;
} llmx_entry;
// One batch: portions of prompts beside single decoded tokens, cut anywhere.  `logits` (host, [wanted, vocab]
// float32) may be null; `device_logits` (may be null) receives the device buffer, valid until the next call.
int llmx_engine_forward(llmx_engine*, const llmx_entry* entries, int n, float* logits, const float** device_logits);
int llmx_engine_end(llmx_engine*, long long request);                 // what the request holds is given back
int llmx_engine_truncate(llmx_engine*, long long request, int length);
int llmx_engine_length(llmx_engine*, long long request);              // tokens in the cache (0: not live)

// ---- generation: the engine schedules ------------------------------------------------------------------------------
long long llmx_engine_add_request(llmx_engine*, const int* ids, int n, const llmx_sampling*);   // id >= 0, or -code
typedef struct llmx_step_result {
    long long request;
    int token;                      // the token drawn (-1: the reply ended without one, at an end-of-sequence id)
    int finished;                   // 0 no; 1 end of sequence; 2 max_tokens; 3 the cache cannot hold it
} llmx_step_result;
// Plans one step, runs it, draws a token for every request whose logits it asked for, books them.  Returns how many
// results were written (at most `capacity`; a step yields at most max_requests), 0 when nothing is left to do, or -code.
int llmx_engine_step(llmx_engine*, llmx_step_result* out, int capacity);
int llmx_engine_idle(llmx_engine*);
// The two halves of llmx_engine_step, for a caller that draws the tokens itself.  llmx_engine_plan plans a step,
// reserves its pages and runs it; it writes the planned entries and returns their number (0: nothing to run).
// llmx_engine_book takes one token for every entry that wanted one, in the entries' order, books them, and writes the
// results (with those of requests that ended while the step was planned).  An engine made by
// llmx_engine_create(NULL, desc) with desc->device < 0 keeps the books alone (no model, no device memory): the
// scheduler's decisions and the cache's pages can then be followed on any machine.
typedef struct llmx_planned_entry {
    long long request;
    int n_tokens, first_token, want_last;
} llmx_planned_entry;
int llmx_engine_plan(llmx_engine*, llmx_planned_entry* out, int capacity);
int llmx_engine_book(llmx_engine*, const int* drawn, int n, llmx_step_result* out, int capacity);
// The logits of the step that ran last, [wanted, vocab] float32: copied to `out` (host, may be null); `device` (may be
// null) receives the device buffer, valid until the next step.  Returns the number of wanted places or -code.
int llmx_engine_last_logits(llmx_engine*, float* out, const float** device);
// A request's reply so far (tokens written up to `capacity`; returns their number or -code); *finished as above.
int llmx_engine_output(llmx_engine*, long long request, int* tokens, int capacity, int* finished);
int llmx_engine_forget(llmx_engine*, long long request);              // a finished request's record

// ---- accounting (tests, a caller's own policy) ---------------------------------------------------------------------
int llmx_engine_groups(llmx_engine*);
int llmx_engine_pages(llmx_engine*, int group, long long* total, long long* free_pages);
int llmx_engine_held_pages(llmx_engine*, long long request, int group);
int llmx_engine_check(llmx_engine*);        // no page lost, held twice or freed twice; 0 when so
long long llmx_engine_preemptions(llmx_engine*);
long long llmx_engine_steps(llmx_engine*);
long long llmx_engine_replays(llmx_engine*);                 // steps that replayed a recorded (CUDA graph) step
void llmx_engine_record_steps(llmx_engine*, int on);         // whether shapes that keep coming are recorded (on at the start)
long long llmx_engine_last_h2d_bytes(llmx_engine*);          // metadata bytes the last step copied to the device
int llmx_engine_vocab(llmx_engine*);
int llmx_engine_max_positions(llmx_engine*);

#ifdef __cplusplus
}  // extern "C"

#include <string>
#include <vector>

namespace llmx {

// The same engine for C++ callers.
class Engine {
public:
    struct Result { long long request; int token; int finished; };

    static Engine load(const std::string& dir, const llmx_engine_options& options) {
        return Engine(llmx_engine_load(dir.c_str(), &options));
    }
    Engine(llmx_model* model, const llmx_engine_desc& desc) : Engine(llmx_engine_create(model, &desc)) {}
    Engine(Engine&& other) noexcept : e_(other.e_) { other.e_ = nullptr; }
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;
    ~Engine() { llmx_engine_destroy(e_); }

    long long add_request(const std::vector<int>& ids, const llmx_sampling& sampling) {
        const long long id = llmx_engine_add_request(e_, ids.data(), (int)ids.size(), &sampling);
        if (id < 0) throw Error{(int)-id, llmx_engine_last_error()};
        return id;
    }
    std::vector<Result> step() {
        std::vector<llmx_step_result> raw(1024);
        const int n = llmx_engine_step(e_, raw.data(), (int)raw.size());
        if (n < 0) throw Error{-n, llmx_engine_last_error()};
        std::vector<Result> out;
        for (int i = 0; i < n; ++i) out.push_back(Result{raw[i].request, raw[i].token, raw[i].finished});
        return out;
    }
    bool idle() const { return llmx_engine_idle(e_) != 0; }
    // Float32 logits [wanted, vocab] of one batch.
    std::vector<float> forward(const std::vector<llmx_entry>& entries) {
        size_t wanted = 0;
        for (const llmx_entry& en : entries) wanted += (size_t)en.n_want;
        std::vector<float> logits(wanted * (size_t)llmx_engine_vocab(e_));
        const int err = llmx_engine_forward(e_, entries.data(), (int)entries.size(), logits.data(), nullptr);
        if (err) throw Error{err, llmx_engine_last_error()};
        return logits;
    }
    void end(long long request) { llmx_engine_end(e_, request); }
    std::vector<int> output(long long request, int* finished = nullptr) {
        std::vector<int> tokens(llmx_engine_max_positions(e_));
        const int n = llmx_engine_output(e_, request, tokens.data(), (int)tokens.size(), finished);
        if (n < 0) throw Error{-n, llmx_engine_last_error()};
        tokens.resize(n);
        return tokens;
    }
    llmx_engine* get() const { return e_; }

private:
    explicit Engine(llmx_engine* e) : e_(e) {
        if (!e_) throw Error{LLMX_ENGINE_ERR_REFUSED, llmx_engine_last_error()};
    }
    llmx_engine* e_;
};

}  // namespace llmx
#endif
