// llmx_b200 native runtime: the model's forward pass as host code.
//
// A step of the engine is a few hundred kernel launches whose arguments follow from the batch's shape.  This
// library makes them from native code: the parts of a layer (norm, attention, gated feed-forward, their
// arrangement in a block), the embedding and the logits head are C++ objects built once from device pointers
// to the weights, and `llmx_model_forward` walks the layer order for the rows of one step.  It is the
// counterpart of the reference's header-only model runtime (src/model/passes.hpp:13-25 `Model::forward`,
// src/model/arch/qwen3.hpp:272-312 for the layer) and is what the Python engine, `bin/trace_run` and the
// recorded (CUDA-graph) steps all run: there is one forward pass.
//
// What stays outside: files, configuration, the cache's bookkeeping and the scheduler hand this library
// pointers and numbers.  A caller describes a step with `llmx_step` (where the batch's metadata lies on the
// device, the rows each request brings, a workspace) and gets float32 logits for the wanted rows.
//
// The kernels live in libraries of their own (one per .cu file); the runtime calls them through a table that is
// filled by `llmx_rt_bind` (a caller that has the function pointers) or `llmx_rt_load_kernels` (a folder of
// built libraries).  A kernel that is not bound makes the call that needs it fail with its name.
//
// Every function returns 0 on success or an error code (a CUDA error, or one of LLMX_ERR_*);
// `llmx_rt_last_error` gives the text for the calling thread.  Nothing here synchronises the device.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLMX_RT_VERSION 2
#define LLMX_MAX_GROUPS 8

enum { LLMX_DT_F32 = 0, LLMX_DT_BF16 = 1 };
enum { LLMX_RT_ERR_BAD_ARGUMENT = 10001, LLMX_RT_ERR_UNSUPPORTED = 10002, LLMX_RT_ERR_TOO_LARGE = 10004,
       LLMX_RT_ERR_UNBOUND = 10010, LLMX_RT_ERR_WORKSPACE = 10011, LLMX_RT_ERR_CALLBACK = 10012, LLMX_RT_ERR_INJECTED = 10013 };

// Flags of a path (what `precision` means for every part built with them).
enum { LLMX_FLAG_INVARIANT = 1 };   // schedules that do not depend on what else is in the batch (see llmx_attention_desc)

typedef struct llmx_part llmx_part;       // a norm, mixer, feed-forward, block, embedding or head
typedef struct llmx_model llmx_model;
typedef struct llmx_caches llmx_caches;   // where every cache entry's storage lies
typedef struct llmx_plan llmx_plan;       // launch decisions of one step shape (see llmx_plan_make)

// ---- kernels -----------------------------------------------------------------------------------------------
int llmx_rt_version(void);
int llmx_rt_bind(const char* name, void* function);        // an exported kernel entry point, e.g. "llmx_rmsnorm"
int llmx_rt_load_kernels(const char* folder);              // every llmx_*.so of a folder; returns how many functions were bound, or < 0
const char* llmx_rt_last_error(void);
long long llmx_rt_launches(void);                          // kernels launched through the runtime so far
void llmx_rt_count_launches(long long n);                  // ... plus those a replayed recording launched
// Entry point i (from 0) that the last dry runs (llmx_*_workspace) would have called and found unbound; 0 at the end.
int llmx_rt_missing(int i, const char** name);
// Which products of many tokens may run on pairs of SMs: a sum of 1 (plain products), 2 (the gated product) and 4 (the
// q/k/v product that finishes its heads); all at the start.  Returns the setting before.
int llmx_rt_pair_products(int which);
void llmx_rt_reset_caches(void);                           // forget what was learnt of the device and the kernel libraries
// For tests of what a failed step leaves behind: the nth call (from now) of the entry point `name` fails on the host,
// before anything is launched, with LLMX_RT_ERR_INJECTED.  nth <= 0 or a null name: no failure is pending.
void llmx_rt_fail_call(const char* name, int nth);
// Device time by kernel entry point: while on, every kernel call is bracketed by events on its stream.
int llmx_rt_profile(int on);
// After llmx_rt_profile(0): entry i of the calls made while it was on.  Returns 0 when i is out of range.
int llmx_rt_profile_read(int i, const char** name, float* ms, float* idle_ms_before);

// ---- launch decisions, exposed so that one implementation serves callers and tests -------------------------
// (schedule, token tile, k ranges) of the tensor-core product out[m, n] (+)= a[m, k] w[n, k]^T.  Schedule 0: whole
// tiles, a thread block each; 1: stream-K; 2: whole tiles of 256 weight rows, a pair of thread blocks each.
void llmx_gemm_plan(int m, int n, int k, int accumulate, int sms, int* schedule, int* token_tile, int* splits);
int llmx_heads_tile(int m, int heads, int kv_heads, int sms);
// (key ranges, keys per range) of the split-KV decode kernel; clusters[s] = clusters of s blocks the device runs
// at once (s = 0..16; 0 where unknown or off).
void llmx_decode_schedule(int n_requests, int kv_heads, int max_context, int head_dim, const int* clusters,
                          int* splits, int* chunk);
// 0: only the plain attention kernel takes this shape; 1: split-KV decode and warp-level prefill; 2: and tcgen05 prefill.
int llmx_tiled_attention(int heads, int kv_heads, int head_dim, int page_size);
void llmx_prefill_shape(int n_requests, int kv_heads, int ratio, int max_rows, int max_context, int window, int sms,
                        int* tiles, int* splits);

// ---- the cache as the kernels see it ----------------------------------------------------------------------
llmx_caches* llmx_caches_create(int entries);
void llmx_caches_destroy(llmx_caches*);
// A key/value entry: storage [pages, 2, kv_heads, page_size, head_dim] of `dtype`, in cache group `group`.
int llmx_caches_set_kv(llmx_caches*, int entry, int group, void* storage, int dtype, long long pages, int kv_heads,
                       int page_size, int head_dim);
// A state entry: `slots` tensors of `bytes_per_slot` bytes each.
int llmx_caches_set_state(llmx_caches*, int entry, void* storage, long long slots, long long bytes_per_slot);

// ---- a step --------------------------------------------------------------------------------------------------
// The batch's metadata is one int32 buffer on the device; the offsets below (in ints) say where each section
// lies.  Rows are the step's tokens in entry order; request r owns rows row_start[r] .. + row_count[r], after
// history[r] tokens.
typedef struct llmx_step {
    int rows, requests, wanted, groups, position_streams, room;   // room > 0: a recorded step with room for that context
    const int* meta;                  // device
    int token_ids, positions, row_request, row_start, row_count, history, state_slots, logit_rows, state_slots_out;   // offsets
    //  (state_slots: where each request's fixed-size state lies; state_slots_out: where the step leaves it)
    int block_tables[LLMX_MAX_GROUPS], table_stride[LLMX_MAX_GROUPS], slots[LLMX_MAX_GROUPS], page_size[LLMX_MAX_GROUPS];
    int plan_offset;                  // where the plan's ints lie in `meta`
    const llmx_plan* plan;            // launch decisions for this shape (may be null when no part needs any)
    const llmx_caches* caches;
    void* workspace;                  // device scratch for the step's intermediates, 256-byte aligned
    size_t workspace_bytes;
    int* error_word;                  // device int the tensor-core kernels record a failed wait in
    int* counters;                    // device ints (LLMX_COUNTERS of them, zero) for the split-KV kernel
    void* stream;                     // cudaStream_t
} llmx_step;
#define LLMX_COUNTERS 65536

// ---- launch plans ----------------------------------------------------------------------------------------------
// A plan holds what the parts of a model decide from a step's shape before anything is launched: which
// requests run which attention kernel, how many key ranges, what scratch.  `counts[r]`: rows request r brings;
// `histories[r]`: tokens before them.  With room > 0 (a step that is recorded and replayed) every decision that
// shapes a launch is taken for a context of `room` tokens and `histories` may be null; `llmx_plan_fill` then
// writes the values that follow the actual histories.  The plan's ints go into the step's metadata at
// llmx_step.plan_offset.
llmx_plan* llmx_plan_make(const llmx_model* model, llmx_part* const* parts, int n_parts, const int* counts,
                          const int* histories, int requests, int room, int typical_context);
//   (of a whole model and/or of single parts; typical_context: with room > 0, the context the recorded step is likely to
//    meet, which shapes only what is a matter of speed; 0: none known)
int llmx_plan_ints(const llmx_plan*);
int llmx_plan_fill(llmx_plan*, const int* histories, int* out);
void llmx_plan_free(llmx_plan*);
// Forces the tcgen05 prefill attention's item shape (tests): row tiles an item (1, 2; 0 free), key ranges (0 free).
void llmx_plan_force_prefill_shape(llmx_plan*, int tiles, int splits);
// Forces the split-KV decode kernel's key ranges and keys per range (a multiple of 64) (tests).
void llmx_plan_force_decode(llmx_plan*, int splits, int chunk);
// What the plan decided for the first attention shape: out[0..7] = small requests, large requests, splits, chunk,
// prefill tiles, prefill splits, rows of the largest small request, rows of the largest large one.
int llmx_plan_describe(const llmx_plan*, int* out);

// ---- parts -----------------------------------------------------------------------------------------------------
typedef struct llmx_linear_desc {
    const void* weight;     // [out_features, in_features] row-major on the device, of `dtype`
    int dtype, out_features, in_features, flags;
} llmx_linear_desc;

typedef struct llmx_attention_desc {
    int hidden, heads, kv_heads, head_dim, window;     // window 0: every key
    float scale, qk_norm_eps;
    const float* q_norm;    // [head_dim] or null (no per-head norm)
    const float* k_norm;
    const float* cos;       // [positions, rot_half] or null (no rotation)
    const float* sin;
    int rot_half, table_positions, position_stream;
    llmx_linear_desc qkv;   // stacked rows: queries, keys, values
    llmx_linear_desc o;
    int flags;
} llmx_attention_desc;

typedef struct llmx_mlp_desc {
    int hidden, intermediate;
    llmx_linear_desc gate_up;   // stacked rows: gate, up
    llmx_linear_desc down;
    int flags;
} llmx_mlp_desc;

// A block, mixer or feed-forward written elsewhere (another language, a test): called with the step and the rows.
// kind 0 block(x), 1 mixer(h, residual), 2 feed-forward(h, residual).  Returns 0 or an error code.
typedef int (*llmx_callback)(void* user, const llmx_step* step, int kind, void* h, float* x_or_residual, int rows,
                             int cache_entry, int write_cache);

llmx_part* llmx_rmsnorm_create(const float* weight, int width, float eps, int out_dtype);
llmx_part* llmx_attention_create(const llmx_attention_desc*);
llmx_part* llmx_gated_mlp_create(const llmx_mlp_desc*);
llmx_part* llmx_linear_create(const llmx_linear_desc*);
llmx_part* llmx_prenorm_block_create(llmx_part* mixer_norm, llmx_part* mixer, llmx_part* ffn_norm, llmx_part* ffn);
llmx_part* llmx_callback_create(int kind, llmx_callback fn, void* user, int hidden);
llmx_part* llmx_embedding_create(const void* table, int dtype, int vocab, int width);
llmx_part* llmx_head_create(llmx_part* norm, const llmx_linear_desc* weight);
void llmx_part_destroy(llmx_part*);      // parts do not own the parts they were built from
// New tables for an attention part (the engine sizes them when the cache is made).
int llmx_attention_set_tables(llmx_part*, const float* cos, const float* sin, int rot_half, int positions);

// One part alone (each is what the model's forward calls).  Activations `h` have the part's path type.
int llmx_norm_forward(llmx_part*, const llmx_step*, const float* x, void* out, int out_dtype, const int* row_index,
                      int rows, float* zero, long long zero_count);
int llmx_mixer_forward(llmx_part*, const llmx_step*, const void* h, int rows, int cache_entry, float* residual,
                       int write_cache, float* cleared);   // `cleared`: what llmx_part_wants_cleared gave, already zero
int llmx_ffn_forward(llmx_part*, const llmx_step*, const void* h, int rows, float* residual, float* cleared);
int llmx_block_forward(llmx_part*, const llmx_step*, float* x, int rows, int cache_entry, int write_cache);
int llmx_embedding_forward(llmx_part*, const llmx_step*, const int* ids, float* x, int rows);
int llmx_head_forward(llmx_part*, const llmx_step*, const float* x, float* logits);
int llmx_linear_forward(llmx_part*, const llmx_step*, const void* a, int rows, float* out, int accumulate, int cleared);
int llmx_linear_gated(llmx_part*, const llmx_step*, const void* a, int rows, void* out);
// Floats (a multiple of 4, or 0) a mixer or feed-forward wants zeroed before its forward for this many rows: the
// norm in front of it clears them in passing.  The buffer itself is the caller's.
long long llmx_part_wants_cleared(llmx_part*, const llmx_step*, int rows);
int llmx_linear_adds_pieces(llmx_part*, int rows);
// Workspace bytes one call of the part's forward (on this cache entry, where it has one) needs for this step.  The
// walk also notes the kernels it would call and that are not bound (llmx_rt_missing).
size_t llmx_part_workspace(llmx_part*, const llmx_step*, int rows, int cache_entry);

// The attention kernels alone, as a mixer runs them once its queries are made: out = attention of the step's rows
// (q/out [rows, heads * head_dim] of q_dtype) over cache entry `entry`.
llmx_part* llmx_attention_shape(int heads, int kv_heads, int head_dim, int window);   // a mixer's shape alone, for plans
int llmx_paged_attention(const llmx_step*, const void* q, int q_dtype, int entry, void* out, int heads, int kv_heads,
                         int head_dim, int window, float scale);
size_t llmx_paged_attention_workspace(const llmx_step*, int entry, int heads, int kv_heads, int head_dim, int window);
// The decode kernel taking the q/k/v product's float32 output as it is (steps of decoding rows only).  0: ran;
// -1: the step or the shapes do not qualify and nothing was done.
int llmx_decode_from_qkv(const llmx_step*, const float* qkv, int entry, const float* q_weight, const float* k_weight,
                         float eps, const float* cos, const float* sin, int rot_half, void* out, int heads, int kv_heads,
                         int head_dim, int window, float scale);

// ---- the model ------------------------------------------------------------------------------------------------
typedef struct llmx_layer_step { int block, cache_entry, write_cache; } llmx_layer_step;   // cache_entry < 0: none
llmx_model* llmx_model_create(llmx_part* embedding, llmx_part* const* blocks, int n_blocks, const llmx_layer_step* order,
                              int n_order, llmx_part* head, int hidden, int vocab);
void llmx_model_destroy(llmx_model*);
size_t llmx_model_workspace(const llmx_model*, const llmx_step*);
// The step's rows through every layer in order; float32 logits [wanted, vocab] (ignored when nothing is wanted).
int llmx_model_forward(llmx_model*, const llmx_step*, float* logits);

#ifdef __cplusplus
}  // extern "C"

// A thin C++ face over the same objects, for programs that link the runtime directly.
namespace llmx {
struct Error { int code; const char* what; };
inline void check(int code) { if (code) throw Error{code, llmx_rt_last_error()}; }

class Model {
public:
    Model(llmx_part* embedding, llmx_part* const* blocks, int n_blocks, const llmx_layer_step* order, int n_order,
          llmx_part* head, int hidden, int vocab)
        : m_(llmx_model_create(embedding, blocks, n_blocks, order, n_order, head, hidden, vocab)) {
        if (!m_) throw Error{LLMX_RT_ERR_BAD_ARGUMENT, llmx_rt_last_error()};
    }
    ~Model() { llmx_model_destroy(m_); }
    Model(const Model&) = delete;
    Model& operator=(const Model&) = delete;
    size_t workspace(const llmx_step& step) const { return llmx_model_workspace(m_, &step); }
    void forward(const llmx_step& step, float* logits) { check(llmx_model_forward(m_, &step, logits)); }
    llmx_model* get() const { return m_; }
private:
    llmx_model* m_;
};
}  // namespace llmx
#endif
