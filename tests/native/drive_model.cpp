// A C++ program that runs a model through the native runtime's header alone (no Python in the process).
//
//   drive_model DUMP_DIR KERNEL_DIR OUT_FILE
//
// DUMP_DIR holds what tests/test_native_gpu.py wrote from a model folder: `manifest.txt` (sizes, then one line per
// tensor: name, element type, element count, file) and the raw tensors.  The program uploads them, builds the
// parts (llmx_*_create) and the model, then feeds the token ids of the manifest as a portion of a prompt, a second
// portion and single tokens, each step described by an `llmx_step` whose metadata it lays out itself, over a paged
// cache whose block table it owns.  It writes the float32 logits of every position to OUT_FILE.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "llmx_runtime.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 1; } } while (0)
#define CHECK_RT(x) do { int e_ = (x); if (e_) { fprintf(stderr, "%s: %d %s\n", #x, e_, llmx_rt_last_error()); return 1; } } while (0)

struct Tensor { void* dev = nullptr; int dtype = 0; size_t count = 0; };

int main(int argc, char** argv) {
    if (argc != 4) { fprintf(stderr, "usage: drive_model DUMP_DIR KERNEL_DIR OUT_FILE\n"); return 2; }
    const std::string dir = argv[1];
    std::ifstream man(dir + "/manifest.txt");
    if (!man) { fprintf(stderr, "no manifest in %s\n", dir.c_str()); return 1; }
    int layers, hidden, heads, kv_heads, head_dim, inter, vocab, dtype, positions, page, tied;
    float eps;
    man >> layers >> hidden >> heads >> kv_heads >> head_dim >> inter >> vocab >> dtype >> eps >> positions >> page >> tied;
    int n_ids;
    man >> n_ids;
    std::vector<int> ids(n_ids);
    for (int& t : ids) man >> t;
    std::map<std::string, Tensor> T;
    std::string name, file;
    int dt;
    size_t count;
    while (man >> name >> dt >> count >> file) {
        std::ifstream f(dir + "/" + file, std::ios::binary);
        const size_t bytes = count * (dt == LLMX_DT_BF16 ? 2 : 4);
        std::vector<char> host(bytes);
        f.read(host.data(), (std::streamsize)bytes);
        if (!f) { fprintf(stderr, "short file %s\n", file.c_str()); return 1; }
        Tensor t;
        t.dtype = dt, t.count = count;
        CHECK_CUDA(cudaMalloc(&t.dev, bytes));
        CHECK_CUDA(cudaMemcpy(t.dev, host.data(), bytes, cudaMemcpyHostToDevice));
        T[name] = t;
    }
    const int bound = llmx_rt_load_kernels(argv[2]);
    if (bound <= 0) { fprintf(stderr, "no kernels bound from %s: %s\n", argv[2], llmx_rt_last_error()); return 1; }

    // ---- parts and model ----
    auto linear = [&](const std::string& n, int out, int in) {
        llmx_linear_desc d = {T.at(n).dev, dtype, out, in, 0};
        return d;
    };
    std::vector<llmx_part*> blocks;
    for (int l = 0; l < layers; ++l) {
        const std::string p = "layers." + std::to_string(l) + ".";
        llmx_attention_desc a = {};
        a.hidden = hidden, a.heads = heads, a.kv_heads = kv_heads, a.head_dim = head_dim, a.window = 0;
        a.scale = 1.0f / sqrtf((float)head_dim), a.qk_norm_eps = eps;
        a.q_norm = (const float*)T.at(p + "q_norm").dev, a.k_norm = (const float*)T.at(p + "k_norm").dev;
        a.cos = (const float*)T.at("cos").dev, a.sin = (const float*)T.at("sin").dev;
        a.rot_half = head_dim / 2, a.table_positions = positions, a.position_stream = 0;
        a.qkv = linear(p + "qkv", (heads + 2 * kv_heads) * head_dim, hidden);
        a.o = linear(p + "o", hidden, heads * head_dim);
        llmx_mlp_desc m = {};
        m.hidden = hidden, m.intermediate = inter;
        m.gate_up = linear(p + "gate_up", 2 * inter, hidden);
        m.down = linear(p + "down", hidden, inter);
        llmx_part* n1 = llmx_rmsnorm_create((const float*)T.at(p + "norm1").dev, hidden, eps, dtype);
        llmx_part* n2 = llmx_rmsnorm_create((const float*)T.at(p + "norm2").dev, hidden, eps, dtype);
        llmx_part* block = llmx_prenorm_block_create(n1, llmx_attention_create(&a), n2, llmx_gated_mlp_create(&m));
        if (!block) { fprintf(stderr, "block %d: %s\n", l, llmx_rt_last_error()); return 1; }
        blocks.push_back(block);
    }
    llmx_part* embedding = llmx_embedding_create(T.at("embed").dev, dtype, vocab, hidden);
    llmx_linear_desc head_w = linear(tied ? "embed" : "head", vocab, hidden);
    llmx_part* head = llmx_head_create(llmx_rmsnorm_create((const float*)T.at("norm").dev, hidden, eps, dtype), &head_w);
    std::vector<llmx_layer_step> order;
    for (int l = 0; l < layers; ++l) order.push_back({l, l, 1});
    llmx::Model model(embedding, blocks.data(), layers, order.data(), layers, head, hidden, vocab);

    // ---- the cache: one group, pages handed out in reverse so that page ids are not positions ----
    const int max_pages = (n_ids + page - 1) / page;
    const size_t per_layer = (size_t)max_pages * 2 * kv_heads * page * head_dim;
    const size_t el = dtype == LLMX_DT_BF16 ? 2 : 4;
    char* kv = nullptr;
    CHECK_CUDA(cudaMalloc((void**)&kv, per_layer * el * layers));
    CHECK_CUDA(cudaMemset(kv, 0, per_layer * el * layers));
    llmx_caches* caches = llmx_caches_create(layers);
    for (int l = 0; l < layers; ++l) CHECK_RT(llmx_caches_set_kv(caches, l, 0, kv + per_layer * el * l, dtype, max_pages, kv_heads, page, head_dim));
    std::vector<int> table(max_pages);
    for (int i = 0; i < max_pages; ++i) table[i] = max_pages - 1 - i;

    int *error_word = nullptr, *counters = nullptr;
    CHECK_CUDA(cudaMalloc((void**)&error_word, sizeof(int)));
    CHECK_CUDA(cudaMemset(error_word, 0, sizeof(int)));
    CHECK_CUDA(cudaMalloc((void**)&counters, LLMX_COUNTERS * sizeof(int)));
    CHECK_CUDA(cudaMemset(counters, 0, LLMX_COUNTERS * sizeof(int)));
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));

    std::vector<float> all_logits((size_t)n_ids * vocab);
    // The prompt in two portions, then single tokens.
    std::vector<int> cuts;
    const int first = n_ids * 3 / 5, second = (n_ids - first) / 2;
    cuts.push_back(first);
    if (second > 0) cuts.push_back(second);
    for (int at = first + second; at < n_ids; ++at) cuts.push_back(1);
    int history = 0;
    for (int n : cuts) {
        // Metadata, one buffer: tokens, positions, request of each row, first row, rows, history, state slots (read,
        // written), wanted rows, block table, cache slots, the plan's ints; every section on a 16-byte boundary.
        auto pad = [](int v) { return (v + 3) & ~3; };
        llmx_step s = {};
        s.rows = n, s.requests = 1, s.wanted = n, s.groups = 1, s.position_streams = 1, s.room = 0;
        int at = 0;
        auto take = [&](int ints) { const int o = at; at += pad(ints > 0 ? ints : 1); return o; };
        s.token_ids = take(n), s.positions = take(n), s.row_request = take(n), s.row_start = take(1), s.row_count = take(1);
        s.history = take(1), s.state_slots = take(1), s.state_slots_out = take(1), s.logit_rows = take(n);
        s.block_tables[0] = take(max_pages), s.table_stride[0] = max_pages, s.slots[0] = take(n), s.page_size[0] = page;
        llmx_plan* plan = llmx_plan_make(model.get(), nullptr, 0, &n, &history, 1, 0, 0);
        if (!plan) { fprintf(stderr, "plan: %s\n", llmx_rt_last_error()); return 1; }
        s.plan = plan, s.plan_offset = take(llmx_plan_ints(plan));
        std::vector<int> meta(at, 0);
        for (int i = 0; i < n; ++i) {
            const int pos = history + i;
            meta[s.token_ids + i] = ids[pos], meta[s.positions + i] = pos, meta[s.row_request + i] = 0, meta[s.logit_rows + i] = i;
            meta[s.slots[0] + i] = table[pos / page] * page + pos % page;
        }
        meta[s.row_start] = 0, meta[s.row_count] = n, meta[s.history] = history, meta[s.state_slots] = -1, meta[s.state_slots_out] = -1;
        for (int i = 0; i < max_pages; ++i) meta[s.block_tables[0] + i] = table[i];
        CHECK_RT(llmx_plan_fill(plan, &history, meta.data() + s.plan_offset));
        int* meta_dev = nullptr;
        CHECK_CUDA(cudaMalloc((void**)&meta_dev, meta.size() * sizeof(int)));
        CHECK_CUDA(cudaMemcpyAsync(meta_dev, meta.data(), meta.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
        s.meta = meta_dev, s.caches = caches, s.error_word = error_word, s.counters = counters, s.stream = stream;
        s.workspace_bytes = model.workspace(s);
        CHECK_CUDA(cudaMalloc(&s.workspace, s.workspace_bytes));
        float* logits = nullptr;
        CHECK_CUDA(cudaMalloc((void**)&logits, (size_t)n * vocab * sizeof(float)));
        try {
            model.forward(s, logits);
        } catch (const llmx::Error& e) {
            fprintf(stderr, "forward: %d %s\n", e.code, e.what);
            return 1;
        }
        CHECK_CUDA(cudaMemcpyAsync(all_logits.data() + (size_t)history * vocab, logits, (size_t)n * vocab * sizeof(float), cudaMemcpyDeviceToHost, stream));
        CHECK_CUDA(cudaStreamSynchronize(stream));
        cudaFree(logits), cudaFree(s.workspace), cudaFree(meta_dev);
        llmx_plan_free(plan);
        history += n;
    }
    int word = 0;
    CHECK_CUDA(cudaMemcpy(&word, error_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (word) { fprintf(stderr, "a kernel gave up a wait: %d\n", word); return 1; }
    std::ofstream out(argv[3], std::ios::binary);
    out.write((const char*)all_logits.data(), (std::streamsize)(all_logits.size() * sizeof(float)));
    printf("steps %zu kernels %lld\n", cuts.size(), llmx_rt_launches());
    return 0;
}
