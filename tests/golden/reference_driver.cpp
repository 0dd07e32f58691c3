// Drives mxxm-t/llmx's own CPU model code (float32 weights, float32 cache) on a tiny model whose
// weights and metadata this repository's generator wrote, and dumps the logits of every position.
// Built and run only by tests/golden/make_golden.py; it is not part of the engine.
//
//   reference_driver META MANIFEST WEIGHTS IDS OUT
//     META      lines "key u32|f32|str value" (keys without the "qwen3." prefix)
//     MANIFEST  lines "name ndim ne0 [ne1] offset_in_floats" (ne0 fastest)
//     WEIGHTS   raw little-endian float32
//     IDS       whitespace-separated token ids
//     OUT       raw float32 [tokens, vocab]: `score` (whole prompt), then the same positions
//               through single steps appended after it
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>
#include "backends/cpu/cpu_backend.hpp"
#include "format/gguf.hpp"
#include "model/runtime.hpp"
#include "model/arch/registry.hpp"
#include "model/passes.hpp"
#include "model/history.hpp"

int main(int argc, char** argv) {
    if (argc != 6) { std::fprintf(stderr, "usage: reference_driver META MANIFEST WEIGHTS IDS OUT\n"); return 2; }
    gguf::GGUFModel m;
    {
        std::ifstream in(argv[1]);
        std::string key, type, value;
        while (in >> key >> type >> value) {
            gguf::MetaValue v;
            if (type == "u32") { v.vtype = gguf::V_UINT32; v.u = std::stoull(value); }
            else if (type == "f32") { v.vtype = gguf::V_FLOAT32; float f = std::stof(value); std::memcpy(&v.fb, &f, 4); }
            else { v.vtype = gguf::V_STRING; v.s = value; }
            m.kv.push_back({"qwen3." + key, v});
        }
    }
    {
        std::ifstream w(argv[3], std::ios::binary);
        std::vector<char> all((std::istreambuf_iterator<char>(w)), std::istreambuf_iterator<char>());
        m.blob.assign(all.begin(), all.end());
        std::ifstream in(argv[2]);
        std::string line;
        while (std::getline(in, line)) {
            std::istringstream ls(line);
            std::string name; int ndim; ls >> name >> ndim;
            std::vector<uint64_t> shape(ndim);
            for (auto& d : shape) ls >> d;
            uint64_t off; ls >> off;
            m.tensors.push_back({name, shape, quant::GGML_TYPE_F32, 0});
            m.offsets.push_back(off * sizeof(float));
        }
    }
    std::vector<uint32_t> ids;
    { std::ifstream in(argv[4]); uint32_t t; while (in >> t) ids.push_back(t); }
    infer::ModelOptions o;
    o.kv_k = o.kv_v = backend::KVType::f32;
    o.dtype = backend::Dtype::f32;
    infer::Model model(infer::gguf_weights(m), backend::make_cpu_backend(), o);
    model.set_threads(1);
    const size_t V = model.n_vocab();
    std::vector<float> out;
    model.score(ids, [&](size_t, const float* row) { out.insert(out.end(), row, row + V); });
    model.reset();
    for (uint32_t id : ids) { const float* p = model.step((int)id); out.insert(out.end(), p, p + V); }
    std::ofstream f(argv[5], std::ios::binary);
    f.write((const char*)out.data(), (std::streamsize)(out.size() * sizeof(float)));
    std::printf("vocab %zu tokens %zu\n", V, ids.size());
    return 0;
}
