// Files to a model, natively: config.json (strictly read), safetensors by tensor name, the architecture's parts put
// together through the runtime's C interface (llmx_runtime.h).  `llmx_engine_load` is the reference's
// `infer::load_model` (src/inference/load.hpp:74-94, :769): the model class is chosen by config.json through one
// registry from architecture name to builder (src/model/architecture.hpp:73-86).
//
// What is checked where the reference checks it: the key table and value rules of the architecture
// (src/model/arch/qwen3.hpp:47-139, rope scaling src/model/arch/hf_config.hpp:125-155), the file-level rules of
// safetensors (src/format/safetensors.hpp:20-138), and the model-level comparison of tensors, which names every
// missing, unexpected and ill-shaped tensor in one error (the reference refuses them one at a time:
// src/model/arch/hf_config.hpp:317-336, src/model/weights.hpp:77-92).
#include "engine_internal.h"

#include <fcntl.h>
#include <math.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <functional>
#include <map>
#include <set>

namespace llmx_engine_detail {

// ---------------------------------------------------------------------------------------------------------------
// JSON: a small strict reader (objects keep their keys' order; a repeated key is an error).
// ---------------------------------------------------------------------------------------------------------------
struct Json {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    bool integral = false;      // a number written without fraction or exponent, within 64 bits
    long long i = 0;
    double num = 0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
    const Json* get(const std::string& key) const {
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is_int() const { return kind == NUM && integral; }
    std::string show() const {
        switch (kind) {
            case NUL: return "null";
            case BOOL: return b ? "true" : "false";
            case NUM: {
                char buf[64];
                if (integral) snprintf(buf, sizeof buf, "%lld", i);
                else snprintf(buf, sizeof buf, "%g", num);
                return buf;
            }
            case STR: return "\"" + str + "\"";
            case ARR: {
                std::string s = "[";
                for (size_t k = 0; k < arr.size(); ++k) s += (k ? ", " : "") + arr[k].show();
                return s + "]";
            }
            default: return "{...}";
        }
    }
};

class JsonReader {
public:
    JsonReader(const char* text, size_t n) : p_(text), end_(text + n) {}
    Json parse() {
        Json v = value(0);
        space();
        if (p_ != end_) bad("text after the value");
        return v;
    }

private:
    const char* p_;
    const char* end_;
    [[noreturn]] void bad(const std::string& what) { throw Failure{LLMX_ENGINE_ERR_FILE, "not JSON: " + what}; }
    void space() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool take(const char* word) {
        const size_t n = strlen(word);
        if ((size_t)(end_ - p_) >= n && !memcmp(p_, word, n)) {
            p_ += n;
            return true;
        }
        return false;
    }
    std::string string() {
        std::string out;
        ++p_;      // the opening quote
        while (true) {
            if (p_ >= end_) bad("an unterminated string");
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') return out;
            if (c < 0x20) bad("a control character in a string");
            if (c != '\\') {
                out += (char)c;
                continue;
            }
            if (p_ >= end_) bad("an unterminated escape");
            const char e = *p_++;
            switch (e) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    if (end_ - p_ < 4) bad("a short \\u escape");
                    unsigned cp = 0;
                    for (int k = 0; k < 4; ++k) {
                        const char h = *p_++;
                        cp = cp * 16 + (h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : 99);
                        if (cp > 0xFFFF * 16) bad("a bad \\u escape");
                    }
                    // UTF-8 of the code unit (names here are ASCII; surrogate pairs are kept as they come)
                    if (cp < 0x80) out += (char)cp;
                    else if (cp < 0x800) out += (char)(0xC0 | (cp >> 6)), out += (char)(0x80 | (cp & 0x3F));
                    else out += (char)(0xE0 | (cp >> 12)), out += (char)(0x80 | ((cp >> 6) & 0x3F)), out += (char)(0x80 | (cp & 0x3F));
                    break;
                }
                default: bad("an unknown escape");
            }
        }
    }
    Json number() {
        const char* start = p_;
        if (p_ < end_ && *p_ == '-') ++p_;
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') bad("a number without digits");
        if (*p_ == '0' && p_ + 1 < end_ && p_[1] >= '0' && p_[1] <= '9') bad("a number with a leading zero");
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        bool integral = true;
        if (p_ < end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') bad("a fraction without digits");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') bad("an exponent without digits");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        const std::string text(start, p_);
        Json v;
        v.kind = Json::NUM;
        v.num = strtod(text.c_str(), nullptr);
        if (integral && text.size() <= 18) {
            v.integral = true;
            v.i = strtoll(text.c_str(), nullptr, 10);
        }
        return v;
    }
    Json value(int depth) {
        if (depth > 64) bad("nesting too deep");
        space();
        if (p_ >= end_) bad("an empty value");
        Json v;
        const char c = *p_;
        if (c == '{') {
            ++p_;
            v.kind = Json::OBJ;
            space();
            if (p_ < end_ && *p_ == '}') { ++p_; return v; }
            while (true) {
                space();
                if (p_ >= end_ || *p_ != '"') bad("an object key that is not a string");
                std::string key = string();
                if (v.get(key)) throw Failure{LLMX_ENGINE_ERR_FILE, "repeats the key \"" + key + "\""};
                space();
                if (p_ >= end_ || *p_++ != ':') bad("a key without a colon");
                v.obj.emplace_back(std::move(key), value(depth + 1));
                space();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return v; }
                bad("an object that does not end");
            }
        }
        if (c == '[') {
            ++p_;
            v.kind = Json::ARR;
            space();
            if (p_ < end_ && *p_ == ']') { ++p_; return v; }
            while (true) {
                v.arr.push_back(value(depth + 1));
                space();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return v; }
                bad("an array that does not end");
            }
        }
        if (c == '"') {
            v.kind = Json::STR;
            v.str = string();
            return v;
        }
        if (take("true")) { v.kind = Json::BOOL; v.b = true; return v; }
        if (take("false")) { v.kind = Json::BOOL; v.b = false; return v; }
        if (take("null")) return v;
        if (c == '-' || (c >= '0' && c <= '9')) return number();
        bad(std::string("an unexpected character '") + c + "'");
    }
};

static std::string read_text(const std::string& path, const std::string& absent) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) throw Failure{LLMX_ENGINE_ERR_FILE, absent};
    std::string text;
    char buf[65536];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, n);
    fclose(f);
    return text;
}

// ---------------------------------------------------------------------------------------------------------------
// The dense Qwen3 configuration: every key of config.json must be one the architecture knows.
// ---------------------------------------------------------------------------------------------------------------
struct Yarn {
    bool on = false;
    double factor = 1, beta_fast = 32, beta_slow = 1;
    long long original = 0;
    double attention_factor() const { return 0.1 * log(factor) + 1.0; }      // on cos and sin (src/model/rope.hpp:145)
};
struct Qwen3Config {
    long long layers = 0, hidden = 0, intermediate = 0, heads = 0, kv_heads = 0, head_dim = 0, vocab = 0, max_positions = 4096;
    double rope_theta = 10000.0, eps = 1e-6;
    bool tied = false;
    Yarn yarn;
    std::vector<int> eos_ids;
};

static Qwen3Config read_qwen3(const Json& raw) {
    const char* where = "qwen3";
    auto bad = [&](const std::string& what) -> void { throw Failure{LLMX_ENGINE_ERR_FILE, std::string(where) + ": " + what}; };
    static const char* integers[] = {"num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads",
                                     "head_dim", "max_position_embeddings", "vocab_size"};
    static const char* required[] = {"num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads", "vocab_size"};
    static const char* reals[] = {"rope_theta", "rms_norm_eps"};
    static const char* kept[] = {"rope_scaling", "bos_token_id", "eos_token_id", "pad_token_id"};
    static const char* ignored[] = {"attention_dropout", "initializer_range", "max_window_layers", "sliding_window",
                                    "transformers_version", "use_cache", "unsloth_fixed"};
    static const char* checked[] = {"attention_bias", "hidden_act", "use_sliding_window", "layer_types", "torch_dtype", "dtype",
                                    "architectures", "model_type", "tie_word_embeddings"};
    auto in = [](const std::string& k, const char* const* list, size_t n) {
        for (size_t i = 0; i < n; ++i)
            if (k == list[i]) return true;
        return false;
    };
#define IN(k, list) in(k, list, sizeof list / sizeof list[0])
    std::vector<std::string> unknown, missing;
    for (const auto& kv : raw.obj)
        if (!IN(kv.first, integers) && !IN(kv.first, reals) && !IN(kv.first, kept) && !IN(kv.first, ignored) && !IN(kv.first, checked))
            unknown.push_back(kv.first);
    std::sort(unknown.begin(), unknown.end());
    auto joined = [](const std::vector<std::string>& v) {
        std::string s;
        for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + v[i];
        return s;
    };
    if (!unknown.empty()) bad("unknown config.json key(s): " + joined(unknown));
    for (const char* k : required)
        if (!raw.get(k)) missing.push_back(k);
    std::sort(missing.begin(), missing.end());
    if (!missing.empty()) bad("missing config.json key(s): " + joined(missing));
#undef IN
    Qwen3Config c;
    auto integer = [&](const char* key, long long& out) {
        const Json* v = raw.get(key);
        if (!v) return false;
        if (!v->is_int() || v->i < 1) bad(std::string(key) + " must be an integer >= 1, got " + v->show());
        out = v->i;
        return true;
    };
    integer("num_hidden_layers", c.layers);
    integer("hidden_size", c.hidden);
    integer("intermediate_size", c.intermediate);
    integer("num_attention_heads", c.heads);
    integer("vocab_size", c.vocab);
    integer("max_position_embeddings", c.max_positions);
    if (!integer("num_key_value_heads", c.kv_heads)) c.kv_heads = c.heads;
    if (!integer("head_dim", c.head_dim)) {
        if (c.hidden % c.heads) bad("embedding width does not determine an integral head width");
        c.head_dim = c.hidden / c.heads;
    }
    auto real = [&](const char* key, double& out) {
        const Json* v = raw.get(key);
        if (!v) return;
        if (v->kind != Json::NUM || !std::isfinite(v->num)) bad(std::string(key) + " must be a finite number, got " + v->show());
        out = v->num;
    };
    real("rope_theta", c.rope_theta);
    real("rms_norm_eps", c.eps);
    if (const Json* v = raw.get("tie_word_embeddings")) {
        if (v->kind != Json::BOOL) bad("tie_word_embeddings must be true or false, got " + v->show());
        c.tied = v->b;
    }
    auto one_of = [&](const char* key, std::initializer_list<const char*> allowed) {
        const Json* v = raw.get(key);
        if (!v) return;
        for (const char* a : allowed)
            if (v->kind == Json::STR && v->str == a) return;
        std::string list;
        for (const char* a : allowed) list += std::string(list.empty() ? "" : ", ") + "'" + a + "'";
        bad(std::string(key) + " must be one of [" + list + "], got " + v->show());
    };
    one_of("hidden_act", {"silu"});
    one_of("torch_dtype", {"bfloat16", "float16", "float32"});
    one_of("dtype", {"bfloat16", "float16", "float32"});
    one_of("model_type", {"qwen3"});
    for (const char* key : {"attention_bias", "use_sliding_window"})
        if (const Json* v = raw.get(key))
            if (v->kind != Json::BOOL || v->b) bad(std::string(key) + " must be one of [False], got " + v->show());
    if (const Json* v = raw.get("layer_types")) {
        bool ok = v->kind == Json::ARR;
        if (ok)
            for (const Json& t : v->arr) ok = ok && t.kind == Json::STR && t.str == "full_attention";
        if (!ok) bad("every entry of layer_types must be one of ['full_attention'], got " + v->show());
    }
    if (const Json* v = raw.get("architectures"))
        if (v->kind != Json::ARR || v->arr.size() != 1 || v->arr[0].kind != Json::STR || v->arr[0].str != "Qwen3ForCausalLM")
            bad("architectures must be [\"Qwen3ForCausalLM\"]");
    if (c.heads % c.kv_heads) bad("head count must be divisible by KV head count");
    if (c.head_dim <= 0 || c.head_dim % 2) bad("invalid attention projection dimensions (head_dim must be even and positive)");
    if (!(c.rope_theta > 0)) bad("invalid rope base");
    if (!(c.eps >= 0)) bad("rms_norm_eps must not be negative");
    // rope_scaling: null, or YaRN with the keys this engine reads
    if (const Json* rs = raw.get("rope_scaling")) {
        if (rs->kind != Json::NUL) {
            if (rs->kind != Json::OBJ) bad("rope_scaling is not an object or null");
            if (!rs->get("rope_type") && !rs->get("type")) bad("rope_scaling gives no rope_type");
            for (const char* k : {"rope_type", "type"})
                if (const Json* t = rs->get(k))
                    if (t->kind != Json::STR || t->str != "yarn") bad(std::string("rope_scaling.") + k + " = " + t->show() + " is not supported (\"yarn\")");
            for (const auto& kv : rs->obj) {
                const std::string& k = kv.first;
                if (k == "attention_factor" || k == "mscale" || k == "mscale_all_dim") bad("rope_scaling." + k + " is not supported");
                if (k != "rope_type" && k != "type" && k != "factor" && k != "original_max_position_embeddings" && k != "beta_fast" && k != "beta_slow")
                    bad("rope_scaling." + k + " is not a key this engine reads");
            }
            if (!rs->get("factor")) bad("rope_scaling gives no factor");
            auto rreal = [&](const char* k, double fallback) {
                const Json* v = rs->get(k);
                if (!v) return fallback;
                if (v->kind != Json::NUM || !std::isfinite(v->num)) bad(std::string("rope_scaling.") + k + " must be a finite number, got " + v->show());
                return v->num;
            };
            c.yarn.on = true;
            c.yarn.factor = rreal("factor", 1.0);
            if (!(c.yarn.factor > 1.0)) bad("rope_scaling.factor must be above 1 for YaRN");
            c.yarn.original = c.max_positions;
            if (const Json* o = rs->get("original_max_position_embeddings")) {
                if (!o->is_int() || o->i < 1) bad("rope_scaling.original_max_position_embeddings must be a positive integer, got " + o->show());
                c.yarn.original = o->i;
            }
            c.yarn.beta_fast = rreal("beta_fast", 32.0);
            c.yarn.beta_slow = rreal("beta_slow", 1.0);
            if (!(c.yarn.beta_fast > c.yarn.beta_slow)) bad("rope_scaling.beta_fast must be above beta_slow");
        }
    }
    for (const char* k : {"bos_token_id", "eos_token_id", "pad_token_id"}) {
        const Json* v = raw.get(k);
        if (!v || v->kind == Json::NUL) continue;
        bool ok = v->is_int();
        if (v->kind == Json::ARR) {
            ok = true;
            for (const Json& x : v->arr) ok = ok && x.is_int();
        }
        if (!ok) bad(std::string(k) + " must be an integer, a list of integers or null, got " + v->show());
        if (!strcmp(k, "eos_token_id")) {
            if (v->kind == Json::ARR)
                for (const Json& x : v->arr) c.eos_ids.push_back((int)x.i);
            else
                c.eos_ids.push_back((int)v->i);
        }
    }
    return c;
}

// ---------------------------------------------------------------------------------------------------------------
// safetensors: 8 bytes of header length, a JSON header (name -> dtype, shape, data_offsets), the data.
// ---------------------------------------------------------------------------------------------------------------
struct TensorEntry {
    std::string dtype;
    std::vector<long long> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
    long long count() const {
        long long n = 1;
        for (long long d : shape) n *= d;
        return n;
    }
};
struct MappedFile {
    void* base = nullptr;
    size_t size = 0;
    ~MappedFile() {
        if (base) munmap(base, size);
    }
};
struct TensorFiles {
    std::vector<std::unique_ptr<MappedFile>> files;
    std::map<std::string, TensorEntry> tensors;

    void add_file(const std::string& path) {
        auto bad = [&](const std::string& what) -> void { throw Failure{LLMX_ENGINE_ERR_FILE, path + ": " + what}; };
        const int fd = open(path.c_str(), O_RDONLY);
        if (fd < 0) bad("cannot be opened");
        struct stat st;
        if (fstat(fd, &st) != 0) {
            close(fd);
            bad("cannot be measured");
        }
        std::unique_ptr<MappedFile> m(new MappedFile);
        m->size = (size_t)st.st_size;
        if (m->size < 8) {
            close(fd);
            bad("shorter than a safetensors header");
        }
        m->base = mmap(nullptr, m->size, PROT_READ, MAP_PRIVATE, fd, 0);
        close(fd);
        if (m->base == MAP_FAILED) {
            m->base = nullptr;
            bad("cannot be mapped");
        }
        const unsigned char* p = (const unsigned char*)m->base;
        unsigned long long n = 0;
        for (int k = 7; k >= 0; --k) n = (n << 8) | p[k];
        if (n > 100ull * 1024 * 1024) bad("header of " + std::to_string(n) + " bytes exceeds " + std::to_string(100 * 1024 * 1024));
        if (8 + n > m->size) bad("header runs past the end of the file");
        Json head;
        try {
            head = JsonReader((const char*)p + 8, (size_t)n).parse();
        } catch (const Failure& f) {
            bad("header " + f.what);
        }
        if (head.kind != Json::OBJ) bad("header is not a JSON object");
        const size_t base = 8 + (size_t)n;
        std::vector<std::pair<size_t, size_t>> spans;
        for (const auto& kv : head.obj) {
            const std::string& name = kv.first;
            if (name == "__metadata__") continue;
            const Json& e = kv.second;
            if (e.kind != Json::OBJ || e.obj.size() != 3 || !e.get("dtype") || !e.get("shape") || !e.get("data_offsets"))
                bad("tensor '" + name + "' must have exactly dtype, shape and data_offsets");
            TensorEntry t;
            const Json* dt = e.get("dtype");
            static const std::map<std::string, int> widths = {{"F32", 4}, {"F16", 2}, {"BF16", 2}, {"F64", 8}, {"I64", 8}, {"I32", 4},
                                                              {"I16", 2}, {"I8", 1}, {"U8", 1}, {"BOOL", 1}};
            if (dt->kind != Json::STR || !widths.count(dt->str)) bad("tensor '" + name + "' has unsupported dtype " + dt->show());
            t.dtype = dt->str;
            const int width = widths.at(t.dtype);
            const Json* sh = e.get("shape");
            bool ok = sh->kind == Json::ARR && sh->arr.size() <= 5;
            if (ok)
                for (const Json& d : sh->arr) ok = ok && d.is_int() && d.i >= 0;
            if (!ok) bad("tensor '" + name + "' has an invalid shape " + sh->show());
            for (const Json& d : sh->arr) t.shape.push_back(d.i);
            const Json* off = e.get("data_offsets");
            if (off->kind != Json::ARR || off->arr.size() != 2 || !off->arr[0].is_int() || !off->arr[1].is_int() || off->arr[0].i < 0 ||
                off->arr[0].i > off->arr[1].i)
                bad("tensor '" + name + "' has invalid data_offsets " + off->show());
            const size_t a = (size_t)off->arr[0].i, b = (size_t)off->arr[1].i;
            if ((long long)(b - a) != t.count() * width)
                bad("tensor '" + name + "': offsets span " + std::to_string(b - a) + " bytes, shape " + sh->show() + " of " + t.dtype + " needs " +
                    std::to_string(t.count() * width));
            if (base + b > m->size) bad("tensor '" + name + "' runs past the end of the file");
            t.data = p + base + a;
            t.bytes = b - a;
            if (tensors.count(name)) bad("tensor '" + name + "' is also in another file of the folder");
            tensors[name] = std::move(t);
            if (b > a) spans.emplace_back(a, b);
        }
        std::sort(spans.begin(), spans.end());
        size_t at = 0;
        for (const auto& s : spans) {
            if (s.first != at) bad(s.first < at ? "tensors overlap" : "a gap between tensors");
            at = s.second;
        }
        if (base + at != m->size) bad("data does not end at the end of the file");
        files.push_back(std::move(m));
    }

    // The files of a model folder: those its model.safetensors.index.json names, each holding exactly the tensors the
    // index maps to it, or its single model.safetensors (src/format/safetensors.hpp:133-171).
    void add_folder(const std::string& dir) {
        const std::string index = dir + "/model.safetensors.index.json";
        struct stat st;
        if (stat(index.c_str(), &st) != 0) {
            const std::string single = dir + "/model.safetensors";
            if (stat(single.c_str(), &st) != 0)
                throw Failure{LLMX_ENGINE_ERR_FILE, dir + ": neither model.safetensors nor model.safetensors.index.json"};
            add_file(single);
            return;
        }
        auto bad = [&](const std::string& what) -> void { throw Failure{LLMX_ENGINE_ERR_FILE, index + ": " + what}; };
        const std::string text = read_text(index, index + ": cannot be read");
        Json root;
        try {
            root = JsonReader(text.data(), text.size()).parse();
        } catch (const Failure& f) {
            bad(f.what);
        }
        const Json* map = root.kind == Json::OBJ ? root.get("weight_map") : nullptr;
        if (!map || map->kind != Json::OBJ) bad("weight_map must map tensor names to file names");
        std::map<std::string, std::set<std::string>> named;       // file -> the tensors the index gives it
        for (const auto& kv : map->obj) {
            if (kv.second.kind != Json::STR) bad("weight_map must map tensor names to file names");
            const std::string& file = kv.second.str;
            if (file.empty() || file == "." || file == ".." || file.find_first_of("/\\:") != std::string::npos)
                bad("'" + file + "' names a path outside the model folder");
            named[file].insert(kv.first);
        }
        for (const auto& item : named) {
            std::set<std::string> had;
            for (const auto& t : tensors) had.insert(t.first);
            add_file(dir + "/" + item.first);
            std::vector<std::string> differ;
            for (const auto& t : tensors)
                if (!had.count(t.first) && !item.second.count(t.first)) differ.push_back(t.first);
            for (const std::string& name : item.second)
                if (!tensors.count(name) || had.count(name)) differ.push_back(name);
            if (!differ.empty()) {
                std::sort(differ.begin(), differ.end());
                std::string list;
                for (size_t i = 0; i < differ.size() && i < 8; ++i) list += (i ? ", " : "") + differ[i];
                bad("weight_map and " + item.first + " disagree on " + list);
            }
        }
    }
};

// ---------------------------------------------------------------------------------------------------------------
// Weights onto the device.  Matrices take the path's type (bfloat16 or float32; a bfloat16 file widened to float32 is
// exact, a float32 file rounded to bfloat16 is round-to-nearest-even); vectors of norms are always float32.
// ---------------------------------------------------------------------------------------------------------------
static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);      // a NaN stays one
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
static inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while (!(m & 0x400));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// `count` values of a stored tensor into `dst` as `dtype` (LLMX_DT_*).
static void convert(const TensorEntry& t, int dtype, void* dst) {
    const long long n = t.count();
    if (dtype == LLMX_DT_F32) {
        float* out = (float*)dst;
        if (t.dtype == "F32") memcpy(out, t.data, (size_t)n * 4);
        else if (t.dtype == "BF16")
            for (long long i = 0; i < n; ++i) { uint16_t v; memcpy(&v, t.data + 2 * i, 2); out[i] = bf16_to_f32(v); }
        else
            for (long long i = 0; i < n; ++i) { uint16_t v; memcpy(&v, t.data + 2 * i, 2); out[i] = f16_to_f32(v); }
    } else {
        uint16_t* out = (uint16_t*)dst;
        if (t.dtype == "BF16") memcpy(out, t.data, (size_t)n * 2);
        else if (t.dtype == "F32")
            for (long long i = 0; i < n; ++i) { float v; memcpy(&v, t.data + 4 * i, 4); out[i] = f32_to_bf16(v); }
        else
            for (long long i = 0; i < n; ++i) { uint16_t v; memcpy(&v, t.data + 2 * i, 2); out[i] = f32_to_bf16(f16_to_f32(v)); }
    }
}

struct DeviceWeights {
    std::vector<void*> blocks;
    ~DeviceWeights() {
        for (void* p : blocks) cudaFree(p);
    }
    // The tensors `names`, one after the other (stacked rows), on the device as `dtype`.
    void* upload(const TensorFiles& files, const std::vector<std::string>& names, int dtype) {
        size_t total = 0;
        const size_t elem = dtype == LLMX_DT_BF16 ? 2 : 4;
        for (const std::string& n : names) total += (size_t)files.tensors.at(n).count() * elem;
        std::vector<unsigned char> host(total);
        size_t at = 0;
        for (const std::string& n : names) {
            const TensorEntry& t = files.tensors.at(n);
            convert(t, dtype, host.data() + at);
            at += (size_t)t.count() * elem;
        }
        void* dev = nullptr;
        if (cudaMalloc(&dev, std::max<size_t>(total, 256)) != cudaSuccess)
            throw Failure{LLMX_ENGINE_ERR_DEVICE, "allocating " + std::to_string(total) + " bytes for weights failed"};
        blocks.push_back(dev);
        if (cudaMemcpy(dev, host.data(), total, cudaMemcpyHostToDevice) != cudaSuccess)
            throw Failure{LLMX_ENGINE_ERR_DEVICE, "copying weights to the device failed"};
        return dev;
    }
    void* upload_raw(const void* host, size_t bytes) {
        void* dev = nullptr;
        if (cudaMalloc(&dev, std::max<size_t>(bytes, 256)) != cudaSuccess || cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess)
            throw Failure{LLMX_ENGINE_ERR_DEVICE, "allocating or copying a table failed"};
        blocks.push_back(dev);
        return dev;
    }
};

// Rotation tables in float32, in the reference's order of operations (src/model/rope.hpp:25-28 base frequency, :159-188
// the YaRN blend, :191-217 the fill): freq_i = powf(theta, -2 i / D); angle = (float) pos * freq_i; cos/sin of it, times
// the attention factor under YaRN; indexed [pos, i], i < D / 2.
static void rope_tables(const Qwen3Config& c, long long positions, std::vector<float>& cos_t, std::vector<float>& sin_t) {
    const int dim = (int)c.head_dim, half = dim / 2;
    std::vector<float> freq(half);
    const float theta = (float)c.rope_theta;
    if (!c.yarn.on) {
        for (int i = 0; i < half; ++i) freq[i] = powf(theta, -2.0f * (float)i / (float)dim);
    } else {
        auto correction = [&](double rotations) {
            return dim * log((double)c.yarn.original / (rotations * 2 * M_PI)) / (2 * log(c.rope_theta));
        };
        double low = std::max(floor(correction(c.yarn.beta_fast)), 0.0);
        double high = std::min(ceil(correction(c.yarn.beta_slow)), (double)(dim - 1));
        if (low == high) high += 0.001;
        for (int i = 0; i < half; ++i) {
            const float power = powf(theta, (2.0f * (float)i) / (float)dim);
            const float extra = 1.0f / power, inter = 1.0f / ((float)c.yarn.factor * power);
            float ramp = ((float)i - (float)low) / (float)(high - low);
            ramp = ramp < 0.0f ? 0.0f : ramp > 1.0f ? 1.0f : ramp;
            const float extrapolate = 1.0f - ramp;
            freq[i] = inter * (1.0f - extrapolate) + extra * extrapolate;
        }
    }
    const float scale = c.yarn.on ? (float)c.yarn.attention_factor() : 1.0f;
    cos_t.resize((size_t)positions * half);
    sin_t.resize((size_t)positions * half);
    for (long long p = 0; p < positions; ++p)
        for (int i = 0; i < half; ++i) {
            const float angle = (float)p * freq[i];
            float cv = cosf(angle), sv = sinf(angle);
            if (c.yarn.on) cv *= scale, sv *= scale;
            cos_t[(size_t)p * half + i] = cv;
            sin_t[(size_t)p * half + i] = sv;
        }
}

// ---------------------------------------------------------------------------------------------------------------
// A loaded dense Qwen3: per layer a pre-norm residual block of grouped-query attention with per-head q/k RMSNorm before
// the rotation, and a SwiGLU feed-forward; a final RMSNorm and a head that is the embedding when tie_word_embeddings
// (src/model/arch/qwen3.hpp:272-312; tensor names, Hugging Face's, :140-153).
// ---------------------------------------------------------------------------------------------------------------
struct Qwen3Model : LoadedModel {
    DeviceWeights weights;
    std::vector<llmx_part*> parts;       // everything made, to be destroyed
    ~Qwen3Model() override {
        if (model) llmx_model_destroy(model);
        for (llmx_part* p : parts) llmx_part_destroy(p);
    }
};

static std::string shape_text(const std::vector<long long>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); ++i) out += (i ? ", " : "") + std::to_string(s[i]);
    return out + "]";
}

static std::unique_ptr<LoadedModel> load_qwen3(const Json& raw, const std::string& dir, const llmx_engine_options& opt) {
    const Qwen3Config c = read_qwen3(raw);
    TensorFiles files;
    files.add_folder(dir);
    // What the model expects, by name: matrices [out, in], vectors [width].
    std::map<std::string, std::vector<long long>> expect;
    const long long q = c.heads * c.head_dim, kv = c.kv_heads * c.head_dim;
    expect["model.embed_tokens.weight"] = {c.vocab, c.hidden};
    expect["model.norm.weight"] = {c.hidden};
    if (!c.tied) expect["lm_head.weight"] = {c.vocab, c.hidden};
    for (long long l = 0; l < c.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        expect[p + "input_layernorm.weight"] = {c.hidden};
        expect[p + "post_attention_layernorm.weight"] = {c.hidden};
        expect[p + "self_attn.q_proj.weight"] = {q, c.hidden};
        expect[p + "self_attn.k_proj.weight"] = {kv, c.hidden};
        expect[p + "self_attn.v_proj.weight"] = {kv, c.hidden};
        expect[p + "self_attn.o_proj.weight"] = {c.hidden, q};
        expect[p + "self_attn.q_norm.weight"] = {c.head_dim};
        expect[p + "self_attn.k_norm.weight"] = {c.head_dim};
        expect[p + "mlp.gate_proj.weight"] = {c.intermediate, c.hidden};
        expect[p + "mlp.up_proj.weight"] = {c.intermediate, c.hidden};
        expect[p + "mlp.down_proj.weight"] = {c.hidden, c.intermediate};
    }
    std::vector<std::string> missing, unexpected, wrong;
    for (const auto& kv2 : expect) {
        const auto it = files.tensors.find(kv2.first);
        if (it == files.tensors.end()) {
            missing.push_back(kv2.first);
            continue;
        }
        if (it->second.shape != kv2.second) wrong.push_back(kv2.first + ": shape " + shape_text(it->second.shape) + ", expected " + shape_text(kv2.second));
        else if (it->second.dtype != "F32" && it->second.dtype != "BF16" && it->second.dtype != "F16")
            wrong.push_back(kv2.first + ": type " + it->second.dtype + ", expected float32, float16 or bfloat16");
    }
    for (const auto& kv2 : files.tensors)
        if (!expect.count(kv2.first) && !(c.tied && kv2.first == "lm_head.weight")) unexpected.push_back(kv2.first);
    if (!missing.empty() || !unexpected.empty() || !wrong.empty()) {
        auto list = [](const char* title, const std::vector<std::string>& v) {
            if (v.empty()) return std::string();
            std::string s = std::string("\n  ") + title + " (" + std::to_string(v.size()) + "):";
            for (size_t i = 0; i < v.size() && i < 20; ++i) s += "\n    " + v[i];
            if (v.size() > 20) s += "\n    ... and " + std::to_string(v.size() - 20) + " more";
            return s;
        };
        throw Failure{LLMX_ENGINE_ERR_WEIGHTS, dir + ": the tensors do not fit the model" + list("missing", missing) +
                                                   list("unexpected", unexpected) + list("wrong", wrong)};
    }

    // The files say what they must; from here on the device is needed.
    if (cudaSetDevice(opt.device) != cudaSuccess) throw Failure{LLMX_ENGINE_ERR_DEVICE, "no such CUDA device"};
    if (opt.kernel_dir && llmx_rt_load_kernels(opt.kernel_dir) < 0)
        throw Failure{LLMX_ENGINE_ERR_FILE, std::string("kernel libraries: ") + llmx_rt_last_error()};
    std::unique_ptr<Qwen3Model> m(new Qwen3Model);
    const int dtype = opt.dtype;
    const int flags = opt.invariant ? LLMX_FLAG_INVARIANT : 0;
    const long long kv_tokens = opt.kv_tokens > 0 ? opt.kv_tokens : 8192;
    // Position tables reach as far as a request can: the pool's size, or the model's context when that is less.
    const long long positions = std::max<long long>(std::min(c.max_positions, kv_tokens), 1);
    std::vector<float> cos_t, sin_t;
    rope_tables(c, positions, cos_t, sin_t);
    const float* cos_d = (const float*)m->weights.upload_raw(cos_t.data(), cos_t.size() * sizeof(float));
    const float* sin_d = (const float*)m->weights.upload_raw(sin_t.data(), sin_t.size() * sizeof(float));
    auto keep = [&](llmx_part* p) {
        if (!p) throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("building the model: ") + llmx_rt_last_error()};
        m->parts.push_back(p);
        return p;
    };
    auto vec = [&](const std::string& name) { return (const float*)m->weights.upload(files, {name}, LLMX_DT_F32); };
    auto linear = [&](const std::vector<std::string>& names, long long out, long long in) {
        return llmx_linear_desc{m->weights.upload(files, names, dtype), dtype, (int)out, (int)in, flags};
    };
    std::vector<llmx_part*> blocks;
    std::vector<llmx_layer_step> order;
    for (long long l = 0; l < c.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        llmx_attention_desc a = {};
        a.hidden = (int)c.hidden, a.heads = (int)c.heads, a.kv_heads = (int)c.kv_heads, a.head_dim = (int)c.head_dim, a.window = 0;
        a.scale = 1.0f / sqrtf((float)c.head_dim), a.qk_norm_eps = (float)c.eps;
        a.q_norm = vec(p + "self_attn.q_norm.weight"), a.k_norm = vec(p + "self_attn.k_norm.weight");
        a.cos = cos_d, a.sin = sin_d, a.rot_half = (int)c.head_dim / 2, a.table_positions = (int)positions, a.position_stream = 0;
        a.qkv = linear({p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"}, q + 2 * kv, c.hidden);
        a.o = linear({p + "self_attn.o_proj.weight"}, c.hidden, q);
        a.flags = flags;
        llmx_mlp_desc f = {};
        f.hidden = (int)c.hidden, f.intermediate = (int)c.intermediate;
        f.gate_up = linear({p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"}, 2 * c.intermediate, c.hidden);
        f.down = linear({p + "mlp.down_proj.weight"}, c.hidden, c.intermediate);
        f.flags = flags;
        llmx_part* n1 = keep(llmx_rmsnorm_create(vec(p + "input_layernorm.weight"), (int)c.hidden, (float)c.eps, dtype));
        llmx_part* n2 = keep(llmx_rmsnorm_create(vec(p + "post_attention_layernorm.weight"), (int)c.hidden, (float)c.eps, dtype));
        llmx_part* mixer = keep(llmx_attention_create(&a));
        llmx_part* ffn = keep(llmx_gated_mlp_create(&f));
        blocks.push_back(keep(llmx_prenorm_block_create(n1, mixer, n2, ffn)));
        order.push_back(llmx_layer_step{(int)l, (int)l, 1});
        m->entries.push_back(llmx_cache_entry_desc{1, (int)c.kv_heads, (int)c.head_dim, 0, 0});
    }
    const void* table = m->weights.upload(files, {"model.embed_tokens.weight"}, dtype);
    llmx_part* embedding = keep(llmx_embedding_create(table, dtype, (int)c.vocab, (int)c.hidden));
    llmx_part* final_norm = keep(llmx_rmsnorm_create(vec("model.norm.weight"), (int)c.hidden, (float)c.eps, dtype));
    llmx_linear_desc head_w = {c.tied ? table : m->weights.upload(files, {"lm_head.weight"}, dtype), dtype, (int)c.vocab, (int)c.hidden, flags};
    llmx_part* head = keep(llmx_head_create(final_norm, &head_w));
    m->model = llmx_model_create(embedding, blocks.data(), (int)blocks.size(), order.data(), (int)order.size(), head, (int)c.hidden, (int)c.vocab);
    if (!m->model) throw Failure{LLMX_ENGINE_ERR_REFUSED, std::string("building the model: ") + llmx_rt_last_error()};
    m->eos_ids = c.eos_ids;
    llmx_engine_desc& d = m->desc;
    d.vocab = (int)c.vocab, d.max_positions = (int)std::min<long long>(c.max_positions, 2147483647ll), d.position_streams = 1;
    return std::unique_ptr<LoadedModel>(m.release());
}

// One registry from the architecture's name (config.json's `architectures[0]`, else `model_type`) to its loader.
typedef std::function<std::unique_ptr<LoadedModel>(const Json&, const std::string&, const llmx_engine_options&)> Loader;
static std::map<std::string, Loader>& registry() {
    static std::map<std::string, Loader> r = {{"Qwen3ForCausalLM", load_qwen3}, {"qwen3", load_qwen3}};
    return r;
}

}  // namespace llmx_engine_detail

using namespace llmx_engine_detail;

#define LLMX_API extern "C" __attribute__((visibility("default")))

LLMX_API llmx_engine* llmx_engine_load(const char* model_dir, const llmx_engine_options* options) {
    try {
        if (!model_dir || !options) throw Failure{LLMX_ENGINE_ERR_REFUSED, "llmx_engine_load: a folder and options"};
        if (options->dtype != LLMX_DT_BF16 && options->dtype != LLMX_DT_F32)
            throw Failure{LLMX_ENGINE_ERR_REFUSED, "dtype must be bfloat16 or float32"};
        const std::string dir = model_dir;
        const std::string text = read_text(dir + "/config.json", dir + ": no config.json");
        Json raw;
        try {
            raw = JsonReader(text.data(), text.size()).parse();
        } catch (const Failure& f) {
            throw Failure{LLMX_ENGINE_ERR_FILE, dir + "/config.json: " + f.what};
        }
        if (raw.kind != Json::OBJ) throw Failure{LLMX_ENGINE_ERR_FILE, dir + "/config.json: config.json must hold an object"};
        // The one place a name is accepted.
        std::string name;
        if (const Json* a = raw.get("architectures"))
            if (a->kind == Json::ARR && !a->arr.empty() && a->arr[0].kind == Json::STR) name = a->arr[0].str;
        std::string by_type;
        if (const Json* t = raw.get("model_type"))
            if (t->kind == Json::STR) by_type = t->str;
        auto it = registry().find(name);
        if (it == registry().end()) it = registry().find(by_type);
        if (it == registry().end()) {
            std::string known;
            for (const auto& kv : registry()) known += (known.empty() ? "" : ", ") + kv.first;
            throw Failure{LLMX_ENGINE_ERR_FILE, dir + ": architectures " + (name.empty() ? "(none)" : name) + ", model_type " +
                                                    (by_type.empty() ? "(none)" : by_type) + ": no such architecture is registered (" + known + ")"};
        }
        std::unique_ptr<LoadedModel> loaded = it->second(raw, dir, *options);
        llmx_engine_desc d = loaded->desc;
        d.page_size = options->page_size > 0 ? options->page_size : 16;
        d.kv_tokens = options->kv_tokens > 0 ? options->kv_tokens : 8192;
        d.window_kv_tokens = options->window_kv_tokens;
        d.max_requests = options->max_requests > 0 ? options->max_requests : 16;
        d.kv_dtype = options->kv_dtype >= 0 ? options->kv_dtype : options->dtype;
        d.entries = loaded->entries.data();
        d.n_entries = (int)loaded->entries.size();
        d.eos_ids = loaded->eos_ids.data();
        d.n_eos = (int)loaded->eos_ids.size();
        d.max_batch_tokens = options->max_batch_tokens;
        d.max_queue = options->max_queue;
        d.reserve_prompt_only = options->reserve_prompt_only;
        d.device = options->device;
        llmx_model* model = loaded->model;
        return new llmx_engine(model, d, std::move(loaded));
    } catch (const Failure& f) {
        fail(f.code, f.what);
    } catch (const std::exception& e) {
        fail(LLMX_ENGINE_ERR_REFUSED, e.what());
    }
    return nullptr;
}
