// loader.cu — checkpoint directory -> resident model: config.json + safetensors (single file or
// sharded) of a gemma3-style MLX-affine checkpoint, read on the host and uploaded through the
// same entry points a cgo shim would call (lthn_model_create / upload_linear / upload_norm /
// finalize). Host code only; it launches no kernel of its own.
//
// What it follows in the reference (paths relative to its go/ directory):
//   model.Load                      model/load.go:19-108        probe model_type, parse the config, map the tensors
//   safetensors header + shards     model/safetensors/header_parse.go, sharded.go:  8-byte LE header length, JSON
//                                   directory {name: {dtype, shape, data_offsets}}, model.safetensors.index.json
//   gemma3 Config                   model/arch/google/gemma3/gemma3.go:30-59       the fields read here; the text
//                                   arch may nest under "text_config"
//   QuantConfig                     model/quant_config.go:39-88   group_size / bits defaults and per-module
//                                   overrides keyed by tensor path (language_model. prefix stripped)
//   LoadLinear / affineGeometry     model/linear.go:42-102        groupSize = inDim / scales.shape[-1],
//                                   bits = packedCols*32 / inDim, checked against the config
//   WidenF16TensorsToBF16           model/safetensors/widen.go    IEEE-half scales/biases/norms widened to bf16
//   foldNormBiasOne                 model/norm_bias.go:22-49      gemma norms store w-1: +1 in the tensor's dtype
//   weight names                    model/assemble.go:56-75
// The tensors are read from a read-only mmap that is unmapped before the call returns: uploads
// copy (the library retains no host pointer).
#include "common.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace lthn {
namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, true/false/null) -----------------
struct JValue {
    enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JValue> arr;
    std::vector<std::pair<std::string, JValue>> obj;
    const JValue* get(const std::string& k) const {
        if (type != Obj) return nullptr;
        for (auto& kv : obj) if (kv.first == k) return &kv.second;
        return nullptr;
    }
    bool number(const std::string& k, double* out) const {
        const JValue* v = get(k);
        if (!v || v->type != Num) return false;
        *out = v->num;
        return true;
    }
};

struct JParser {
    const char* p;
    const char* end;
    std::string err;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool fail(const char* m) { if (err.empty()) err = m; return false; }
    bool parse_string(std::string* out) {
        if (p >= end || *p != '"') return fail("expected a string");
        p++;
        out->clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("unterminated escape");
                switch (*p) {
                    case 'n': out->push_back('\n'); break;
                    case 't': out->push_back('\t'); break;
                    case 'r': out->push_back('\r'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'u': {
                        if (end - p < 5) return fail("short \\u escape");
                        unsigned cp = 0;
                        for (int i = 1; i <= 4; i++) {
                            const char c = p[i];
                            cp = cp * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 0);
                        }
                        p += 4;
                        if (cp < 0x80) out->push_back((char)cp);
                        else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                        else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                        break;
                    }
                    default: out->push_back(*p);
                }
                p++;
            } else {
                out->push_back(*p++);
            }
        }
        if (p >= end) return fail("unterminated string");
        p++;
        return true;
    }
    bool parse_value(JValue* v, int depth) {
        if (depth > 64) return fail("JSON nested too deeply");
        ws();
        if (p >= end) return fail("unexpected end of JSON");
        if (*p == '{') {
            v->type = JValue::Obj;
            p++;
            ws();
            if (p < end && *p == '}') { p++; return true; }
            for (;;) {
                ws();
                std::string key;
                if (!parse_string(&key)) return false;
                ws();
                if (p >= end || *p != ':') return fail("expected ':'");
                p++;
                JValue child;
                if (!parse_value(&child, depth + 1)) return false;
                v->obj.emplace_back(std::move(key), std::move(child));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (*p == '[') {
            v->type = JValue::Arr;
            p++;
            ws();
            if (p < end && *p == ']') { p++; return true; }
            for (;;) {
                JValue child;
                if (!parse_value(&child, depth + 1)) return false;
                v->arr.push_back(std::move(child));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (*p == '"') { v->type = JValue::Str; return parse_string(&v->str); }
        if (end - p >= 4 && !strncmp(p, "true", 4)) { v->type = JValue::Bool; v->b = true; p += 4; return true; }
        if (end - p >= 5 && !strncmp(p, "false", 5)) { v->type = JValue::Bool; v->b = false; p += 5; return true; }
        if (end - p >= 4 && !strncmp(p, "null", 4)) { v->type = JValue::Null; p += 4; return true; }
        char* e = nullptr;
        const std::string tmp(p, (size_t)std::min<ptrdiff_t>(end - p, 64));
        const double d = strtod(tmp.c_str(), &e);
        if (e == tmp.c_str()) return fail("unexpected character in JSON");
        v->type = JValue::Num;
        v->num = d;
        p += e - tmp.c_str();
        return true;
    }
};

bool parse_json(const char* data, size_t n, JValue* out, std::string* err) {
    JParser ps{data, data + n, {}};
    if (!ps.parse_value(out, 0)) { *err = ps.err; return false; }
    ps.ws();
    if (ps.p != ps.end) { *err = "trailing characters after the JSON value"; return false; }
    return true;
}

// ---- files ------------------------------------------------------------------------------------
struct Mapping {
    void* base = nullptr;
    size_t size = 0;
    ~Mapping() { if (base && base != MAP_FAILED) munmap(base, size); }
};

bool map_file(const std::string& path, Mapping* m, std::string* err) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) { *err = "cannot open " + path; return false; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) { close(fd); *err = "cannot stat " + path; return false; }
    m->size = (size_t)st.st_size;
    m->base = mmap(nullptr, m->size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m->base == MAP_FAILED) { m->base = nullptr; *err = "cannot map " + path; return false; }
    return true;
}

bool read_text(const std::string& path, std::string* out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char buf[65536];
    size_t n;
    out->clear();
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) out->append(buf, n);
    fclose(f);
    return true;
}

struct Tensor {
    std::string dtype;
    std::vector<int64_t> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
};

size_t dtype_size(const std::string& d) {
    if (d == "U32" || d == "F32" || d == "I32") return 4;
    if (d == "BF16" || d == "F16" || d == "U16" || d == "I16") return 2;
    if (d == "U8" || d == "I8" || d == "BOOL") return 1;
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    return 0;
}

// One safetensors file: 8-byte LE header length, JSON directory, then the tensor bytes.
bool read_shard(const std::string& path, std::vector<std::unique_ptr<Mapping>>* maps, std::map<std::string, Tensor>* tensors,
                std::string* err) {
    auto mp = std::make_unique<Mapping>();
    if (!map_file(path, mp.get(), err)) return false;
    const unsigned char* base = (const unsigned char*)mp->base;
    if (mp->size < 8) { *err = path + ": shorter than a safetensors header"; return false; }
    uint64_t hlen = 0;
    for (int i = 0; i < 8; i++) hlen |= (uint64_t)base[i] << (8 * i);
    if (hlen == 0 || hlen > mp->size - 8 || hlen > (uint64_t)1 << 30) { *err = path + ": header length out of range"; return false; }
    JValue hdr;
    std::string jerr;
    if (!parse_json((const char*)base + 8, (size_t)hlen, &hdr, &jerr) || hdr.type != JValue::Obj) {
        *err = path + ": header is not a JSON object (" + jerr + ")";
        return false;
    }
    const size_t data0 = 8 + (size_t)hlen, data_len = mp->size - data0;
    for (auto& kv : hdr.obj) {
        if (kv.first == "__metadata__") continue;
        const JValue& e = kv.second;
        const JValue *dt = e.get("dtype"), *sh = e.get("shape"), *off = e.get("data_offsets");
        if (!dt || dt->type != JValue::Str || !sh || sh->type != JValue::Arr || !off || off->type != JValue::Arr || off->arr.size() != 2) {
            *err = path + ": malformed directory entry for " + kv.first;
            return false;
        }
        Tensor t;
        t.dtype = dt->str;
        int64_t elems = 1;
        for (auto& d : sh->arr) {
            if (d.type != JValue::Num || d.num < 0) { *err = path + ": bad shape for " + kv.first; return false; }
            t.shape.push_back((int64_t)d.num);
            elems *= (int64_t)d.num;
        }
        const double a = off->arr[0].num, b = off->arr[1].num;
        if (a < 0 || b < a || b > (double)data_len) { *err = path + ": data_offsets of " + kv.first + " outside the file"; return false; }
        t.data = base + data0 + (size_t)a;
        t.bytes = (size_t)(b - a);
        const size_t es = dtype_size(t.dtype);
        if (es == 0 || (size_t)elems * es != t.bytes) { *err = path + ": " + kv.first + " has " + std::to_string(t.bytes) + " bytes for its shape and dtype " + t.dtype; return false; }
        // the multimodal wrapper nests the text model under language_model. (model/quant_config.go:54)
        std::string name = kv.first;
        const std::string pre = "language_model.";
        if (name.compare(0, pre.size(), pre) == 0) name = name.substr(pre.size());
        (*tensors)[name] = std::move(t);
    }
    maps->push_back(std::move(mp));
    return true;
}

struct Checkpoint {
    std::vector<std::unique_ptr<Mapping>> maps;
    std::map<std::string, Tensor> tensors;
    JValue config;
    // resolved
    int layers = 0, hidden = 0, q_heads = 0, kv_heads = 0, head_dim = 0, ffn = 0, vocab = 0, gs = 0, bits = 0;
    int sliding_window = 0, sliding_pattern = 0, max_pos = 0;
    float rope_local = 10000.0f;  // gemma3 default (model/arch/google/gemma3/gemma3.go:24)
    float eps = 1e-6f, rope_theta = 1000000.0f;
    std::string model_type;
    std::map<std::string, std::pair<int, int>> overrides;  // module path -> (group_size, bits)
};

const JValue* text_cfg(const JValue& cfg) {
    const JValue* t = cfg.get("text_config");
    return t && t->type == JValue::Obj ? t : &cfg;
}

bool open_checkpoint(const std::string& dir, Checkpoint* ck, std::string* err) {
    std::string cfg_text;
    if (!read_text(dir + "/config.json", &cfg_text)) { *err = "cannot read " + dir + "/config.json"; return false; }
    std::string jerr;
    if (!parse_json(cfg_text.data(), cfg_text.size(), &ck->config, &jerr) || ck->config.type != JValue::Obj) {
        *err = "config.json is not a JSON object (" + jerr + ")";
        return false;
    }
    const JValue& top = ck->config;
    const JValue* tc = text_cfg(top);
    if (const JValue* mt = top.get("model_type")) if (mt->type == JValue::Str) ck->model_type = mt->str;
    std::string text_mt = ck->model_type;
    if (const JValue* mt = tc->get("model_type")) if (mt->type == JValue::Str) text_mt = mt->str;
    if (ck->model_type != "gemma3" && ck->model_type != "gemma3_text" && text_mt != "gemma3_text" && text_mt != "gemma3") {
        *err = "no architecture for model_type \"" + ck->model_type + "\": this engine serves the gemma3 block";
        return false;
    }
    auto geti = [&](const char* k, int* out) { double d; if (tc->number(k, &d)) { *out = (int)d; return true; } return false; };
    geti("num_hidden_layers", &ck->layers);
    geti("hidden_size", &ck->hidden);
    geti("num_attention_heads", &ck->q_heads);
    geti("num_key_value_heads", &ck->kv_heads);
    geti("head_dim", &ck->head_dim);
    geti("intermediate_size", &ck->ffn);
    geti("vocab_size", &ck->vocab);
    geti("sliding_window", &ck->sliding_window);
    geti("sliding_window_pattern", &ck->sliding_pattern);
    geti("max_position_embeddings", &ck->max_pos);
    double d;
    if (tc->number("rms_norm_eps", &d)) ck->eps = (float)d;
    if (tc->number("rope_theta", &d)) ck->rope_theta = (float)d;
    if (tc->number("rope_local_base_freq", &d) && d > 0) ck->rope_local = (float)d;
    // quantization block: top level or nested (gemma3.go:50-59)
    const JValue* q = top.get("quantization");
    if (!q || q->type != JValue::Obj) q = tc->get("quantization");
    if (!q || q->type != JValue::Obj) { *err = "config.json has no quantization block: this engine serves MLX-affine quantized checkpoints"; return false; }
    if (const JValue* mode = q->get("mode"))
        if (mode->type == JValue::Str && !mode->str.empty() && mode->str != "affine") { *err = "quantization mode \"" + mode->str + "\" is not affine"; return false; }
    for (auto& kv : q->obj) {
        if (kv.first == "group_size" && kv.second.type == JValue::Num) ck->gs = (int)kv.second.num;
        else if (kv.first == "bits" && kv.second.type == JValue::Num) ck->bits = (int)kv.second.num;
        else if (kv.second.type == JValue::Obj) {
            double ob = 0, og = 0;
            kv.second.number("bits", &ob);
            kv.second.number("group_size", &og);
            if ((int)ob == 0) continue;
            std::string name = kv.first;
            const std::string pre = "language_model.";
            if (name.compare(0, pre.size(), pre) == 0) name = name.substr(pre.size());
            ck->overrides[name] = {(int)og, (int)ob};
        }
    }
    // shards: model.safetensors.index.json names the file of every tensor; else one model.safetensors
    std::string index_text;
    std::vector<std::string> files;
    if (read_text(dir + "/model.safetensors.index.json", &index_text)) {
        JValue idx;
        if (!parse_json(index_text.data(), index_text.size(), &idx, &jerr)) { *err = "model.safetensors.index.json: " + jerr; return false; }
        const JValue* wm = idx.get("weight_map");
        if (!wm || wm->type != JValue::Obj) { *err = "model.safetensors.index.json has no weight_map"; return false; }
        for (auto& kv : wm->obj) {
            if (kv.second.type != JValue::Str) continue;
            bool seen = false;
            for (auto& f : files) seen = seen || f == kv.second.str;
            if (!seen) files.push_back(kv.second.str);
        }
        if (files.empty()) { *err = "model.safetensors.index.json lists no shard"; return false; }
    } else {
        files.push_back("model.safetensors");
    }
    for (auto& f : files) {
        if (f.find('/') != std::string::npos || f.find("..") != std::string::npos) { *err = "shard name leaves the checkpoint directory: " + f; return false; }
        if (!read_shard(dir + "/" + f, &ck->maps, &ck->tensors, err)) return false;
    }
    // dims the config omits come from the weight shapes (InferFromWeights, model/load.go:63)
    auto shape_of = [&](const std::string& n) -> const std::vector<int64_t>* {
        auto it = ck->tensors.find(n);
        return it == ck->tensors.end() ? nullptr : &it->second.shape;
    };
    if (ck->vocab == 0) if (auto s = shape_of("model.embed_tokens.weight")) if (s->size() == 2) ck->vocab = (int)(*s)[0];
    if (ck->head_dim == 0 && ck->q_heads > 0) if (auto s = shape_of("model.layers.0.self_attn.q_proj.weight")) if (s->size() == 2) ck->head_dim = (int)((*s)[0] / ck->q_heads);
    if (ck->kv_heads == 0) ck->kv_heads = ck->q_heads;
    if (ck->layers <= 0 || ck->hidden <= 0 || ck->q_heads <= 0 || ck->head_dim <= 0 || ck->ffn <= 0 || ck->vocab <= 0) {
        *err = "config.json does not give the model dimensions (layers/hidden/heads/head_dim/intermediate/vocab)";
        return false;
    }
    if (ck->gs == 0 || ck->bits == 0) { *err = "quantization block gives no group_size/bits"; return false; }
    return true;
}

inline float half_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
    else u = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// bf16 view of a 16-bit float tensor: BF16 as is, F16 widened (WidenF16TensorsToBF16)
bool as_bf16(const Tensor& t, std::vector<uint16_t>* tmp, const uint16_t** out, std::string* err, const std::string& name) {
    if (t.dtype == "BF16") { *out = (const uint16_t*)t.data; return true; }
    if (t.dtype == "F16") {
        tmp->resize(t.bytes / 2);
        const uint16_t* src = (const uint16_t*)t.data;
        for (size_t i = 0; i < tmp->size(); i++) (*tmp)[i] = f32_to_bf16_bits(half_to_f32(src[i]));
        *out = tmp->data();
        return true;
    }
    *err = name + ": scales and biases must be BF16 or F16, not " + t.dtype;
    return false;
}

// effective norm weights: the stored w-1 plus one, added in the tensor's dtype (foldNormBiasOne)
bool norm_weights(const Tensor& t, int64_t n, std::vector<float>* out, std::string* err, const std::string& name) {
    out->resize((size_t)n);
    int64_t elems = 1;
    for (auto d : t.shape) elems *= d;
    if (elems != n) { *err = name + ": expected " + std::to_string(n) + " elements"; return false; }
    if (t.dtype == "F32") {
        const float* s = (const float*)t.data;
        for (int64_t i = 0; i < n; i++) (*out)[i] = s[i] + 1.0f;
    } else if (t.dtype == "BF16" || t.dtype == "F16") {
        const uint16_t* s = (const uint16_t*)t.data;
        for (int64_t i = 0; i < n; i++) {
            const uint16_t b = t.dtype == "BF16" ? s[i] : f32_to_bf16_bits(half_to_f32(s[i]));
            (*out)[i] = bf16_bits_to_f32(f32_to_bf16_bits(bf16_bits_to_f32(b) + 1.0f));
        }
    } else {
        *err = name + ": unsupported norm dtype " + t.dtype;
        return false;
    }
    return true;
}

}  // namespace
}  // namespace lthn

using namespace lthn;

extern "C" {

int32_t lthn_checkpoint_inspect(const char* dir, char* json_out, size_t json_len) {
    clear_error();
    LTHN_REQUIRE(dir && json_out && json_len > 0, "lthn_checkpoint_inspect: NULL argument");
    Checkpoint ck;
    std::string err;
    if (!open_checkpoint(dir, &ck, &err)) return fail(LTHN_ERR_INVALID, "lthn_checkpoint_inspect: " + err);
    std::string s = "{\"model_type\": \"" + ck.model_type + "\", \"layers\": " + std::to_string(ck.layers) + ", \"hidden\": " + std::to_string(ck.hidden) +
                    ", \"q_heads\": " + std::to_string(ck.q_heads) + ", \"kv_heads\": " + std::to_string(ck.kv_heads) + ", \"head_dim\": " +
                    std::to_string(ck.head_dim) + ", \"ffn\": " + std::to_string(ck.ffn) + ", \"vocab\": " + std::to_string(ck.vocab) +
                    ", \"group_size\": " + std::to_string(ck.gs) + ", \"bits\": " + std::to_string(ck.bits) + ", \"overrides\": " +
                    std::to_string(ck.overrides.size()) + ", \"tensors\": " + std::to_string(ck.tensors.size()) + ", \"shards\": " +
                    std::to_string(ck.maps.size()) + ", \"sliding_window\": " + std::to_string(ck.sliding_window) + "}";
    if (s.size() + 1 > json_len) return fail(LTHN_ERR_INVALID, "lthn_checkpoint_inspect: output buffer too small");
    memcpy(json_out, s.c_str(), s.size() + 1);
    return LTHN_OK;
}

int32_t lthn_model_load_dir(const char* dir, const lthn_load_options* opts, void** model) {
    clear_error();
    LTHN_REQUIRE(dir && model, "lthn_model_load_dir: NULL argument");
    *model = nullptr;
    lthn_load_options o{};
    if (opts) o = *opts;
    Checkpoint ck;
    std::string err;
    if (!open_checkpoint(dir, &ck, &err)) return fail(LTHN_ERR_INVALID, "lthn_model_load_dir: " + err);
    lthn_model_config c{};
    c.layers = ck.layers; c.hidden = ck.hidden; c.q_heads = ck.q_heads; c.kv_heads = ck.kv_heads; c.head_dim = ck.head_dim;
    c.ffn = ck.ffn; c.vocab = ck.vocab; c.group_size = ck.gs; c.bits = ck.bits;
    c.max_len = o.max_len > 0 ? o.max_len : (ck.max_pos > 0 ? std::min(ck.max_pos, 4096) : 4096);
    c.max_lanes = o.max_lanes > 0 ? o.max_lanes : 1;
    c.eps = ck.eps; c.rope_base = ck.rope_theta;
    c.tp_rank = o.tp_rank; c.tp_size = o.tp_size;
    if (ck.sliding_window > 0 && !o.uniform_attention) {
        // gemma3 layer types: sliding blocks with the local rope base, every pattern-th block global
        c.sliding_window = ck.sliding_window;
        c.sliding_pattern = ck.sliding_pattern > 0 ? ck.sliding_pattern : 6;
        c.rope_local_base = ck.rope_local;
    }
    void* m = nullptr;
    int32_t rc = lthn_model_create(&c, &m);
    if (rc) return rc;
    auto bail = [&](int32_t code, const std::string& msg) {
        lthn_model_destroy(m);
        return fail(code, "lthn_model_load_dir: " + msg);
    };
    auto bail_keep = [&](int32_t code) {
        const std::string keep = lthn_last_error();
        lthn_model_destroy(m);
        return fail(code, keep);
    };
    // one quantized linear: <base>.weight (U32), .scales, .biases; geometry as affineGeometry derives it
    auto upload_linear = [&](const std::string& base, int layer, int role, int64_t N, int64_t K) -> int32_t {
        auto w = ck.tensors.find(base + ".weight"), s = ck.tensors.find(base + ".scales"), b = ck.tensors.find(base + ".biases");
        if (w == ck.tensors.end() || s == ck.tensors.end() || b == ck.tensors.end()) return bail(LTHN_ERR_INVALID, "missing tensor " + base + ".{weight,scales,biases}");
        const Tensor &tw = w->second, &ts = s->second, &tb = b->second;
        if (tw.dtype != "U32" || tw.shape.size() != 2 || ts.shape.size() != 2 || tb.shape != ts.shape)
            return bail(LTHN_ERR_INVALID, base + ": want a rank-2 U32 weight with rank-2 scales and biases of one shape");
        int gs = ck.gs, bits = ck.bits;
        auto ov = ck.overrides.find(base);
        if (ov != ck.overrides.end()) { gs = ov->second.first ? ov->second.first : gs; bits = ov->second.second; }
        if (tw.shape[0] != N || ts.shape[0] != N || ts.shape[1] <= 0) return bail(LTHN_ERR_INVALID, base + ": row count does not match the configuration");
        const int64_t groups = ts.shape[1];
        if (K % groups != 0) return bail(LTHN_ERR_INVALID, base + ": scales do not divide the input width");
        const int64_t got_gs = K / groups, got_bits = tw.shape[1] * 32 / K;
        if (got_gs != gs || got_bits != bits || tw.shape[1] * 32 != K * got_bits)
            return bail(LTHN_ERR_INVALID, base + ": tensor geometry says group " + std::to_string(got_gs) + " / " + std::to_string(got_bits) +
                                              " bit, the quantization block says group " + std::to_string(gs) + " / " + std::to_string(bits) + " bit");
        // 4-bit group-64 everywhere; an 8-bit group-64 override on an MLP projection of a one-GPU model
        const bool mlp = layer >= 0 && (role == LTHN_ROLE_GATE || role == LTHN_ROLE_UP || role == LTHN_ROLE_DOWN);
        const bool wide = bits == 8 && gs == 64 && mlp && o.tp_size <= 1;
        if (gs != 64 || (bits != 4 && !wide))
            return bail(LTHN_ERR_INVALID, base + ": " + std::to_string(bits) + "-bit group-" + std::to_string(gs) +
                                              " weights: the decoder engine serves 4-bit group-64 linears (8-bit group-64 for the MLP"
                                              " projections on one GPU) only");
        std::vector<uint16_t> ts16, tb16;
        const uint16_t *ps, *pb;
        std::string e2;
        if (!as_bf16(ts, &ts16, &ps, &e2, base + ".scales") || !as_bf16(tb, &tb16, &pb, &e2, base + ".biases")) return bail(LTHN_ERR_INVALID, e2);
        const int32_t r = lthn_model_upload_linear_bits(m, layer, role, tw.data, ps, pb, N, K, bits);
        return r ? bail_keep(r) : LTHN_OK;
    };
    auto upload_norm = [&](const std::string& name, int layer, int role, int64_t n) -> int32_t {
        auto it = ck.tensors.find(name);
        if (it == ck.tensors.end()) return bail(LTHN_ERR_INVALID, "missing tensor " + name);
        std::vector<float> w;
        std::string e2;
        if (!norm_weights(it->second, n, &w, &e2, name)) return bail(LTHN_ERR_INVALID, e2);
        const int32_t r = lthn_model_upload_norm(m, layer, role, w.data(), n);
        return r ? bail_keep(r) : LTHN_OK;
    };
    const int64_t H = ck.hidden, D = ck.head_dim, F = ck.ffn;
    for (int li = 0; li < ck.layers; li++) {
        const std::string L = "model.layers." + std::to_string(li);
        if ((rc = upload_linear(L + ".self_attn.q_proj", li, LTHN_ROLE_Q, (int64_t)ck.q_heads * D, H))) return rc;
        if ((rc = upload_linear(L + ".self_attn.k_proj", li, LTHN_ROLE_K, (int64_t)ck.kv_heads * D, H))) return rc;
        if ((rc = upload_linear(L + ".self_attn.v_proj", li, LTHN_ROLE_V, (int64_t)ck.kv_heads * D, H))) return rc;
        if ((rc = upload_linear(L + ".self_attn.o_proj", li, LTHN_ROLE_O, H, (int64_t)ck.q_heads * D))) return rc;
        if ((rc = upload_linear(L + ".mlp.gate_proj", li, LTHN_ROLE_GATE, F, H))) return rc;
        if ((rc = upload_linear(L + ".mlp.up_proj", li, LTHN_ROLE_UP, F, H))) return rc;
        if ((rc = upload_linear(L + ".mlp.down_proj", li, LTHN_ROLE_DOWN, H, F))) return rc;
        if ((rc = upload_norm(L + ".input_layernorm.weight", li, LTHN_NORM_INPUT, H))) return rc;
        if ((rc = upload_norm(L + ".post_attention_layernorm.weight", li, LTHN_NORM_POST_ATTN, H))) return rc;
        if ((rc = upload_norm(L + ".pre_feedforward_layernorm.weight", li, LTHN_NORM_PRE_FF, H))) return rc;
        if ((rc = upload_norm(L + ".post_feedforward_layernorm.weight", li, LTHN_NORM_POST_FF, H))) return rc;
        if ((rc = upload_norm(L + ".self_attn.q_norm.weight", li, LTHN_NORM_Q, D))) return rc;
        if ((rc = upload_norm(L + ".self_attn.k_norm.weight", li, LTHN_NORM_K, D))) return rc;
    }
    if ((rc = upload_linear("model.embed_tokens", -1, 0, ck.vocab, H))) return rc;
    if ((rc = upload_norm("model.norm.weight", -1, 0, H))) return rc;
    if (o.comm && (rc = lthn_model_set_comm(m, o.comm))) return bail_keep(rc);
    if ((rc = lthn_model_finalize(m))) return bail_keep(rc);
    *model = m;
    return LTHN_OK;
}

}  // extern "C"
