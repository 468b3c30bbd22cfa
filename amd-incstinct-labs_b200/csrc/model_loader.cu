// ---------------------------------------------------------------------------
// model_loader.cu -- the reference's on-disk model format, read into device
// memory: cdna3::runtime::ModelLoader
// (cdna3-prims/include/cdna3/runtime/model_loader.hpp:83-204).
//
// A model directory holds meta.json (flat: n_layers, hidden, n_heads,
// n_kv_heads, head_dim, ffn_dim, vocab_size, optional rope_theta, qkv_bias and --
// an extension -- "dtype": "bf16") and one raw little-endian 16-bit file per
// tensor: embed_tokens.bin, lm_head.bin, final_norm.bin and, per layer i,
// layer_<i>_{q,k,v,o}_proj.bin, layer_<i>_{q,k,v}_bias.bin (with qkv_bias),
// layer_<i>_{gate,up,down}_proj.bin, layer_<i>_norm_{attn,mlp}.bin.
// Unlike the reference, which throws, every failure is a status code.
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "b200p_runtime.h"
#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

struct b200p_model {
    b200p_model_weights w{};
    std::vector<b200p_layer_weights> layers;
    std::vector<void*> owned;
};

namespace {

// The minimal flat-JSON reader of model_loader.hpp:103-129: "key": value pairs, values kept as text.
bool read_meta(const std::string& path, std::map<std::string, std::string>& kv) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return false;
    std::string src;
    char buf[4096];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) src.append(buf, n);
    std::fclose(f);
    size_t pos = 0;
    while (pos < src.size()) {
        const size_t qs = src.find('"', pos); if (qs == std::string::npos) break;
        const size_t qe = src.find('"', qs + 1); if (qe == std::string::npos) break;
        const std::string key = src.substr(qs + 1, qe - qs - 1);
        const size_t colon = src.find(':', qe); if (colon == std::string::npos) break;
        size_t vs = colon + 1;
        while (vs < src.size() && (src[vs] == ' ' || src[vs] == '\t' || src[vs] == '\n' || src[vs] == '\r')) ++vs;
        std::string val;
        if (vs < src.size() && src[vs] == '"') {
            const size_t ve = src.find('"', vs + 1); if (ve == std::string::npos) break;
            val = src.substr(vs + 1, ve - vs - 1); pos = ve + 1;
        } else {
            size_t ve = vs;
            while (ve < src.size() && src[ve] != ',' && src[ve] != '}' && src[ve] != '\n') ++ve;
            val = src.substr(vs, ve - vs); pos = ve;
            while (!val.empty() && (val.back() == ' ' || val.back() == '\r' || val.back() == '\t')) val.pop_back();
        }
        kv[key] = val;
    }
    return true;
}

int parse_meta(const char* dir, b200p_model_config* c, int* qkv_bias, int* dtype) {
    std::map<std::string, std::string> kv;
    if (!read_meta(std::string(dir) + "/meta.json", kv)) return B200P_E_IO;
    const char* need[] = {"n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn_dim", "vocab_size"};
    int* dst[] = {&c->n_layers, &c->hidden, &c->n_heads, &c->n_kv_heads, &c->head_dim, &c->ffn_dim, &c->vocab_size};
    for (int i = 0; i < 7; ++i) {
        auto it = kv.find(need[i]);
        if (it == kv.end()) return B200P_E_IO;
        char* end = nullptr;
        const long v = std::strtol(it->second.c_str(), &end, 10);
        if (end == it->second.c_str() || v <= 0) return B200P_E_IO;
        *dst[i] = int(v);
    }
    c->rope_theta = kv.count("rope_theta") ? std::strtof(kv["rope_theta"].c_str(), nullptr) : 10000.0f;
    if (qkv_bias) *qkv_bias = kv.count("qkv_bias") && (kv["qkv_bias"] == "1" || kv["qkv_bias"] == "true");
    if (dtype) *dtype = (kv.count("dtype") && (kv["dtype"] == "bf16" || kv["dtype"] == "bfloat16")) ? B200P_BF16 : B200P_F16;
    return B200P_OK;
}

// load_tensor (model_loader.hpp:89-98): n_elems raw 16-bit values -> device memory.
int load_tensor(b200p_model* m, const std::string& path, size_t n_elems, const void** out) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return B200P_E_IO;
    std::vector<uint16_t> host(n_elems);
    const size_t got = std::fread(host.data(), 2, n_elems, f);
    std::fclose(f);
    if (got != n_elems) return B200P_E_IO;                       // short read
    void* dev = nullptr;
    if (cudaError_t e = cudaMalloc(&dev, n_elems * 2)) return int(e);
    m->owned.push_back(dev);
    if (cudaError_t e = cudaMemcpy(dev, host.data(), n_elems * 2, cudaMemcpyHostToDevice)) return int(e);
    *out = dev;
    return B200P_OK;
}

} // namespace

extern "C" int b200p_model_read_meta(const char* model_dir, b200p_model_config* cfg, int* qkv_bias, int* dtype) {
    if (!model_dir || !cfg) return B200P_E_NULL;
    return parse_meta(model_dir, cfg, qkv_bias, dtype);
}

extern "C" void b200p_model_free(b200p_model* m) {
    if (!m) return;
    for (void* p : m->owned) cudaFree(p);
    delete m;
}

extern "C" b200p_model* b200p_model_load(const char* model_dir, int* status) {
    int dummy; if (!status) status = &dummy;
    *status = B200P_OK;
    if (!model_dir) { *status = B200P_E_NULL; return nullptr; }
    b200p_model* m = new b200p_model();
    int bias = 0, dtype = B200P_F16;
    if ((*status = parse_meta(model_dir, &m->w.cfg, &bias, &dtype))) { delete m; return nullptr; }
    if (b200p::sm_count() <= 0) { *status = B200P_E_NO_DEVICE; delete m; return nullptr; }
    m->w.dtype = dtype;
    const b200p_model_config& c = m->w.cfg;
    const size_t H = size_t(c.hidden), F = size_t(c.ffn_dim), V = size_t(c.vocab_size);
    const size_t qd = size_t(c.n_heads) * c.head_dim, kvd = size_t(c.n_kv_heads) * c.head_dim;
    const std::string dir(model_dir);
    auto top = [&](const char* name) { return dir + "/" + name + ".bin"; };
    int rc = load_tensor(m, top("embed_tokens"), V * H, &m->w.embed_tokens);
    if (!rc) rc = load_tensor(m, top("lm_head"), V * H, &m->w.lm_head);
    if (!rc) rc = load_tensor(m, top("final_norm"), H, &m->w.final_norm);
    m->layers.assign(size_t(c.n_layers), b200p_layer_weights{});
    for (int i = 0; i < c.n_layers && !rc; ++i) {
        auto lp = [&](const char* t) { return dir + "/layer_" + std::to_string(i) + "_" + t + ".bin"; };
        b200p_layer_weights& L = m->layers[size_t(i)];
        rc = load_tensor(m, lp("q_proj"), qd * H, &L.Wq);
        if (!rc) rc = load_tensor(m, lp("k_proj"), kvd * H, &L.Wk);
        if (!rc) rc = load_tensor(m, lp("v_proj"), kvd * H, &L.Wv);
        if (!rc) rc = load_tensor(m, lp("o_proj"), H * qd, &L.Wo);
        if (bias) {
            if (!rc) rc = load_tensor(m, lp("q_bias"), qd, &L.bq);
            if (!rc) rc = load_tensor(m, lp("k_bias"), kvd, &L.bk);
            if (!rc) rc = load_tensor(m, lp("v_bias"), kvd, &L.bv);
        }
        if (!rc) rc = load_tensor(m, lp("gate_proj"), F * H, &L.Wgate);
        if (!rc) rc = load_tensor(m, lp("up_proj"), F * H, &L.Wup);
        if (!rc) rc = load_tensor(m, lp("down_proj"), H * F, &L.Wdown);
        if (!rc) rc = load_tensor(m, lp("norm_attn"), H, &L.norm_attn);
        if (!rc) rc = load_tensor(m, lp("norm_mlp"), H, &L.norm_mlp);
    }
    if (rc) { *status = rc; b200p_model_free(m); return nullptr; }
    m->w.layers = m->layers.data();
    return m;
}

extern "C" const b200p_model_weights* b200p_model_weights_of(const b200p_model* m) { return m ? &m->w : nullptr; }
