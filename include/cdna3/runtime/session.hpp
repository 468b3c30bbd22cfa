// ---------------------------------------------------------------------------
// cdna3/runtime/session.hpp -- cdna3::runtime::{ModelConfig, GenerateCfg, ModelLoader,
// Session} with the reference's constructor and method shapes
// (cdna3-prims/include/cdna3/runtime/model_loader.hpp:51-60,134-204 and
//  cdna3-prims/include/cdna3/runtime/session.hpp:44-50,253-318), forwarding to the
// C ABI of libb200p (b200p_runtime.h).  Host C++ only: compiles with any C++17
// compiler.  Failures throw std::runtime_error, as the reference's loader does.
// ---------------------------------------------------------------------------
#pragma once
#include <stdexcept>
#include <string>
#include <vector>
#include "../../b200p_runtime.h"

namespace cdna3 {
namespace runtime {

using ModelConfig = b200p_model_config;

struct GenerateCfg {
    int max_new_tokens = 32;
    int eos_token_id = -1;     // -1: never stop early
};

class ModelLoader {
    std::string dir_;
    b200p_model* m_ = nullptr;
public:
    explicit ModelLoader(const std::string& model_dir) : dir_(model_dir) {}
    ModelLoader(const ModelLoader&) = delete;
    ModelLoader& operator=(const ModelLoader&) = delete;
    ~ModelLoader() { b200p_model_free(m_); }
    void load() {
        int st = 0;
        b200p_model_free(m_);
        m_ = b200p_model_load(dir_.c_str(), &st);
        if (!m_) throw std::runtime_error("ModelLoader: " + dir_ + ": " + b200p_strerror(st));
    }
    const b200p_model_weights& weights() const {
        if (!m_) throw std::runtime_error("ModelLoader: load() has not been called");
        return *b200p_model_weights_of(m_);
    }
};

// One sequence per session, like the reference's (batch = 1).
class Session {
    ModelLoader loader_;
    b200p_session* s_ = nullptr;
    int max_seq_;
public:
    Session(const std::string& model_dir, int max_seq = 4096) : loader_(model_dir), max_seq_(max_seq) {
        loader_.load();
        int st = 0;
        s_ = b200p_session_create(&loader_.weights(), max_seq, 1, &st);
        if (!s_) throw std::runtime_error(std::string("Session: ") + b200p_strerror(st));
    }
    Session(const Session&) = delete;
    Session& operator=(const Session&) = delete;
    ~Session() { b200p_session_destroy(s_); }

    const ModelConfig& config() const { return loader_.weights().cfg; }

    // Greedy generation: returns the input followed by the generated tokens, cut after eos_token_id if it
    // appears (the decode loop runs on the device for max_new_tokens; what follows an eos is dropped).
    std::vector<int> generate(const std::vector<int>& input_ids, const GenerateCfg& cfg) {
        std::vector<int> seq = input_ids;
        if (cfg.max_new_tokens <= 0 || input_ids.empty()) return seq;
        std::vector<int> out(size_t(cfg.max_new_tokens));
        const int rc = b200p_session_generate(s_, input_ids.data(), int(input_ids.size()), cfg.max_new_tokens, out.data(),
                                              nullptr, nullptr);
        if (rc) throw std::runtime_error(std::string("Session::generate: ") + b200p_strerror(rc));
        for (int t : out) {
            seq.push_back(t);
            if (cfg.eos_token_id >= 0 && t == cfg.eos_token_id) break;
        }
        return seq;
    }

    // Prefill only: fp32 logits of the last prompt token.
    std::vector<float> prefill_logits(const std::vector<int>& input_ids) {
        std::vector<float> logits(size_t(config().vocab_size));
        const int rc = b200p_session_prefill_logits(s_, input_ids.data(), int(input_ids.size()), logits.data(), nullptr);
        if (rc) throw std::runtime_error(std::string("Session::prefill_logits: ") + b200p_strerror(rc));
        return logits;
    }
};

} // namespace runtime
} // namespace cdna3
