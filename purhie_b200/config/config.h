// Typed model configurations and the architecture registry.
//
// A configuration is read from the keys of the architecture's own config.json; no size or constant that
// config.json gives is written in code anywhere else in the library.  The registry maps the name in
// architectures[0] to a function that reads a typed configuration and to one that turns it into a ModelSpec
// (the description from which the generic decoder is assembled).  The reference keeps the same mapping as a
// whitelist of architecture names (src/inference.cpp:1237-1239, error for an unknown one at :1267-1268) and, on
// the converter side, as a name -> package registry (perl/ROCm-Inference/lib/ROCm/Inference/Convert.pm:34,
// 1475-1479).
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "../host/common.h"
#include "../host/json.h"
#include "../parts/parts.h"

namespace qe {

// Base of every architecture's configuration.
class QE_API ModelConfig {
public:
    virtual ~ModelConfig() = default;
    std::string architecture;
    virtual Json to_json() const = 0;                // the config.json this configuration would be read from
    virtual ModelSpec build_spec() const = 0;
    virtual std::vector<int> eos_token_ids() const { return {}; }
};

struct Architecture {
    std::string name;
    std::function<std::unique_ptr<ModelConfig>(const Json&)> read;     // throws ConfigError
};

QE_API void register_architecture(const std::string& name, std::function<std::unique_ptr<ModelConfig>(const Json&)> read);
QE_API void unregister_architecture(const std::string& name);
QE_API std::vector<std::string> registered_architectures();
QE_API const Architecture& lookup_architecture(const std::string& name);      // ConfigError naming what is registered

QE_API Json read_config_json(const std::string& model_dir);                     // ConfigError: missing, not JSON, not an object
QE_API std::string architecture_name(const Json& config);
QE_API std::unique_ptr<ModelConfig> config_from_json(const Json& config);       // through the registry
QE_API std::unique_ptr<ModelConfig> load_config(const std::string& model_dir);

// ---- helpers for typed reading: every error names the key --------------------------------------------------------
QE_API long long take_int(const Json& d, const std::string& key, long long minimum = 1);
QE_API long long take_int(const Json& d, const std::string& key, long long dflt, long long minimum);
QE_API bool has_value(const Json& d, const std::string& key);                   // present and not null
QE_API double take_float(const Json& d, const std::string& key);
QE_API double take_float(const Json& d, const std::string& key, double dflt);
QE_API bool take_bool(const Json& d, const std::string& key, bool dflt);

// ---- Qwen3 dense ("Qwen3ForCausalLM") ---------------------------------------------------------------------------------
// Keys and their meaning follow the reference: the converter reads num_hidden_layers, hidden_size,
// intermediate_size, num_attention_heads, num_key_value_heads, head_dim, max_position_embeddings, rope_theta
// (plain or inside rope_parameters) and rms_norm_eps (Convert.pm:72-80, 555-615); the loader's defaults are
// head_dim = hidden/heads (src/inference.cpp:1326), context 4096 (:1338-1339), rope base 10000 (:1359) and eps
// 1e-6 (:1360); a missing lm_head.weight means a tied head (:1392-1396) and optional q/k/v biases are bound when
// present (:631-633).  The window keys (use_sliding_window, sliding_window, max_window_layers, layer_types)
// choose, layer by layer, between attention over all earlier positions and attention over the last
// sliding_window of them (the meaning of `window` in src/attention.h:73: a token at p sees positions
// > p - window); the reference itself runs Qwen3 without windows, so that reading rests on that line alone.
class QE_API Qwen3Config : public ModelConfig {
public:
    long long num_hidden_layers = 0, hidden_size = 0, intermediate_size = 0, num_attention_heads = 0;
    long long num_key_value_heads = 0, head_dim = 0, vocab_size = 0, max_position_embeddings = 0;
    double rope_theta = 10000.0, rms_norm_eps = 1e-6;
    bool tie_word_embeddings = false, attention_bias = false;
    std::vector<std::string> layer_types;            // "full_attention" | "sliding_attention" per layer
    long long sliding_window = 0;                    // 0: no layer slides
    std::vector<int> eos_ids;

    static std::unique_ptr<ModelConfig> read(const Json& d);
    void validate() const;
    Json to_json() const override;
    ModelSpec build_spec() const override;
    std::vector<int> eos_token_ids() const override { return eos_ids; }
    long long q_width() const { return num_attention_heads * head_dim; }
    long long kv_width() const { return num_key_value_heads * head_dim; }
    long long parameter_count() const;
};

QE_API void register_builtin_architectures();

}  // namespace qe
