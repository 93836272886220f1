#include "config.h"

#include <cerrno>
#include <cmath>
#include <fstream>
#include <mutex>
#include <sstream>

namespace qe {

namespace {
std::mutex g_mutex;
std::map<std::string, Architecture>& registry() {
    static std::map<std::string, Architecture> r;
    return r;
}
std::string brief(const Json& v) {
    std::string s = v.dump();
    return s.size() > 60 ? s.substr(0, 57) + "..." : s;
}
}  // namespace

void register_architecture(const std::string& name, std::function<std::unique_ptr<ModelConfig>(const Json&)> read) {
    std::lock_guard<std::mutex> lock(g_mutex);
    registry()[name] = Architecture{name, std::move(read)};
}
void unregister_architecture(const std::string& name) {
    std::lock_guard<std::mutex> lock(g_mutex);
    registry().erase(name);
}
std::vector<std::string> registered_architectures() {
    std::lock_guard<std::mutex> lock(g_mutex);
    std::vector<std::string> out;
    for (const auto& kv : registry()) out.push_back(kv.first);
    return out;
}
const Architecture& lookup_architecture(const std::string& name) {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = registry().find(name);
    if (it == registry().end()) {
        std::string have;
        for (const auto& kv : registry()) have += (have.empty() ? "" : ", ") + kv.first;
        throw ConfigError("unsupported architecture '" + name + "'; registered: " + (have.empty() ? "(none)" : have));
    }
    return it->second;
}

Json read_config_json(const std::string& model_dir) {
    const std::string path = model_dir + "/config.json";
    std::ifstream f(path, std::ios::binary);
    if (!f) throw ConfigError(path + ": no config.json in the model folder");
    std::ostringstream ss;
    ss << f.rdbuf();
    Json d;
    try {
        d = Json::parse(ss.str());
    } catch (const JsonError& e) {
        throw ConfigError(path + ": not valid JSON (" + e.what() + ")");
    }
    if (!d.is_object()) throw ConfigError(path + ": the top level must be an object");
    return d;
}

std::string architecture_name(const Json& d) {
    const Json* a = d.find("architectures");
    if (!a || !a->is_array() || a->size() == 0 || !(*a)[0].is_string())
        throw ConfigError("config.json: 'architectures' must be a non-empty list of names");
    return (*a)[0].as_string();
}

std::unique_ptr<ModelConfig> config_from_json(const Json& d) {
    if (!d.is_object()) throw ConfigError("config.json: the top level must be an object");
    register_builtin_architectures();
    Architecture arch = lookup_architecture(architecture_name(d));
    std::unique_ptr<ModelConfig> c = arch.read(d);
    c->architecture = arch.name;
    return c;
}
std::unique_ptr<ModelConfig> load_config(const std::string& model_dir) { return config_from_json(read_config_json(model_dir)); }

// ---- typed reading ----------------------------------------------------------------------------------------------
bool has_value(const Json& d, const std::string& key) {
    const Json* v = d.find(key);
    return v && !v->is_null();
}
static long long int_of(const Json& v, const std::string& key, long long minimum) {
    long long n;
    if (v.is_int()) n = v.as_int();
    else if (v.kind() == Json::Real && v.as_double() == std::floor(v.as_double())) n = (long long)v.as_double();
    else throw ConfigError("config.json: '" + key + "' must be an integer, got " + brief(v));
    if (n < minimum) throw ConfigError("config.json: '" + key + "' must be >= " + std::to_string(minimum) + ", got " + std::to_string(n));
    return n;
}
long long take_int(const Json& d, const std::string& key, long long minimum) {
    if (!has_value(d, key)) throw ConfigError("config.json: missing key '" + key + "'");
    return int_of(d.at(key), key, minimum);
}
long long take_int(const Json& d, const std::string& key, long long dflt, long long minimum) {
    return has_value(d, key) ? int_of(d.at(key), key, minimum) : dflt;
}
double take_float(const Json& d, const std::string& key) {
    if (!has_value(d, key)) throw ConfigError("config.json: missing key '" + key + "'");
    const Json& v = d.at(key);
    if (!v.is_number()) throw ConfigError("config.json: '" + key + "' must be a number, got " + brief(v));
    return v.as_double();
}
double take_float(const Json& d, const std::string& key, double dflt) { return has_value(d, key) ? take_float(d, key) : dflt; }
bool take_bool(const Json& d, const std::string& key, bool dflt) {
    if (!has_value(d, key)) return dflt;
    const Json& v = d.at(key);
    if (!v.is_bool()) throw ConfigError("config.json: '" + key + "' must be true or false, got " + brief(v));
    return v.as_bool();
}

// ---- Qwen3 ---------------------------------------------------------------------------------------------------------
static const char* kFull = "full_attention";
static const char* kSliding = "sliding_attention";

std::unique_ptr<ModelConfig> Qwen3Config::read(const Json& d) {
    std::unique_ptr<Qwen3Config> c(new Qwen3Config());
    const Json* archs = d.find("architectures");
    c->architecture = (archs && archs->is_array() && archs->size() && (*archs)[0].is_string()) ? (*archs)[0].as_string() : "Qwen3ForCausalLM";
    c->num_hidden_layers = take_int(d, "num_hidden_layers");
    c->hidden_size = take_int(d, "hidden_size");
    c->num_attention_heads = take_int(d, "num_attention_heads");
    c->num_key_value_heads = take_int(d, "num_key_value_heads", c->num_attention_heads, 1);
    if (has_value(d, "head_dim")) c->head_dim = take_int(d, "head_dim");
    else {
        if (c->hidden_size % c->num_attention_heads)
            throw ConfigError("config.json: no 'head_dim' and hidden_size " + std::to_string(c->hidden_size) +
                              " is not a multiple of num_attention_heads " + std::to_string(c->num_attention_heads));
        c->head_dim = c->hidden_size / c->num_attention_heads;
    }
    const Json* rope_params = d.find("rope_parameters");
    if (rope_params && !rope_params->is_object()) rope_params = nullptr;
    const Json* theta = has_value(d, "rope_theta") ? &d.at("rope_theta") : nullptr;
    if (!theta && rope_params && has_value(*rope_params, "rope_theta")) theta = &rope_params->at("rope_theta");
    if (theta) {
        if (!theta->is_number() || !(theta->as_double() > 0))
            throw ConfigError("config.json: 'rope_theta' must be a positive number, got " + brief(*theta));
        c->rope_theta = theta->as_double();
    }
    // plain rotary position encoding only: any other rope type is refused by name
    std::string rope_type;
    if (has_value(d, "rope_scaling")) {
        const Json& s = d.at("rope_scaling");
        if (s.is_object()) rope_type = s.get_string("rope_type", s.get_string("type", ""));
        else if (s.is_string()) rope_type = s.as_string();
        else rope_type = brief(s);
    } else if (rope_params) {
        rope_type = rope_params->get_string("rope_type", "default");
    }
    if (!rope_type.empty() && rope_type != "default")
        throw ConfigError("config.json: rope scaling '" + rope_type + "' is not supported (only plain rotary position encoding)");
    const std::string act = d.get_string("hidden_act", "silu");
    if (act != "silu") throw ConfigError("config.json: hidden_act '" + act + "' is not supported (silu only)");

    const long long n = c->num_hidden_layers;
    long long window = has_value(d, "sliding_window") ? take_int(d, "sliding_window") : 0;
    const bool use_window = take_bool(d, "use_sliding_window", false);
    if (has_value(d, "layer_types")) {
        const Json& lt = d.at("layer_types");
        bool ok = lt.is_array() && (long long)lt.size() == n;
        if (ok)
            for (const Json& t : lt.items()) ok = ok && t.is_string() && (t.as_string() == kFull || t.as_string() == kSliding);
        if (!ok)
            throw ConfigError("config.json: 'layer_types' must list " + std::to_string(n) + " entries of '" + kFull + "' / '" + kSliding + "'");
        for (const Json& t : lt.items()) c->layer_types.push_back(t.as_string());
    } else if (use_window) {
        const long long first = take_int(d, "max_window_layers", n, 0);
        for (long long i = 0; i < n; i++) c->layer_types.push_back(i >= first ? kSliding : kFull);
    } else {
        c->layer_types.assign((size_t)n, kFull);
    }
    bool slides = false;
    for (const auto& t : c->layer_types) slides |= (t == kSliding);
    if (slides && window == 0) throw ConfigError("config.json: a layer uses sliding attention but 'sliding_window' is not given");
    c->sliding_window = slides ? window : 0;

    c->intermediate_size = take_int(d, "intermediate_size");
    c->vocab_size = take_int(d, "vocab_size");
    c->max_position_embeddings = take_int(d, "max_position_embeddings", 4096, 1);
    c->rms_norm_eps = take_float(d, "rms_norm_eps", 1e-6);
    c->tie_word_embeddings = take_bool(d, "tie_word_embeddings", false);
    c->attention_bias = take_bool(d, "attention_bias", false);
    if (has_value(d, "eos_token_id")) {
        const Json& e = d.at("eos_token_id");
        if (e.is_int()) c->eos_ids.push_back((int)e.as_int());
        else if (e.is_array())
            for (const Json& v : e.items()) if (v.is_int()) c->eos_ids.push_back((int)v.as_int());
    }
    c->validate();
    return std::unique_ptr<ModelConfig>(c.release());
}

void Qwen3Config::validate() const {
    if (num_attention_heads % num_key_value_heads)
        throw ConfigError("num_attention_heads " + std::to_string(num_attention_heads) + " is not a multiple of num_key_value_heads " +
                          std::to_string(num_key_value_heads));
    if (head_dim % 2) throw ConfigError("head_dim " + std::to_string(head_dim) + " must be even (rotary pairs)");
    if (!(rms_norm_eps > 0)) throw ConfigError("rms_norm_eps must be > 0, got " + std::to_string(rms_norm_eps));
}

Json Qwen3Config::to_json() const {
    Json d = Json::object();
    Json archs = Json::array();
    archs.push(architecture.empty() ? std::string("Qwen3ForCausalLM") : architecture);
    d.set("architectures", archs);
    d.set("model_type", "qwen3");
    d.set("num_hidden_layers", num_hidden_layers);
    d.set("hidden_size", hidden_size);
    d.set("intermediate_size", intermediate_size);
    d.set("num_attention_heads", num_attention_heads);
    d.set("num_key_value_heads", num_key_value_heads);
    d.set("head_dim", head_dim);
    d.set("vocab_size", vocab_size);
    d.set("max_position_embeddings", max_position_embeddings);
    d.set("rope_theta", rope_theta);
    d.set("rms_norm_eps", rms_norm_eps);
    d.set("tie_word_embeddings", tie_word_embeddings);
    d.set("attention_bias", attention_bias);
    d.set("hidden_act", "silu");
    if (sliding_window) {
        d.set("use_sliding_window", true);
        d.set("sliding_window", sliding_window);
        Json lt = Json::array();
        for (const auto& t : layer_types) lt.push(t);
        d.set("layer_types", lt);
    } else {
        d.set("use_sliding_window", false);
    }
    if (!eos_ids.empty()) {
        Json e = Json::array();
        for (int id : eos_ids) e.push(id);
        d.set("eos_token_id", e);
    }
    return d;
}

long long Qwen3Config::parameter_count() const {
    const long long e = hidden_size, ff = intermediate_size, v = vocab_size;
    long long per_layer = (q_width() + 2 * kv_width()) * e + e * q_width() + 3 * e * ff + 2 * e + 2 * head_dim;
    if (attention_bias) per_layer += q_width() + 2 * kv_width();
    long long total = num_hidden_layers * per_layer + v * e + e;
    if (!tie_word_embeddings) total += v * e;
    return total;
}

// Qwen3 dense as parts: per layer RMSNorm -> grouped-query attention (per-head RMSNorm on q and k, rotate-half
// rotary) -> residual, RMSNorm -> SwiGLU -> residual; then a final RMSNorm and the output matrix, shared with the
// embedding when tie_word_embeddings (the order of src/qwen_model.cpp:1196-1279 with full_attention :940-975 and
// ffn :1170-1189).
ModelSpec Qwen3Config::build_spec() const {
    auto names = [](std::initializer_list<std::pair<const char*, std::string>> list) {
        Json n = Json::object();
        for (const auto& kv : list) n.set(kv.first, kv.second);
        return n;
    };
    auto norm = [&](const std::string& weight) {
        Json p = Json::object();
        p.set("size", hidden_size);
        p.set("eps", rms_norm_eps);
        p.set("names", names({{"weight", weight}}));
        return PartSpec("rmsnorm", p);
    };
    Json pos_params = Json::object();
    pos_params.set("theta", rope_theta);
    pos_params.set("n_rot", head_dim);
    pos_params.set("max_position", max_position_embeddings);
    const PartSpec position("rope_neox", pos_params);

    ModelSpec spec;
    spec.hidden_size = hidden_size;
    spec.vocab_size = vocab_size;
    spec.max_position = max_position_embeddings;
    for (long long i = 0; i < num_hidden_layers; i++) {
        const std::string p = "model.layers." + std::to_string(i) + ".";
        Json n = names({{"q_proj", p + "self_attn.q_proj.weight"}, {"k_proj", p + "self_attn.k_proj.weight"},
                        {"v_proj", p + "self_attn.v_proj.weight"}, {"o_proj", p + "self_attn.o_proj.weight"},
                        {"q_norm", p + "self_attn.q_norm.weight"}, {"k_norm", p + "self_attn.k_norm.weight"}});
        if (attention_bias) {
            n.set("q_bias", p + "self_attn.q_proj.bias");
            n.set("k_bias", p + "self_attn.k_proj.bias");
            n.set("v_bias", p + "self_attn.v_proj.bias");
        }
        Json a = Json::object();
        a.set("hidden_size", hidden_size);
        a.set("num_heads", num_attention_heads);
        a.set("num_kv_heads", num_key_value_heads);
        a.set("head_dim", head_dim);
        a.set("qk_norm_eps", rms_norm_eps);
        a.set("bias", attention_bias);
        a.set("position", position.to_json());
        a.set("window", layer_types[(size_t)i] == kSliding ? Json(sliding_window) : Json());
        a.set("names", n);
        Json f = Json::object();
        f.set("hidden_size", hidden_size);
        f.set("intermediate_size", intermediate_size);
        f.set("names", names({{"gate_proj", p + "mlp.gate_proj.weight"}, {"up_proj", p + "mlp.up_proj.weight"},
                              {"down_proj", p + "mlp.down_proj.weight"}}));
        LayerSpec layer;
        layer.arrangement = "pre_norm";
        layer.parts = {{"mixer_norm", norm(p + "input_layernorm.weight")},
                       {"mixer", PartSpec("attention", a)},
                       {"feed_forward_norm", norm(p + "post_attention_layernorm.weight")},
                       {"feed_forward", PartSpec("swiglu", f)}};
        spec.layers.push_back(std::move(layer));
        spec.schedule.push_back(LayerCall{(int)i, -1});
    }
    const std::string embed_name = "model.embed_tokens.weight";
    Json e = Json::object();
    e.set("vocab_size", vocab_size);
    e.set("hidden_size", hidden_size);
    e.set("names", names({{"weight", embed_name}}));
    spec.embedding = PartSpec("embedding", e);
    Json h = Json::object();
    h.set("hidden_size", hidden_size);
    h.set("vocab_size", vocab_size);
    if (tie_word_embeddings) {
        h.set("tied_to", embed_name);
        Json ig = Json::array();
        ig.push("lm_head.weight");
        h.set("ignore", ig);
    } else {
        h.set("names", names({{"weight", "lm_head.weight"}}));
    }
    spec.head = PartSpec("lm_head", h);
    spec.final_norm = norm("model.norm.weight");
    spec.validate();
    return spec;
}

void register_builtin_architectures() {
    static std::once_flag once;
    std::call_once(once, [] { register_architecture("Qwen3ForCausalLM", Qwen3Config::read); });
}

}  // namespace qe
