// The part registries and the small pieces of parts.h that need a home.
#include <mutex>

#include "parts.h"

namespace qe {

void ModelSpec::validate() const {
    const int n = (int)layers.size();
    for (size_t i = 0; i < schedule.size(); i++) {
        const LayerCall& call = schedule[i];
        if (call.layer < 0 || call.layer >= n)
            throw ConfigError("schedule[" + std::to_string(i) + "] names layer " + std::to_string(call.layer) +
                              ", the model has " + std::to_string(n));
        if (call.cache_from >= 0) {
            if (call.cache_from >= (int)i)
                throw ConfigError("schedule[" + std::to_string(i) + "].cache_from must name an earlier call, got " +
                                  std::to_string(call.cache_from));
            if (schedule[call.cache_from].cache_from >= 0)
                throw ConfigError("schedule[" + std::to_string(i) + "].cache_from names a call that itself borrows a cache");
        }
    }
    if (position_columns < 1) throw ConfigError("a model carries at least one column of positions");
}

std::shared_ptr<Part> BuildContext::shared(const std::string& key, const std::function<std::shared_ptr<Part>()>& make) {
    auto it = shared_.find(key);
    if (it == shared_.end()) it = shared_.emplace(key, make()).first;
    return it->second;
}

Part::Part(const Json& p, BuildContext& build) : params(p), compute_dtype(build.compute_dtype) {
    if (const Json* n = p.find("names")) {
        if (!n->is_object()) throw ConfigError("a part's 'names' must map roles to tensor names");
        for (const auto& m : n->members()) names_[m.first] = m.second.as_string();
    }
}

const std::string& Part::name_of(const std::string& role) const {
    auto it = names_.find(role);
    if (it == names_.end()) throw ConfigError("a part's 'names' gives no tensor for the role '" + role + "'");
    return it->second;
}

namespace {
std::mutex g_mutex;
std::map<std::string, std::map<std::string, PartFactory>>& tables() {
    static std::map<std::string, std::map<std::string, PartFactory>> t = {
        {"norm", {}}, {"position", {}}, {"mixer", {}}, {"feed_forward", {}}, {"embedding", {}}, {"head", {}}};
    return t;
}
std::map<std::string, ArrangementFactory>& arrangements() {
    static std::map<std::string, ArrangementFactory> t;
    return t;
}
std::string known(const std::map<std::string, PartFactory>& t) {
    std::string s;
    for (const auto& kv : t) s += (s.empty() ? "" : ", ") + kv.first;
    return s.empty() ? "(none)" : s;
}
}  // namespace

void register_part(const std::string& family, const std::string& kind, PartFactory factory) {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = tables().find(family);
    if (it == tables().end()) throw ConfigError("there is no part family '" + family + "'");
    it->second[kind] = std::move(factory);
}
void unregister_part(const std::string& family, const std::string& kind) {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = tables().find(family);
    if (it != tables().end()) it->second.erase(kind);
}
std::shared_ptr<Part> make_part(const std::string& family, const PartSpec& spec, BuildContext& build) {
    PartFactory f;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = tables().find(family);
        if (it == tables().end()) throw ConfigError("there is no part family '" + family + "'");
        auto k = it->second.find(spec.kind);
        if (k == it->second.end())
            throw ConfigError("no " + family + " part of kind '" + spec.kind + "' is registered (have: " + known(it->second) + ")");
        f = k->second;
    }
    return f(spec.params, build);
}
std::vector<std::string> registered_parts(const std::string& family) {
    std::lock_guard<std::mutex> lock(g_mutex);
    std::vector<std::string> out;
    if (family == "arrangement") {
        for (const auto& kv : arrangements()) out.push_back(kv.first);
        return out;
    }
    auto it = tables().find(family);
    if (it != tables().end())
        for (const auto& kv : it->second) out.push_back(kv.first);
    return out;
}
void register_arrangement(const std::string& kind, ArrangementFactory factory) {
    std::lock_guard<std::mutex> lock(g_mutex);
    arrangements()[kind] = std::move(factory);
}
void unregister_arrangement(const std::string& kind) {
    std::lock_guard<std::mutex> lock(g_mutex);
    arrangements().erase(kind);
}
std::unique_ptr<Arrangement> make_arrangement(const LayerSpec& layer, BuildContext& build) {
    ArrangementFactory f;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = arrangements().find(layer.arrangement);
        if (it == arrangements().end()) throw ConfigError("no block arrangement '" + layer.arrangement + "' is registered");
        f = it->second;
    }
    return f(layer, build);
}

}  // namespace qe
