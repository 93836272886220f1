#include "weights.h"

#include <sys/stat.h>

#include <algorithm>
#include <cerrno>
#include <fstream>
#include <set>
#include <thread>

#include "../parts/model.h"
#include "random.h"

namespace qe {

DType device_dtype(DType stored, Role role, DType compute) {
    if (role == Role::Table) return DType::I32;
    if (role == Role::Vector || compute == DType::F32) return DType::F32;
    if (stored == DType::F32 || stored == DType::F64) return DType::F32;
    return DType::BF16;
}

void check_folder(const SafetensorsFolder& folder, const std::vector<TensorSpec>& expected, const std::vector<std::string>& ignore) {
    std::set<std::string> wanted, ignored(ignore.begin(), ignore.end());
    WeightError err("");
    for (const TensorSpec& s : expected) {
        wanted.insert(s.name);
        const TensorEntry* e = folder.find(s.name);
        if (!e) { err.missing.push_back(s.name); continue; }
        if (e->shape != s.shape)
            err.wrong_shape.push_back(s.name + " is " + shape_text(e->shape) + ", expected " + shape_text(s.shape));
        const bool ok = s.role == Role::Table ? dtype_is_int(e->dtype) : dtype_is_float(e->dtype);
        if (!ok) err.wrong_type.push_back(s.name + " is stored as " + e->dtype_name + ", which a " + role_name(s.role) + " cannot be");
    }
    for (const std::string& n : folder.names())
        if (!wanted.count(n) && !ignored.count(n)) err.unexpected.push_back(n);
    std::sort(err.unexpected.begin(), err.unexpected.end());
    if (err.missing.empty() && err.unexpected.empty() && err.wrong_shape.empty() && err.wrong_type.empty()) return;
    auto join = [](const std::vector<std::string>& v) {
        std::string s;
        for (const auto& x : v) s += (s.empty() ? "" : ", ") + x;
        return s;
    };
    std::string text = folder.model_dir() + ": the tensors do not fit the model";
    if (!err.missing.empty()) text += "\n  missing (" + std::to_string(err.missing.size()) + "): " + join(err.missing);
    if (!err.unexpected.empty()) text += "\n  unexpected (" + std::to_string(err.unexpected.size()) + "): " + join(err.unexpected);
    for (const auto& w : err.wrong_shape) text += "\n  wrong shape: " + w;
    for (const auto& w : err.wrong_type) text += "\n  wrong type: " + w;
    WeightError full(text);
    full.missing = err.missing; full.unexpected = err.unexpected; full.wrong_shape = err.wrong_shape; full.wrong_type = err.wrong_type;
    throw full;
}

// ---- a checkpoint folder ------------------------------------------------------------------------------------------
FolderSource::FolderSource(const std::string& model_dir, const std::vector<TensorSpec>& expected, const std::vector<std::string>& ignore,
                           DType compute, DeviceArena& arena, cudaStream_t stream)
    : folder_(model_dir), compute_(compute), arena_(arena), stream_(stream) {
    check_folder(folder_, expected, ignore);
    for (const TensorSpec& s : expected) specs_[s.name] = s;
}

namespace {
double read_as_double(const uint8_t* p, DType d, size_t i) {
    switch (d) {
        case DType::F64: { double v; memcpy(&v, p + 8 * i, 8); return v; }
        case DType::F32: { float v; memcpy(&v, p + 4 * i, 4); return v; }
        case DType::BF16: { uint16_t v; memcpy(&v, p + 2 * i, 2); return bf16_to_f32(v); }
        case DType::F16: { uint16_t v; memcpy(&v, p + 2 * i, 2); return f16_to_f32(v); }
        case DType::I64: { int64_t v; memcpy(&v, p + 8 * i, 8); return (double)v; }
        case DType::I32: { int32_t v; memcpy(&v, p + 4 * i, 4); return v; }
        case DType::I16: { int16_t v; memcpy(&v, p + 2 * i, 2); return v; }
        case DType::I8: return (int8_t)p[i];
        default: return p[i];
    }
}
}  // namespace

Tensor FolderSource::fetch(const std::string& name) {
    auto hit = cache_.find(name);
    if (hit != cache_.end()) return hit->second;
    auto sp = specs_.find(name);
    if (sp == specs_.end()) throw Error(kInvalidState, "a part asks for the tensor '" + name + "' that it did not announce");
    const TensorEntry& e = folder_.at(name);
    const DType want = device_dtype(e.dtype, sp->second.role, compute_);
    Tensor t = arena_.alloc(want, e.shape);
    const size_t n = (size_t)e.numel();
    if (n) {
        if (want == e.dtype) {
            QE_CUDA(cudaMemcpy(t.data, e.data, e.bytes, cudaMemcpyHostToDevice));         // straight from the mapping
        } else {
            // converted on the host in slices, so that a large tensor needs no second copy in memory
            const size_t slice = std::min<size_t>(n, (size_t)8 << 20);
            std::vector<uint8_t> buf(slice * dtype_size(want));
            for (size_t first = 0; first < n; first += slice) {
                const size_t m = std::min(slice, n - first);
                for (size_t i = 0; i < m; i++) {
                    const double v = read_as_double(e.data, e.dtype, first + i);
                    if (want == DType::F32) { float f = (float)v; memcpy(buf.data() + 4 * i, &f, 4); }
                    else if (want == DType::BF16) { uint16_t h = f32_to_bf16((float)v); memcpy(buf.data() + 2 * i, &h, 2); }
                    else { int32_t k = (int32_t)v; memcpy(buf.data() + 4 * i, &k, 4); }
                }
                QE_CUDA(cudaMemcpy(static_cast<char*>(t.data) + first * dtype_size(want), buf.data(), m * dtype_size(want),
                                   cudaMemcpyHostToDevice));
            }
        }
    }
    cache_[name] = t;
    return t;
}

// ---- the random generator ------------------------------------------------------------------------------------------
namespace {
void random_kind(const TensorSpec& spec, const RandomInit& init, int& kind, double& a, double& b) {
    if (spec.role == Role::Table) throw Error(kInvalidArg, spec.name + ": integer tables have no random fill");
    if (spec.init == Init::Scale) {
        if (init.scale_low == init.scale_high) { kind = 2; a = init.scale_low; b = 0; }
        else { kind = 1; a = init.scale_low; b = init.scale_high; }
    } else { kind = 0; a = init.std; b = 0; }
}
}  // namespace

RandomSource::RandomSource(const std::vector<TensorSpec>& expected, const RandomInit& init, DType stored, DType compute,
                           DeviceArena& arena, cudaStream_t stream)
    : init_(init), stored_(stored), compute_(compute), arena_(arena), stream_(stream) {
    for (const TensorSpec& s : expected) specs_[s.name] = s;
}

Tensor RandomSource::fetch(const std::string& name) {
    auto hit = cache_.find(name);
    if (hit != cache_.end()) return hit->second;
    auto sp = specs_.find(name);
    if (sp == specs_.end()) throw Error(kInvalidState, "a part asks for the tensor '" + name + "' that it did not announce");
    const TensorSpec& spec = sp->second;
    int kind; double a, b;
    random_kind(spec, init_, kind, a, b);
    const DType stored = spec.role == Role::Matrix ? stored_ : DType::F32;
    const DType want = device_dtype(stored, spec.role, compute_);
    Tensor t = arena_.alloc(want, spec.shape);
    const CoreKernels& k = core_kernels();
    const uint64_t key = rnd::tensor_key(init_.seed, name.c_str());
    if (stored == DType::BF16 && want == DType::F32) {
        // a folder would hold bfloat16 values, widened at load: round through bfloat16
        Tensor tmp = arena_.alloc(DType::BF16, spec.shape);
        QE_LAUNCH(k, k.random_fill(tmp.data, tmp.code(), t.numel(), key, kind, a, b, stream_));
        QE_LAUNCH(k, k.cast(tmp.data, tmp.code(), t.data, t.code(), t.numel(), stream_));
        QE_CUDA(cudaStreamSynchronize(stream_));
        arena_.release(tmp);
    } else {
        QE_LAUNCH(k, k.random_fill(t.data, t.code(), t.numel(), key, kind, a, b, stream_));
    }
    cache_[name] = t;
    return t;
}

std::vector<TensorSpec> expected_tensors(const ModelConfig& config) {
    return DecoderModel(config.build_spec(), DType::F32).tensor_specs();
}

std::vector<float> random_tensor_host(const TensorSpec& spec, const RandomInit& init) {
    int kind; double a, b;
    random_kind(spec, init, kind, a, b);
    size_t n = 1;
    for (auto s : spec.shape) n *= (size_t)s;
    std::vector<float> out(n);
    const uint64_t key = rnd::tensor_key(init.seed, spec.name.c_str());
    for (size_t i = 0; i < n; i++) out[i] = rnd::random_value(key, i, kind, a, b);
    return out;
}

void write_random_model(const std::string& model_dir, const ModelConfig& config, const RandomInit& init, DType matrix_dtype,
                        DType vector_dtype) {
    for (DType d : {matrix_dtype, vector_dtype})
        if (d != DType::BF16 && d != DType::F32) throw Error(kInvalidArg, "random models are stored as bfloat16 or float32");
    if (mkdir(model_dir.c_str(), 0777) != 0 && errno != EEXIST) {
        // create missing parents one by one
        for (size_t i = 1; i <= model_dir.size(); i++)
            if (i == model_dir.size() || model_dir[i] == '/') mkdir(model_dir.substr(0, i).c_str(), 0777);
    }
    Json cfg = config.to_json();
    cfg.set("torch_dtype", matrix_dtype == DType::BF16 ? "bfloat16" : "float32");
    {
        std::ofstream f(model_dir + "/config.json", std::ios::binary);
        if (!f) throw Error(kModelLoad, model_dir + "/config.json: cannot write");
        f << cfg.dump(1) << "\n";
    }
    std::vector<TensorToWrite> out;
    for (const TensorSpec& spec : expected_tensors(config)) {
        TensorToWrite t;
        t.name = spec.name;
        t.dtype = spec.role == Role::Matrix ? matrix_dtype : vector_dtype;
        t.shape = spec.shape;
        const DType dt = t.dtype;
        t.fill = [spec, init, dt](uint8_t* dst) {
            int kind; double a, b;
            random_kind(spec, init, kind, a, b);
            size_t n = 1;
            for (auto s : spec.shape) n *= (size_t)s;
            const uint64_t key = rnd::tensor_key(init.seed, spec.name.c_str());
            // every element is a function of its index: slices of a large tensor are filled by threads side by side
            auto fill_range = [=](size_t first, size_t last) {
                for (size_t i = first; i < last; i++) {
                    const float v = rnd::random_value(key, i, kind, a, b);
                    if (dt == DType::F32) memcpy(dst + 4 * i, &v, 4);
                    else { uint16_t h = f32_to_bf16(v); memcpy(dst + 2 * i, &h, 2); }
                }
            };
            const size_t workers = n < (1u << 16) ? 1 : std::max(1u, std::min(32u, std::thread::hardware_concurrency()));
            if (workers == 1) { fill_range(0, n); return; }
            std::vector<std::thread> pool;
            const size_t per = (n + workers - 1) / workers;
            for (size_t w = 0; w < workers; w++)
                if (w * per < n) pool.emplace_back(fill_range, w * per, std::min(n, (w + 1) * per));
            for (std::thread& t : pool) t.join();
        };
        out.push_back(std::move(t));
    }
    Json meta = Json::object();
    meta.set("format", "pt");
    meta.set("seed", std::to_string(init.seed));
    write_safetensors(model_dir + "/model.safetensors", out, meta);
}

}  // namespace qe
