#include "device.h"

#include <dlfcn.h>

#include <mutex>

namespace qe {

long long g_launches = 0;

// ---- memory -------------------------------------------------------------------------------------------------
DeviceBuffer::DeviceBuffer(size_t bytes) : n_(bytes) {
    if (bytes) {
        cudaError_t e = cudaMalloc(&p_, bytes);
        if (e != cudaSuccess) {
            p_ = nullptr;
            n_ = 0;
            throw Error(e == cudaErrorMemoryAllocation ? kOutOfMemory : kKernelLaunch,
                        "cudaMalloc of " + std::to_string(bytes) + " bytes: " + cudaGetErrorString(e));
        }
    }
}
DeviceBuffer::~DeviceBuffer() { reset(); }
DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) {
        reset();
        p_ = o.p_; n_ = o.n_;
        o.p_ = nullptr; o.n_ = 0;
    }
    return *this;
}
void DeviceBuffer::reset() {
    if (p_) cudaFree(p_);
    p_ = nullptr;
    n_ = 0;
}

PinnedBuffer::PinnedBuffer(size_t bytes) { ensure(bytes); }
PinnedBuffer::~PinnedBuffer() { if (p_) cudaFreeHost(p_); }
void PinnedBuffer::ensure(size_t bytes) {
    if (bytes <= n_) return;
    if (p_) cudaFreeHost(p_);
    p_ = nullptr; n_ = 0;
    QE_CUDA(cudaMallocHost(&p_, bytes));
    n_ = bytes;
}

Tensor DeviceArena::alloc(DType dtype, std::vector<int64_t> shape) {
    Tensor t(nullptr, dtype, std::move(shape));
    DeviceBuffer b(std::max<size_t>(t.bytes(), 16));
    t.data = b.data();
    bytes_ += b.bytes();
    bufs_.emplace(t.data, std::move(b));
    return t;
}
void DeviceArena::release(const Tensor& t) {
    auto it = bufs_.find(t.data);
    if (it == bufs_.end()) return;
    bytes_ -= it->second.bytes();
    bufs_.erase(it);
}

Tensor Workspace::get(const std::string& name, std::vector<int64_t> shape, DType dtype) {
    Tensor t(nullptr, dtype, std::move(shape));
    size_t need = std::max<size_t>(t.bytes(), 16);
    auto it = bufs_.find(name);
    if (it == bufs_.end() || it->second.bytes() < need) {
        if (frozen) throw Error(kInvalidState, "workspace buffer '" + name + "' would have to grow while frozen");
        if (it != bufs_.end()) {
            QE_CUDA(cudaStreamSynchronize(stream));        // a kernel in flight may still use the old block
            bufs_.erase(it);
        }
        it = bufs_.emplace(name, DeviceBuffer(need)).first;
    }
    t.data = it->second.data();
    return t;
}
size_t Workspace::bytes() const {
    size_t n = 0;
    for (const auto& kv : bufs_) n += kv.second.bytes();
    return n;
}

// ---- kernel libraries -----------------------------------------------------------------------------------------
namespace {
std::mutex g_lib_mutex;
std::string g_lib_dir;
std::map<std::string, void*> g_handles;
CoreKernels g_core{};
FlashKernels g_flash{};
GemmKernels g_gemm{};
bool g_core_ok = false, g_flash_ok = false, g_gemm_ok = false;

std::string own_dir() {
    Dl_info info;
    if (dladdr((void*)&own_dir, &info) && info.dli_fname) {
        std::string p(info.dli_fname);
        size_t slash = p.rfind('/');
        return slash == std::string::npos ? "." : p.substr(0, slash);
    }
    return ".";
}

void* open_library(const std::string& name) {
    auto it = g_handles.find(name);
    if (it != g_handles.end()) return it->second;
    std::string dir = g_lib_dir;
    if (dir.empty()) {
        const char* e = getenv("PURHIE_B200_LIB_DIR");
        dir = (e && *e) ? e : own_dir();
    }
    std::string path = dir + "/libpurhie_" + name + ".so";
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h)
        throw KernelError("the '" + name + "' kernel library is missing (" + std::string(dlerror() ? dlerror() : path) +
                          "); build it with `python -m purhie_b200.csrc.build " + name +
                          "`. There is no other implementation of these kernels.");
    g_handles[name] = h;
    return h;
}

template <typename F> void bind(void* h, const std::string& lib, const char* sym, F& out) {
    void* p = dlsym(h, sym);
    if (!p) throw KernelError("libpurhie_" + lib + ".so does not export " + sym + " (stale build?)");
    out = reinterpret_cast<F>(p);
}
}  // namespace

void set_library_dir(const std::string& dir) {
    std::lock_guard<std::mutex> lock(g_lib_mutex);
    g_lib_dir = dir;
}
std::string library_dir() {
    std::lock_guard<std::mutex> lock(g_lib_mutex);
    if (!g_lib_dir.empty()) return g_lib_dir;
    const char* e = getenv("PURHIE_B200_LIB_DIR");
    return (e && *e) ? e : own_dir();
}

const CoreKernels& core_kernels() {
    if (g_core_ok) return g_core;
    std::lock_guard<std::mutex> lock(g_lib_mutex);
    if (g_core_ok) return g_core;
    void* h = open_library("core");
    bind(h, "core", "ph_embed_gather", g_core.embed_gather);
    bind(h, "core", "ph_add_rmsnorm", g_core.add_rmsnorm);
    bind(h, "core", "ph_swiglu", g_core.swiglu);
    bind(h, "core", "ph_cast", g_core.cast);
    bind(h, "core", "ph_qk_norm_rope_kv_write", g_core.qk_norm_rope_kv_write);
    bind(h, "core", "ph_add_weight_sumsq", g_core.add_weight_sumsq);
    bind(h, "core", "ph_attention_generic", g_core.attention_generic);
    bind(h, "core", "ph_gemm_simple", g_core.gemm_simple);
    bind(h, "core", "ph_argmax_parts", g_core.argmax);
    bind(h, "core", "ph_argmax_scratch_bytes", g_core.argmax_scratch_bytes);
    bind(h, "core", "ph_sample_temperature", g_core.sample_temperature);
    bind(h, "core", "ph_sample_chain", g_core.sample_chain);
    bind(h, "core", "ph_sample_chain_max_k", g_core.sample_chain_max_k);
    bind(h, "core", "ph_random_fill", g_core.random_fill);
    bind(h, "core", "ph_core_last_error", g_core.last_error);
    g_core_ok = true;
    return g_core;
}

const FlashKernels& flash_kernels() {
    if (g_flash_ok) return g_flash;
    std::lock_guard<std::mutex> lock(g_lib_mutex);
    if (g_flash_ok) return g_flash;
    void* h = open_library("flash");
    bind(h, "flash", "ph_attention_prefill", g_flash.prefill);
    bind(h, "flash", "ph_attention_decode", g_flash.decode);
    bind(h, "flash", "ph_attention_decode_bulk", g_flash.decode_bulk);
    bind(h, "flash", "ph_attention_prefill_tc5", g_flash.prefill_tc5);
    bind(h, "flash", "ph_flash_last_error", g_flash.last_error);
    g_flash_ok = true;
    return g_flash;
}

const GemmKernels& gemm_kernels() {
    if (g_gemm_ok) return g_gemm;
    std::lock_guard<std::mutex> lock(g_lib_mutex);
    if (g_gemm_ok) return g_gemm;
    void* h = open_library("gemm100");
    bind(h, "gemm100", "ph_gemm_bf16_tcgen05", g_gemm.gemm);
    bind(h, "gemm100", "ph_gemm_bf16_tcgen05_pair", g_gemm.gemm_pair);
    bind(h, "gemm100", "ph_gemm100_last_error", g_gemm.last_error);
    g_gemm_ok = true;
    return g_gemm;
}

void require_library(const std::string& name) {
    if (name == "core") core_kernels();
    else if (name == "flash") flash_kernels();
    else if (name == "gemm100") gemm_kernels();
    else {
        std::lock_guard<std::mutex> lock(g_lib_mutex);
        open_library(name);
    }
}

// ---- time per kernel class ----------------------------------------------------------------------------------------
LaunchProfile::LaunchProfile() {
    const char* e = getenv("PURHIE_PROFILE");
    enabled_ = e && *e && *e != '0';
}
LaunchProfile& LaunchProfile::get() {
    static LaunchProfile p;
    return p;
}
std::string LaunchProfile::launcher_name(const char* call_text) {
    // "k.add_rmsnorm(stream.x, ...)" -> "add_rmsnorm"
    std::string name(call_text);
    size_t paren = name.find('(');
    if (paren != std::string::npos) name.resize(paren);
    size_t dot = name.rfind('.');
    if (dot != std::string::npos) name = name.substr(dot + 1);
    return name;
}
void LaunchProfile::leave_out(const char* names) {
    left_out_.clear();
    std::string all(names ? names : "");
    size_t at = 0;
    while (at <= all.size()) {
        size_t comma = all.find(',', at);
        if (comma == std::string::npos) comma = all.size();
        if (comma > at) left_out_.push_back(all.substr(at, comma - at));
        at = comma + 1;
    }
}
bool LaunchProfile::is_left_out(const char* call_text) const {
    const std::string name = launcher_name(call_text);
    for (const std::string& n : left_out_)
        if (n == name) return true;
    return false;
}
void LaunchProfile::begin(const char* call_text) {
    Record r;
    r.name = launcher_name(call_text);
    r.bytes = pending_bytes_; r.flops = pending_flops_;
    pending_bytes_ = pending_flops_ = 0;
    if (spare_.empty()) {
        cudaEventCreate(&r.start);
        cudaEventCreate(&r.stop);
    } else {
        r.start = spare_.back().first; r.stop = spare_.back().second;
        spare_.pop_back();
    }
    cudaEventRecord(r.start, stream_);
    records_.push_back(r);
    if (records_.size() > 65536) fold();
}
void LaunchProfile::end() {
    if (!records_.empty()) cudaEventRecord(records_.back().stop, stream_);
}
void LaunchProfile::fold() {
    // waits on the events, not on the stream: the engine whose stream they were recorded on may be gone by now
    for (Record& r : records_) {
        float ms = 0;
        if (cudaEventSynchronize(r.stop) == cudaSuccess && cudaEventElapsedTime(&ms, r.start, r.stop) == cudaSuccess) {
            Sum& s = sums_[r.name];
            s.calls++; s.ms += ms; s.bytes += r.bytes; s.flops += r.flops;
        }
        spare_.emplace_back(r.start, r.stop);
    }
    records_.clear();
}
std::string LaunchProfile::report_json(bool reset) {
    fold();
    std::string out = "{";
    bool first = true;
    for (const auto& kv : sums_) {
        char buf[256];
        snprintf(buf, sizeof buf, "%s\"%s\": {\"calls\": %lld, \"ms\": %.6f, \"bytes\": %.0f, \"flops\": %.0f}", first ? "" : ", ",
                 kv.first.c_str(), kv.second.calls, kv.second.ms, kv.second.bytes, kv.second.flops);
        out += buf;
        first = false;
    }
    out += "}";
    if (reset) sums_.clear();
    return out;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    QE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) QE_CUDA(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
    return cached[dev];
}

}  // namespace qe
