// The interfaces of the parts a model is made of, the data that describes a model, and what a step hands to
// the parts.  This header is the whole contract between the framework and a part: a part defined elsewhere (a
// plugin library, a test) includes it, derives from one of the families below and registers a factory.
//
// A model is data (ModelSpec): an embedding, a list of layers, the order in which layers run, a final norm and
// a head.  A layer (LayerSpec) names an arrangement and gives it named sub-parts, each a PartSpec {kind,
// params}; the generic decoder looks every kind up in the registries and builds the part from its params
// alone, so a part gets every size and constant as a parameter and never knows which model it is in.  Tensor
// names are parameters too: params["names"] maps the part's role names to checkpoint names.  The run order is a
// list of LayerCall, which may name a layer twice or let a call read the cache an earlier call wrote.
//
// The reference expresses per-layer variety with a LayerKind enum and per-layer weight records
// (src/inference_internal.h:45-52, 77-90) and runs layers in file order (src/qwen_model.cpp:1196-1279).
//
// Families and what each must provide:
//   Norm              forward(stream, ctx, rows, n_rows): fold the stream's pending addend into the float32
//                     residual, return the normalised rows (all, or the gathered `rows`) in the compute dtype.
//   PositionEncoding  what a mixer needs to place a token: for the rotary family a table of cosines and sines
//                     per position and pair, the number of rotated dimensions, the pairing, and which of the
//                     step's position columns it reads.
//   Mixer             cache_need() tells the cache manager what to keep for it; forward(x, ctx, cache) mixes the
//                     tokens of each request; prepare_step(plan) may add metadata of its own to the step.
//   FeedForward       forward(x, ctx): [T, E] -> [T, E] row by row (routing, if any, lives inside it).
//   Arrangement       strings a layer's sub-parts together.
//   Embedding, Head   token ids -> float32 residual; normed rows -> float32 logits.
// A mixer or feed-forward returns an Addend (a tensor to be added to the residual, possibly as split-K partial
// sums), or an empty one when it has already added its result into ctx.residual.
#pragma once

#include <cuda_runtime.h>

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../host/common.h"
#include "../host/device.h"
#include "../host/json.h"

namespace qe {

// ---- tensors a part reads -------------------------------------------------------------------------------------
enum class Role { Matrix, Vector, Table };      // compute dtype | float32 always | int32
enum class Init { Normal, Scale };              // random weights: N(0, std) | U(low, high) around 1

struct TensorSpec {
    std::string name;
    std::vector<int64_t> shape;
    Role role = Role::Matrix;
    Init init = Init::Normal;
    bool operator==(const TensorSpec& o) const { return name == o.name && shape == o.shape && role == o.role && init == o.init; }
};
inline const char* role_name(Role r) { return r == Role::Matrix ? "matrix" : r == Role::Vector ? "vector" : "table"; }

// Where a part gets its tensors from while it binds: a checkpoint folder or the random generator.  fetch()
// returns the tensor on the device in the dtype the policy gives it (matrix: the compute dtype, except that a
// tensor stored in 32-bit stays 32-bit; vector: float32; table: int32).  The part owns what it keeps: tensors
// from fetch() stay alive as long as the model's arena; release() gives a temporary back early.
class QE_API WeightSource {
public:
    virtual ~WeightSource() = default;
    virtual Tensor fetch(const std::string& name) = 0;
    virtual DeviceArena& arena() = 0;
    virtual cudaStream_t stream() = 0;
    void release(const Tensor& t) { arena().release(t); }
};

// ---- what the cache manager keeps for one run-order entry ----------------------------------------------------
struct CacheNeed {
    enum Kind { None, Pages, State } kind = None;
    int kv_heads = 0, head_dim = 0;
    int value_dim = 0;                            // pages: width of a value row when it differs from a key row's (0: head_dim)
    int window = 0;                               // pages: 0 keeps all keys, W keeps the last W positions
    int v_dim() const { return value_dim > 0 ? value_dim : head_dim; }
    std::vector<int64_t> state_shape;             // state: shape of one request's state
    DType state_dtype = DType::F32;
    static CacheNeed pages(int kv_heads, int head_dim, int window = 0, int value_dim = 0) {
        if (window < 0) throw Error(kInvalidArg, "a window must hold at least one position");
        if (kv_heads < 1 || head_dim < 1 || value_dim < 0) throw Error(kInvalidArg, "a page holds at least one head of at least one element");
        CacheNeed n; n.kind = Pages; n.kv_heads = kv_heads; n.head_dim = head_dim; n.window = window;
        n.value_dim = value_dim == head_dim ? 0 : value_dim;
        return n;
    }
    static CacheNeed state(std::vector<int64_t> shape, DType dtype = DType::F32) {
        CacheNeed n; n.kind = State; n.state_shape = std::move(shape); n.state_dtype = dtype; return n;
    }
};

// ---- the description of a model ---------------------------------------------------------------------------------
struct PartSpec {
    std::string kind;
    Json params = Json::object();
    PartSpec() = default;
    PartSpec(std::string k, Json p) : kind(std::move(k)), params(std::move(p)) {}
    Json to_json() const { Json j = Json::object(); j.set("kind", kind); j.set("params", params); return j; }
    static PartSpec from_json(const Json& j) { return PartSpec(j.at("kind").as_string(), j.has("params") ? j.at("params") : Json::object()); }
};

struct LayerSpec {
    std::string arrangement = "pre_norm";
    std::vector<std::pair<std::string, PartSpec>> parts;          // sub-parts by the names the arrangement reads
    const PartSpec& part(const std::string& name) const {
        for (const auto& p : parts) if (p.first == name) return p.second;
        throw ConfigError("a layer of arrangement '" + arrangement + "' has no sub-part '" + name + "'");
    }
    bool has(const std::string& name) const { for (const auto& p : parts) if (p.first == name) return true; return false; }
};

struct LayerCall {
    int layer = 0;               // index into ModelSpec::layers
    int cache_from = -1;         // -1: a cache entry of its own; else the earlier call whose cache this one reads
};

struct ModelSpec {
    int64_t hidden_size = 0, vocab_size = 0, max_position = 0;
    int position_columns = 1;    // columns of positions a step carries per row (column 0: the index in the request)
    PartSpec embedding, final_norm, head;
    std::vector<LayerSpec> layers;
    std::vector<LayerCall> schedule;
    void validate() const;
};

// ---- what a step hands to the parts ------------------------------------------------------------------------------
struct GroupStep {
    const int32_t* block_table = nullptr;    // [S, table_width]: page of each logical block, -1 = given back
    int table_width = 0;
    const int32_t* slot_mapping = nullptr;   // [T]: page * page_size + offset where each row's k and v go
    int page_size = 0;
};

// The cache of one run-order entry, as its mixer sees it.
struct CacheView {
    CacheNeed::Kind kind = CacheNeed::None;
    int group = -1;
    void* k_base = nullptr;                  // K (V) of this entry in page 0; pages are page_stride elements apart
    void* v_base = nullptr;
    int kv_heads = 0, key_dim = 0, value_dim = 0;   // a page holds [kv_heads][page_size][key_dim] keys, then the values likewise
    DType kv_dtype = DType::F32;
    long long page_stride = 0;
    int page_size = 0;
    int num_pages = 0;
    bool writable = true;                    // false: another entry writes this cache, this one only reads
    Tensor state;                            // [max_requests, *state_shape]
};

struct Addend {
    Tensor tensor;                           // [T, E], or [splits, T, E] partial sums; undefined: already added
    int splits = 1;
    bool activated = false;                  // a product whose activation was applied in the kernel's epilogue
    Addend() : splits(0) {}
    Addend(Tensor t, int s = 1, bool act = false) : tensor(std::move(t)), splits(s), activated(act) {}
};

// A device array of int32 that a part added to the step's metadata (see StepPlan).
struct StepArray {
    const int32_t* data = nullptr;
    int count = 0;
};

// A normalisation whose factor per row has not been applied: the rows a norm hands out are (x * weight) and the row's
// factor is rsqrt(sum over the chunks of sumsq[row][chunk] / width + eps).  Only a consumer that said it applies the
// factor itself (takes_unscaled_rows) ever sees rows like that: a product is linear in its rows, so its epilogue (or
// whoever adds up its partial sums) can multiply by the factor, and the norm's kernel needs no sum over a whole row,
// which lets few rows be spread over many CTAs.
struct RowScale {
    const float* sumsq = nullptr;            // [rows, chunks] float32 on the device
    int chunks = 0, width = 0;
    float eps = 0.0f;
    bool defined() const { return sumsq != nullptr; }
};

// The norm that follows a part's addition into the residual, offered to the part's last product.  A product that adds
// into the residual in its own epilogue may do that norm's pass over the rows there as well: the weighted, unscaled
// rows in bfloat16 and their sums of squares (RowScale).  The norm then finds them in the stream and launches nothing.
// Offering costs nothing and binds nobody: a product that cannot do it leaves `rows` undefined.
struct NormAhead {
    const float* weight = nullptr;           // offered: [width] float32 on the device (null: nothing offered)
    const void* norm = nullptr;              // the Norm that made the offer and may pick the rows up
    int width = 0;
    float eps = 0.0f;
    Tensor rows;                             // done: [T, width] bfloat16, (x + addend) * weight
    RowScale scale;                          // done: the factor the rows lack
    bool offered() const { return weight != nullptr; }
    bool done() const { return rows.defined(); }
};

struct StepContext {
    int T = 0, S = 0;
    const int32_t* token_ids = nullptr;      // [T]
    const int32_t* positions = nullptr;      // [position_columns, T]; column 0: absolute position in the request
    int position_columns = 1;
    const int32_t* row_seg = nullptr;        // [T] segment of each row
    const int32_t* seg_start = nullptr;      // [S + 1] first row of each segment
    const int32_t* seg_ctx_len = nullptr;    // [S] tokens of the request once this step is done
    const int32_t* seg_slot = nullptr;       // [S] state slot of each segment's request
    std::vector<int> q_lens, ctx_lens, slots;   // host copies, for launch decisions
    std::vector<GroupStep> groups;
    Workspace* workspace = nullptr;
    DType compute_dtype = DType::F32;
    cudaStream_t stream = nullptr;
    bool decode_only = false;
    const int32_t* decode_rows = nullptr;    // rows of single-token segments (null when every row is one)
    int n_decode_rows = 0;
    int decode_max_ctx = 0;                  // how far back the decode rows look, as the power of two that holds it
    int prefill_max_ctx = 0;                 // the same for the prompt portions
    float* residual = nullptr;               // the float32 residual [T, E] an addend will be added to
    int64_t residual_width = 0;
    int* gemm_error = nullptr;               // device words where kernels with bounded waits report giving up
    int* attention_error = nullptr;
    RowScale row_scale;                      // set by an arrangement around a consumer that takes unscaled rows, else undefined
    NormAhead norm_ahead;                    // set by an arrangement around a part: the norm after the part's addition
    NormAhead next_layer_norm;               // set by the model around a layer: the first norm of the layer that runs next
    std::map<std::string, StepArray> arrays; // what parts added through StepPlan, by name
    const Json* options = nullptr;           // kernel choices for tests ("decode_kernel": "cp_async", ...)

    const int32_t* position_column(int c) const { return positions + (size_t)c * T; }
    StepArray array(const std::string& name) const {
        auto it = arrays.find(name);
        return it == arrays.end() ? StepArray() : it->second;
    }
    std::string option(const std::string& key) const { return options ? options->get_string(key, "") : std::string(); }
    long long option_int(const std::string& key) const { return options ? options->get_int(key, 0) : 0; }
};

// The step as the host lays it out, before anything is uploaded: a part's prepare_step() reads the segments and
// may add int32 arrays of its own (query tiles for its kernel, say), which travel to the device in the step's one
// metadata copy and come back in StepContext::arrays.  Parts that share a need share a name: the first to ask
// adds the array, the others find it there.
struct StepPlan {
    int T = 0, S = 0;
    std::vector<int> q_lens, ctx_lens, starts;      // per segment: new tokens, tokens afterwards, first new position
    std::vector<int> slots;                         // per segment: the state slot of its request
    std::vector<std::pair<std::string, std::vector<int32_t>>> arrays;
    bool has(const std::string& name) const { for (const auto& a : arrays) if (a.first == name) return true; return false; }
    void add(const std::string& name, std::vector<int32_t> values) { arrays.emplace_back(name, std::move(values)); }
};

// The float32 residual [T, E] plus an addend that the next norm folds in (x += addend, then norm), so that the
// sum and the normalisation are one pass over the row.
struct ResidualStream {
    Tensor x;
    Addend pending;
    bool has_pending = false;
    NormAhead prepared;                      // rows that the last product left for the norm that comes next (x is complete)
    void add(Addend a) {
        if (has_pending) throw Error(kInvalidState, "the residual stream already has a pending addend");
        prepared = NormAhead();
        if (a.tensor.defined()) { pending = std::move(a); has_pending = true; }   // undefined: the part added into x itself
    }
    // after add(): what the part's last product did for the norm ahead (nothing, if it did nothing)
    void prepare(const NormAhead& ahead) { prepared = (!has_pending && ahead.done()) ? ahead : NormAhead(); }
    void clear() { has_pending = false; pending = Addend(); prepared = NormAhead(); }
};

// ---- building ---------------------------------------------------------------------------------------------------
class Part;
class PositionEncoding;

class QE_API BuildContext {
public:
    explicit BuildContext(DType compute = DType::F32, Json options = Json::object()) : compute_dtype(compute), options(std::move(options)) {}
    DType compute_dtype;
    Json options;                            // "gemm": auto|tcgen05|simple, "attention": auto|flash|generic
    // parts that several owners share (one rotary table for all layers): made once per key
    std::shared_ptr<Part> shared(const std::string& key, const std::function<std::shared_ptr<Part>()>& make);
private:
    std::map<std::string, std::shared_ptr<Part>> shared_;
};

// ---- the families ---------------------------------------------------------------------------------------------------
class QE_API Part {
public:
    Part(const Json& params, BuildContext& build);
    virtual ~Part() = default;
    virtual std::vector<TensorSpec> tensor_specs() const { return {}; }     // tensors this part reads
    virtual std::vector<std::string> ignored_tensors() const { return {}; } // may be present, are not read
    virtual void bind(WeightSource& src) {}                                  // fetch tensors, prepare derived buffers
    virtual std::vector<std::string> required_libraries() const { return {"core"}; }
    virtual int preferred_row_multiple() const { return 0; }                 // a step's rows are cheapest in multiples of this
    virtual void prepare_step(StepPlan& plan) {}                             // host side, once per step and part
    virtual std::vector<Part*> children() { return {}; }                     // parts inside this one (a shared position encoding)
    const std::string& name_of(const std::string& role) const;               // checkpoint name of a role
    Json params;
    DType compute_dtype;
protected:
    std::map<std::string, std::string> names_;
};

class QE_API Norm : public Part {
public:
    using Part::Part;
    // rows == nullptr: all T rows, and the pending addend is folded into the stream for good; else the n_rows
    // gathered rows (the stream keeps its pending addend).
    virtual Tensor forward(ResidualStream& stream, StepContext& ctx, const int32_t* rows = nullptr, int n_rows = 0) = 0;
    // As forward() over all rows, for a consumer that applies the row's factor itself: a norm that can leave the
    // factor out returns the weighted, unscaled rows and describes the factor in *scale; one that cannot returns what
    // forward() returns and leaves *scale undefined.
    virtual Tensor forward_unscaled(ResidualStream& stream, StepContext& ctx, RowScale* scale) {
        *scale = RowScale();
        return forward(stream, ctx);
    }
    // What a product in front may do of this norm's work (NormAhead), if forward_unscaled() would pick it up from
    // stream.prepared; a norm that has no such form offers nothing.
    virtual NormAhead offer(const StepContext&) const { return NormAhead(); }
};

class QE_API PositionEncoding : public Part {
public:
    using Part::Part;
    virtual int n_rot() const = 0;                       // rotated dimensions of a head (0: none)
    virtual bool interleaved() const { return false; }   // pairs (2i, 2i+1) instead of (i, i + n_rot/2)
    virtual int position_column() const { return 0; }    // which of the step's position columns it reads
    // float32 [max_position, n_rot] on the device: per position n_rot/2 cosines then n_rot/2 sines (frequency
    // factors and scalings are folded into the angles); undefined: no rotation.
    virtual Tensor rotation_table() = 0;
};

class QE_API Mixer : public Part {
public:
    using Part::Part;
    virtual CacheNeed cache_need() const { return CacheNeed(); }
    // x [T, E] in the compute dtype (already normed); rows of one request arrive in order.
    virtual Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) = 0;
    // True: in this step the mixer applies ctx.row_scale to what its first product gives, so the norm in front may
    // leave the row's factor out (see RowScale).  A mixer that says nothing always gets finished rows.
    virtual bool takes_unscaled_rows(const StepContext&) const { return false; }
};

class QE_API FeedForward : public Part {
public:
    using Part::Part;
    virtual Addend forward(const Tensor& x, StepContext& ctx) = 0;
    virtual bool takes_unscaled_rows(const StepContext&) const { return false; }     // as Mixer's
};

class QE_API Embedding : public Part {
public:
    using Part::Part;
    virtual Tensor forward(StepContext& ctx) = 0;        // float32 [T, E]
};

class QE_API Head : public Part {
public:
    using Part::Part;
    virtual Tensor forward(const Tensor& xn, StepContext& ctx, int n_rows) = 0;   // float32 [n_rows, vocab]
};

class QE_API Arrangement {
public:
    virtual ~Arrangement() = default;
    virtual std::vector<Part*> parts() = 0;
    virtual CacheNeed cache_need() const = 0;            // of the layer's mixer
    virtual void forward(ResidualStream& stream, StepContext& ctx, const CacheView& cache) = 0;
    // The offer of the layer's first norm, if in this step it would take rows prepared by the layer in front (the
    // model hands it to that layer as ctx.next_layer_norm).
    virtual NormAhead first_norm(const StepContext&) const { return NormAhead(); }
};

// ---- registries -------------------------------------------------------------------------------------------------------
using PartFactory = std::function<std::shared_ptr<Part>(const Json& params, BuildContext& build)>;
using ArrangementFactory = std::function<std::unique_ptr<Arrangement>(const LayerSpec& layer, BuildContext& build)>;

// family: "norm", "position", "mixer", "feed_forward", "embedding", "head".  Registering a kind twice replaces it.
QE_API void register_part(const std::string& family, const std::string& kind, PartFactory factory);
QE_API void unregister_part(const std::string& family, const std::string& kind);
QE_API std::shared_ptr<Part> make_part(const std::string& family, const PartSpec& spec, BuildContext& build);
QE_API void register_arrangement(const std::string& kind, ArrangementFactory factory);
QE_API void unregister_arrangement(const std::string& kind);
QE_API std::unique_ptr<Arrangement> make_arrangement(const LayerSpec& layer, BuildContext& build);
QE_API std::vector<std::string> registered_parts(const std::string& family);

template <typename T> std::shared_ptr<T> make_part_as(const std::string& family, const PartSpec& spec, BuildContext& build) {
    auto p = std::dynamic_pointer_cast<T>(make_part(family, spec, build));
    if (!p) throw ConfigError("part '" + spec.kind + "' is not of the '" + family + "' family");
    return p;
}

// Registers the parts this library brings (rmsnorm, rope_neox, attention, swiglu, embedding, lm_head, pre_norm).
QE_API void register_builtin_parts();

}  // namespace qe
