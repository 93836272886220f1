// ph_attention_decode_static: split-key decode attention with its scratch in a fixed device array instead of
// caller-allocated memory.  See attention_decode_static.h for who needs it and what it costs.
//
// The kernels are the ones of attention_flash.cu, compiled into this library a second time by including that
// file; only the source of the scratch differs.  That file's own entry points stay inside this library (hidden),
// so that a host which links both libraries meets every symbol once.
#define PH_EXPORT extern "C" __attribute__((visibility("hidden")))
#include "attention_flash.cu"
#undef PH_EXPORT
#define PH_EXPORT extern "C" __attribute__((visibility("default")))

#include "attention_decode_static.h"

// The scratch itself: part of the library image, present on every GPU that loads the library.
static __device__ __align__(256) float g_decode_scratch[PH_DECODE_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};

// In host code `g_decode_scratch` is only a handle for the symbol, not an address a kernel can use.  The
// device address is asked for once per device, with that device current.
int scratch_for_current_device(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return ph::fail(PH_ERR_LAUNCH, "attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return ph::fail(PH_ERR_UNSUPPORTED, "attention_decode_static: device %d is beyond %d", dev, MAX_DEVICES);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess || !p)
            return ph::fail(PH_ERR_LAUNCH, "attention_decode_static: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
        g_scratch_addr[dev] = (float*)p;
    }
    *out = g_scratch_addr[dev];
    return PH_OK;
}

}  // namespace

PH_DEFINE_LAST_ERROR(ph_decode_static)

PH_EXPORT int ph_attention_decode_static(const void* q, const void* k_base, const void* v_base, long long page_stride,
                                         int page_size, const int32_t* block_table, int table_stride,
                                         const int32_t* row_list, int n_rows, const int32_t* row_seg,
                                         const int32_t* positions, void* out, int HQ, int HKV, int D, int splits,
                                         int window, float scale, cudaStream_t stream) {
    if (n_rows < 0 || HQ < 1 || splits < 1 || D < 1)
        return ph::fail(PH_ERR_ARG, "attention_decode_static: bad arguments (rows %d, HQ %d, D %d, splits %d)", n_rows, HQ, D, splits);
    // part_o [rows][HQ][splits][D] followed by part_ml [rows][HQ][splits][2]; with the keys in one piece the
    // kernel writes its result directly and touches no scratch, so nothing is needed and nothing is refused
    const unsigned long long slots = (unsigned long long)n_rows * HQ * splits;
    const unsigned long long need = splits > 1 ? slots * (unsigned long long)(D + 2) * sizeof(float) : 0;
    if (need > PH_DECODE_STATIC_SCRATCH_BYTES)
        return ph::fail(PH_ERR_UNSUPPORTED,
                        "attention_decode_static: %d rows x %d heads x %d splits x head size %d need %llu bytes of scratch, "
                        "the fixed array holds %u; use fewer splits or rows, or ph_attention_decode with scratch of your own",
                        n_rows, HQ, splits, D, need, PH_DECODE_STATIC_SCRATCH_BYTES);
    float* scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;
    float* part_o = scratch;
    float* part_ml = scratch + slots * (unsigned long long)D;        // D is a multiple of 16: stays 8-byte aligned
    return ph_attention_decode(q, k_base, v_base, page_stride, page_size, block_table, table_stride, row_list, n_rows,
                               row_seg, positions, part_o, part_ml, out, HQ, HKV, D, splits, window, scale, stream);
}
