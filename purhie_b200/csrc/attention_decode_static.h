// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (aardbeiplantje/PURHIE); it exists for this library's
// own users.  ph_attention_decode (attention_flash.cu) splits the keys of every token over several CTAs and
// needs scratch memory for the per-split partial results, which its caller has to allocate and pass in.  Some
// callers cannot do that:
//   * a server that has already handed every free byte of the GPU to its cache pool and must not grow,
//   * a host that links only these C symbols and has no allocator of its own to borrow scratch from
//     (no torch, no pool),
//   * code on a latency path where cudaMalloc / cudaFree are unacceptable because they synchronise the device.
// For them ph_attention_decode_static does the same work with the scratch taken from one fixed array that
// is part of the library image.  It calls no cudaMalloc, no cudaFree and no allocating library routine.
//
// The price and the rules:
//   * The array is PH_DECODE_STATIC_SCRATCH_BYTES (16 MiB) of device memory on EVERY GPU that loads the
//     library, held until the process exits, whether or not the entry point is ever called.
//   * A call with splits > 1 needs n_rows * HQ * splits * (D + 2) floats of it; a call that needs more is refused
//     with PH_ERR_UNSUPPORTED and a message that names both numbers (nothing is launched).  With splits == 1 the
//     kernel writes its result directly, no scratch is touched and no size is refused.
//   * The library exports these two symbols only; the kernels it shares with libpurhie_flash are private copies, so
//     a host may link both libraries.
//   * All calls share the array and it keeps what the last call left there.  Nothing in it has to start at
//     zero: every slot a call reads was written by that same call first.  Two calls whose kernels may run at
//     the same time on one GPU (different streams, different threads) race on the array; issue them on one
//     stream or order them yourself.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with that
//     device current) and remembers it.  Make that first call before any stream capture begins on the
//     device; later calls only launch kernels.
//
// Arguments and result are those of ph_attention_decode without the two scratch pointers; the output is the
// same (the same kernels run).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define PH_DECODE_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

// q [rows, HQ, D] bfloat16; k_base / v_base: K and V of page 0 of one cache entry, pages page_stride elements
// apart, a page laid out [kv head][token][D]; block_table [segments, table_stride]; row_list: the rows to
// process (NULL: rows 0 .. n_rows - 1); row_seg, positions: per row; out [rows, HQ * D] bfloat16.
// Returns 0, or a non-zero status with the text in ph_decode_static_last_error().
int ph_attention_decode_static(const void* q, const void* k_base, const void* v_base, long long page_stride,
                               int page_size, const int32_t* block_table, int table_stride, const int32_t* row_list,
                               int n_rows, const int32_t* row_seg, const int32_t* positions, void* out, int HQ,
                               int HKV, int D, int splits, int window, float scale, cudaStream_t stream);

const char* ph_decode_static_last_error(void);

#ifdef __cplusplus
}
#endif
