// Allocation-free entry point of the kernel library.  (This entry point has no counterpart in the reference engine.)
//
// Who needs it: code that drives the kernels from a place where it must not, or cannot, obtain device memory — a
// plugin running inside another runtime that owns the allocator, a real-time control loop with a no-allocation rule,
// a host whose memory pool is already handed out in full.  Such callers can still own their inputs and outputs, but
// the split-K decode attention kernel also wants scratch space for per-split partial results; this variant brings its
// own, a fixed array compiled into the library image.
//
//   atlas_attn_decode_noalloc(...)   same computation and arguments as atlas_attn_decode for sequences [0, B), except
//                                    that it takes no scratch pointers.
//
// Contract
//   * Calls no cudaMalloc / cudaFree and no allocating library routine.
//   * Limit: B * Hq * num_splits * (D + 2) floats must fit in ATLAS_NOALLOC_DECODE_SCRATCH_FLOATS (4 Mi floats =
//     16 MiB; e.g. 128 sequences x 32 heads x 7 splits at D = 128).  Larger requests return ATLAS_NOALLOC_ERR_TOO_LARGE
//     and launch nothing.  Every GPU that loads the library holds the 16 MiB until the process exits.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current) and remembers it.  Make that first call outside any CUDA stream capture, and from one host thread:
//     the remembered address is written without a lock, so two threads must not race on a device's first call.
//   * All calls on a device share the one array and it keeps the previous call's contents.  Nothing in it needs
//     zeroing (each launch rewrites every entry it later reads), but two calls that overlap on the GPU — different
//     streams, or graphs replayed concurrently — race on it.  Serialise them.
#pragma once
#include <stdint.h>

#define ATLAS_NOALLOC_DECODE_SCRATCH_FLOATS (4 * 1024 * 1024)
#define ATLAS_NOALLOC_ERR_TOO_LARGE (-100)
#define ATLAS_NOALLOC_ERR_DEVICE (-101)
#define ATLAS_NOALLOC_ERR_SYMBOL (-102)

#ifdef __cplusplus
extern "C" {
#endif

int atlas_attn_decode_noalloc(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                              const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                              const int* query_start_loc, int B, float scale, float k_scale, float v_scale, int Hq,
                              int Hkv, int D, int block_size, int window, int num_splits, unsigned long long* status,
                              void* stream);

#ifdef __cplusplus
}
#endif
