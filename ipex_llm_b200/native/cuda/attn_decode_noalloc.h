// Split-KV decode attention through a fixed, library-owned scratch area.
//
// This entry point has no counterpart in the reference project: it exists only in this library.
//
// ipex_attn_decode() asks its caller for two work buffers (split partials and ticket counters).  Callers that come
// through PyTorch take them from the caching allocator.  Some callers cannot do that:
//   * a C or C++ serving host that links this library directly and has no tensor allocator at all;
//   * a process that sized its KV pool to fill the device and must not ask the driver for more memory while it
//     serves, because a device allocation can fail there, or stall every stream of the device while it runs;
//   * code on a latency-critical path where the cost of an allocator call (a lock, maybe a device synchronise when
//     the pool has to grow) is not acceptable.
// For them the work buffers live in one array that is part of the library image on every device.  The call performs
// no device or host allocation: no cudaMalloc / cudaFree family call, no allocating library routine, no torch.
//
// Limits (fixed at build time, also returned by the two *_max_* functions):
//   partials : ipex_attn_decode_scratch_floats(...) <= 2 * 1024 * 1024 floats (8 MiB)
//   tickets  : ipex_attn_decode_counter_ints(...)   <= 4096 ints
// A launch that needs more is refused with IPEX_NOALLOC_E_COUNTERS (checked first) or IPEX_NOALLOC_E_SCRATCH and
// nothing is launched.  A single-split launch (nsplit == 1) writes its result directly, uses neither area and is
// therefore never refused for size.
//
// Set-up: the first call on each device looks up the device address of the array (cudaGetSymbolAddress with that
// device current).  Make that first call (or call ipex_attn_decode_noalloc_setup()) during start-up, before any
// stream capture is begun on that device.  Later calls on the device only read the stored address.
//
// Sharing: every call on a device uses the same array.  The ticket area is cleared on the caller's stream ahead of
// each launch, so a call never sees tickets left by an earlier one; the partials need no clearing.  Two calls whose
// kernels can overlap in time (different streams without an ordering between them, or several host threads
// launching on different streams) race on the array and give wrong results: order them on one stream or with events.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define IPEX_NOALLOC_EXPORT __attribute__((visibility("default")))
#else
#define IPEX_NOALLOC_EXPORT
#endif

#define IPEX_NOALLOC_E_SCRATCH (-1)   // partial-result area needed exceeds the built-in maximum
#define IPEX_NOALLOC_E_COUNTERS (-2)  // ticket area needed exceeds the built-in maximum
#define IPEX_NOALLOC_E_DEVICE (-3)    // device ordinal outside the table kept by the library

IPEX_NOALLOC_EXPORT int64_t ipex_attn_decode_noalloc_max_floats(void);
IPEX_NOALLOC_EXPORT int64_t ipex_attn_decode_noalloc_max_counters(void);

// Looks up the scratch address for the current device.  Returns 0, a cudaError_t (> 0) or IPEX_NOALLOC_E_DEVICE.
IPEX_NOALLOC_EXPORT int ipex_attn_decode_noalloc_setup(void);

// Human-readable text for a return value of the functions in this header.
IPEX_NOALLOC_EXPORT const char* ipex_attn_decode_noalloc_strerror(int code);

// Same arguments and semantics as ipex_attn_decode() minus `scratch` and `counters`.
// Returns 0 on success, a cudaError_t (> 0) from set-up or launch, or one of the IPEX_NOALLOC_E_* codes (< 0).
IPEX_NOALLOC_EXPORT int ipex_attn_decode_noalloc(const void* q, const void* knew, const void* vnew, void* kcache, void* vcache, void* out,
                             const int* past_len, int past_scalar, const float* cosp, const float* sinp,
                             const int64_t* strides /*12*/, int B, int Sq, int Hq, int Hkv, int D, int nsplit, int rope,
                             int R, int causal, int window, float scale, float softcap, int fp8_kv, int dtype, int pdl,
                             void* stream);

#ifdef __cplusplus
}
#endif
