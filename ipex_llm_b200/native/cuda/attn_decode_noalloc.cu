// Decode attention with its work buffers in a fixed array of the library image: see attn_decode_noalloc.h for who
// needs this, the limits, the set-up rule and the sharing rule.  The attention kernel itself is the one behind
// ipex_attn_decode() (attn_decode.cu); this file only supplies the two work buffers and performs no allocation.
#include <cuda_runtime.h>

#include <mutex>

#include "attn_decode_noalloc.h"
#include "common/utils.cuh"

extern "C" {
int64_t ipex_attn_decode_scratch_floats(int B, int Hkv, int G, int Sq, int D, int nsplit);
int64_t ipex_attn_decode_counter_ints(int B, int Hkv, int G, int Sq);
int ipex_attn_decode(const void* q, const void* knew, const void* vnew, void* kcache, void* vcache, void* out,
                     const int* past_len, int past_scalar, const float* cosp, const float* sinp, float* scratch,
                     int* counters, const int64_t* strides, int B, int Sq, int Hq, int Hkv, int D, int nsplit, int rope,
                     int R, int causal, int window, float scale, float softcap, int fp8_kv, int dtype, int pdl,
                     void* stream);
}

namespace {

constexpr int64_t kMaxFloats = 2ll * 1024 * 1024;  // 8 MiB of split partials
constexpr int64_t kMaxCounters = 4096;             // 16 KiB of tickets
constexpr size_t kCounterBytes = kMaxCounters * sizeof(int);
constexpr size_t kScratchBytes = kCounterBytes + kMaxFloats * sizeof(float);

// One copy per device that loads the library.  Tickets first, partials after them; 256-byte alignment keeps both
// parts aligned for the vector accesses of the kernel.  In host code this name is only a handle for
// cudaGetSymbolAddress, never an address to hand to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_dev_ptr[kMaxDevices] = {};  // device address of g_noalloc_scratch, per device ordinal

// Address of the array on the current device; looked up once per device, with that device current.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return IPEX_NOALLOC_E_DEVICE;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_dev_ptr[dev] == nullptr) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return (int)cudaErrorInvalidSymbol;
    g_dev_ptr[dev] = p;
  }
  *out = g_dev_ptr[dev];
  return 0;
}

}  // namespace

IPEX_API int64_t ipex_attn_decode_noalloc_max_floats(void) { return kMaxFloats; }
IPEX_API int64_t ipex_attn_decode_noalloc_max_counters(void) { return kMaxCounters; }

IPEX_API int ipex_attn_decode_noalloc_setup(void) {
  unsigned char* p = nullptr;
  return scratch_for_current_device(&p);
}

IPEX_API const char* ipex_attn_decode_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case IPEX_NOALLOC_E_SCRATCH:
      return "ipex_attn_decode_noalloc: the split partials for this shape exceed the built-in 2 Mi-float scratch; "
             "use fewer splits or ipex_attn_decode() with a caller-provided buffer";
    case IPEX_NOALLOC_E_COUNTERS:
      return "ipex_attn_decode_noalloc: batch x kv-heads x row-blocks exceeds the built-in 4096 tickets; "
             "use ipex_attn_decode() with a caller-provided buffer";
    case IPEX_NOALLOC_E_DEVICE: return "ipex_attn_decode_noalloc: device ordinal outside the library's table (64)";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "ipex_attn_decode_noalloc: unknown code";
  }
}

IPEX_API int ipex_attn_decode_noalloc(const void* q, const void* knew, const void* vnew, void* kcache, void* vcache,
                                      void* out, const int* past_len, int past_scalar, const float* cosp,
                                      const float* sinp, const int64_t* strides, int B, int Sq, int Hq, int Hkv, int D,
                                      int nsplit, int rope, int R, int causal, int window, float scale, float softcap,
                                      int fp8_kv, int dtype, int pdl, void* stream) {
  if (Hkv < 1 || Hq < 1 || Hq % Hkv != 0 || Sq < 1 || nsplit < 1 || B < 1) return (int)cudaErrorInvalidValue;
  const int G = Hq / Hkv;
  // With a single split every CTA writes its result straight to `out` and never reads or writes the partials or
  // the tickets, so such a launch needs nothing from the array and no limit applies to it.
  const int64_t need_f = nsplit == 1 ? 0 : ipex_attn_decode_scratch_floats(B, Hkv, G, Sq, D, nsplit);
  const int64_t need_c = nsplit == 1 ? 0 : ipex_attn_decode_counter_ints(B, Hkv, G, Sq);
  // Tickets first: one ticket stands for at least 16 * 2 * (D + 2) floats of partials, so a launch that is over
  // the ticket limit is over the float limit as well, and the more specific code is the useful one.
  if (need_c > kMaxCounters) return IPEX_NOALLOC_E_COUNTERS;
  if (need_f > kMaxFloats) return IPEX_NOALLOC_E_SCRATCH;
  unsigned char* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc != 0) return rc;
  int* counters = reinterpret_cast<int*>(base);
  float* partials = reinterpret_cast<float*>(base + kCounterBytes);
  // Tickets must be zero when the kernel starts.  A completed launch leaves them zero, but the array is shared with
  // every other caller on the device, so clear the part this launch uses on the caller's stream instead of relying
  // on what an earlier call left behind.
  if (need_c > 0) {
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)need_c * sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
  }
  return ipex_attn_decode(q, knew, vnew, kcache, vcache, out, past_len, past_scalar, cosp, sinp, partials, counters,
                          strides, B, Sq, Hq, Hkv, D, nsplit, rope, R, causal, window, scale, softcap, fp8_kv, dtype,
                          pdl, stream);
}
