// Shared device/host helpers for the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define IPEX_API extern "C" __attribute__((visibility("default")))

// activation dtype codes used across the C ABI
enum { DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2 };

// weight families of the tiled device layouts (see native/host/quant_core.cpp)
enum {
  WF_SYM_INT4 = 0,   // magic nibble order, value = (q - 8) * d
  WF_ASYM_INT4 = 1,  // magic nibble order, value = q * d + m
  WF_LUT4 = 2,       // natural nibble order, value = lut[q] * d   (nf4, fp4)
  WF_FP8_E4M3 = 3,   // bytes, fp32 scale per 128
  WF_FP8_E5M2 = 4,
  WF_INT8 = 5,       // bytes, fp16 scale per 64
  WF_F16 = 6,        // plain row-major half weights [N, K]
  WF_BF16 = 7,
};

__host__ __device__ inline int64_t ceil_to_i64(int64_t a, int64_t b) { return (a + b - 1) / b * b; }
__host__ __device__ inline int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

template <typename T> struct DT;
template <> struct DT<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct DT<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct DT<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start
// while its predecessor in the stream is still running.  pdl_wait() blocks until the predecessor has
// completed and its writes are visible; everything before it may only touch data the predecessor never
// writes (weights).  pdl_launch_dependents() lets the successor start its own weight prefetch early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// L2 prefetch of a contiguous range (16-byte aligned address, size a multiple of 16 bytes).
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_nc_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Host-side launch helper: plain launch or programmatic-dependent launch on `stream`.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
