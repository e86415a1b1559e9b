// Collectives over NVLink peer memory for tensor parallelism (single node, every GPU maps every peer's buffer).
//
// The reference's tensor parallelism ends every row-parallel linear with an all-reduce issued through oneCCL /
// deepspeed.comm (python/llm/src/ipex_llm/transformers/low_bit_linear.py:675-682, 708-712, 752-759).  Decode
// messages are tiny ([B, hidden] = 16-512 KB) and there are two per layer, so what matters is latency: these
// kernels use plain peer loads/stores on symmetric buffers plus one arrival counter per block, no ring, no
// staging copy on a second stream.  (The GEMV fused with its all-reduce lives in gemv_tma.cu; these are the
// stand-alone building blocks for the module path, prefill and tests.)
//
// Protocol shared by the kernels ("parity" = which of two buffer sets a call uses; consecutive calls alternate,
// so a rank that runs ahead can never touch the set a slow peer is still reading):
//   signal : red.release.sys.add  peer_counter[block] += 1      (after this rank's data is in place)
//   wait   : ld.acquire.sys until own_counter[block] == world   (bounded; *err = code on expiry)
//   reset  : own_counter[block] = 0                             (self-cleaning, next use is two calls away)
#include "common/utils.cuh"

namespace {

constexpr int kCommSpin = 1 << 22;

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// cross-rank rendezvous of block `b`; returns false on expiry (thread 0 decides, result broadcast via smem)
__device__ bool block_rendezvous(int* const* flags, int rank, int world, int b, int* err, int code) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x < world) red_release_sys_add(flags[threadIdx.x] + b, 1);
  if (threadIdx.x == 0) {
    int* mine = flags[rank] + b;
    bool ok = false;
    for (int i = 0; i < kCommSpin; i++) {
      if (ld_acquire_sys(mine) >= world) { ok = true; break; }
      __nanosleep(32);
    }
    if (ok) *mine = 0; else atomicExch(err, code);
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

template <typename T>
__global__ void allreduce_oneshot_kernel(const T* const* bufs, int* const* flags, T* out, int64_t n, int rank, int world,
                                         int* err, const T* residual, const T* bias, int ncols) {
  pdl_launch_dependents();
  pdl_wait();
  // this rank's contribution is already in bufs[rank] (written by the previous kernel on this stream)
  __threadfence_system();
  if (!block_rendezvous(flags, rank, world, blockIdx.x, err, 5)) return;
  constexpr int VEC = 16 / sizeof(T);
  const int64_t nvec = n / VEC;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) acc[j] = 0.f;
    // issue every rank's load before the first use: the remote round trips overlap instead of adding up
    uint4 raw[8];
#pragma unroll
    for (int r = 0; r < 8; r++)
      if (r < world) raw[r] = ld_relaxed_sys_v4(bufs[r] + v * VEC);
#pragma unroll
    for (int r = 0; r < 8; r++) {
      if (r < world) {
        const T* e = reinterpret_cast<const T*>(&raw[r]);
#pragma unroll
        for (int j = 0; j < VEC; j++) acc[j] += DT<T>::to_f(e[j]);
      }
    }
    // epilogue of a row-parallel layer: + residual (same shape as out) + bias (per column, ncols columns per row)
    if (residual != nullptr) {
#pragma unroll
      for (int j = 0; j < VEC; j++) acc[j] += DT<T>::to_f(residual[v * VEC + j]);
    }
    if (bias != nullptr) {
#pragma unroll
      for (int j = 0; j < VEC; j++) acc[j] += DT<T>::to_f(bias[(v * VEC + j) % ncols]);
    }
    __align__(16) T o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) o[j] = DT<T>::from_f(acc[j]);
    *reinterpret_cast<uint4*>(out + v * VEC) = *reinterpret_cast<const uint4*>(o);
  }
  // tail elements
  for (int64_t i = nvec * VEC + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < world; r++) acc += DT<T>::to_f(*reinterpret_cast<const volatile T*>(bufs[r] + i));
    if (residual != nullptr) acc += DT<T>::to_f(residual[i]);
    if (bias != nullptr) acc += DT<T>::to_f(bias[i % ncols]);
    out[i] = DT<T>::from_f(acc);
  }
}

__global__ void barrier_kernel(int* const* flags, int rank, int world, int* err) {
  __threadfence_system();
  block_rendezvous(flags, rank, world, blockIdx.x, err, 6);
}

// A wait that nothing satisfies: used by the tests of the time-out path (the counter is private to this GPU and
// nobody increments it).  Returns through *err after `spins` polls; never touches a peer.
__global__ void wait_timeout_probe_kernel(int* counter, int expect, int spins, int* err) {
  if (threadIdx.x == 0) {
    bool ok = false;
    for (int i = 0; i < spins; i++) {
      if (ld_acquire_sys(counter) >= expect) { ok = true; break; }
      __nanosleep(64);
    }
    if (!ok) atomicExch(err, 7);
  }
}

}  // namespace

// bufs / flags: device arrays of `world` pointers (every rank's input buffer and arrival counters for this
// call's parity).  n elements of `dtype`; out is local.  blocks <= number of counters per parity (64).
// Same with the epilogue of a row-parallel layer: out = sum over ranks + residual (n elements, or null) + bias
// (ncols values repeated along the rows, or null).  out may alias residual.
IPEX_API int ipex_allreduce_oneshot_epi(const void* bufs, const void* flags, void* out, int64_t n, int dtype, int rank,
                                        int world, int* err, int blocks, int pdl, const void* residual,
                                        const void* bias, int ncols, void* stream) {
  if (world < 1 || world > 8 || blocks < 1 || blocks > 64 || (bias != nullptr && ncols < 1))
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16)
    return (int)launch_kernel(allreduce_oneshot_kernel<__half>, dim3(blocks), dim3(512), 0, s, pdl != 0,
                              (const __half* const*)bufs, (int* const*)flags, (__half*)out, n, rank, world, err,
                              (const __half*)residual, (const __half*)bias, ncols);
  if (dtype == DT_BF16)
    return (int)launch_kernel(allreduce_oneshot_kernel<__nv_bfloat16>, dim3(blocks), dim3(512), 0, s, pdl != 0,
                              (const __nv_bfloat16* const*)bufs, (int* const*)flags, (__nv_bfloat16*)out, n, rank,
                              world, err, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)bias, ncols);
  if (dtype == DT_F32)
    return (int)launch_kernel(allreduce_oneshot_kernel<float>, dim3(blocks), dim3(512), 0, s, pdl != 0,
                              (const float* const*)bufs, (int* const*)flags, (float*)out, n, rank, world, err,
                              (const float*)residual, (const float*)bias, ncols);
  return (int)cudaErrorInvalidValue;
}

IPEX_API int ipex_allreduce_oneshot(const void* bufs, const void* flags, void* out, int64_t n, int dtype, int rank,
                                    int world, int* err, int blocks, int pdl, void* stream) {
  return ipex_allreduce_oneshot_epi(bufs, flags, out, n, dtype, rank, world, err, blocks, pdl, nullptr, nullptr, 0,
                                    stream);
}

IPEX_API int ipex_symm_barrier(const void* flags, int rank, int world, int* err, void* stream) {
  barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((int* const*)flags, rank, world, err);
  return (int)cudaGetLastError();
}

IPEX_API int ipex_wait_timeout_probe(int* counter, int expect, int spins, int* err, void* stream) {
  wait_timeout_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(counter, expect, spins, err);
  return (int)cudaGetLastError();
}
