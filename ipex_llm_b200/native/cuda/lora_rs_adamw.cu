// Data-parallel LoRA optimizer step as ONE kernel per rank:
//   reduce-scatter of the gradients + AdamW on the owned shard + all-gather of the updated parameters,
// all over NVLink peer memory (plain peer loads / stores on symmetric buffers).
//
// The trainable parameters of a QLoRA run are tiny (rank-8 adapters of a 13B model: ~31 M values, ~63 MB in bf16),
// so the step is latency bound: instead of NCCL reduce-scatter -> optimizer kernels -> NCCL all-gather (three
// launches plus two library collectives) every rank runs this kernel once.
//
//   flat layout (identical on every rank):  grads[n], params[n] in the training dtype, symmetric (peer mapped);
//   rank r owns elements [r * shard, (r + 1) * shard) and keeps fp32 master / exp_avg / exp_avg_sq for them only
//   (optimizer state is sharded: ZeRO-1).
//
//   1. rendezvous A : every rank's gradients are complete (they were written by kernels earlier in its stream);
//   2. owned shard  : g = scale * sum_r grads_r[i];  AdamW on the fp32 master;  the new value, rounded to the
//                     training dtype, is stored into params_r[i] of EVERY rank;
//   3. rendezvous B : every shard has been stored everywhere, so after the kernel the local params are complete.
// Rendezvous = one arrival counter per block and rank (red.release.sys on the peers, bounded ld.acquire.sys spin on
// the own one, self-resetting).  A and B use different counter sets; B of step k orders A of step k+1 behind A of
// step k, so the same two sets serve every step.  A wait that expires writes an error code (12 / 13) and the block
// returns without touching parameters further.
//
// world == 1 degenerates to a fused flat AdamW (no peers, no rendezvous).
//
// Reference counterpart: none as a kernel.  The reference trains LoRA adapters with HF Trainer DDP (oneCCL
// all-reduce) or DeepSpeed ZeRO-2/3 plus torch.optim.AdamW
// (python/llm/example/GPU/LLM-Finetuning/QLoRA/alpaca-qlora/alpaca_qlora_finetuning.py:242-272).
#include "common/utils.cuh"

namespace {

constexpr int kSpin = 1 << 22;

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

__device__ bool rendezvous(int* const* flags, int rank, int world, int b, int* err, int code) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x < world) red_release_sys_add(flags[threadIdx.x] + b, 1);
  if (threadIdx.x == 0) {
    int* mine = flags[rank] + b;
    bool ok = false;
    for (int i = 0; i < kSpin; i++) {
      if (ld_acquire_sys(mine) >= world) { ok = true; break; }
      __nanosleep(32);
    }
    if (ok) *mine = 0; else atomicExch(err, code);
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

struct AdamArgs {
  const void* const* grads;  // [world] flat gradient buffers
  void* const* params;       // [world] flat parameter buffers
  int* const* flags_a;       // [world] arrival counters, set A
  int* const* flags_b;       // [world] arrival counters, set B
  float* master;             // [shard] fp32 copy of the owned parameters
  float* exp_avg;            // [shard]
  float* exp_avg_sq;         // [shard]
  const float* grad_scale;   // device scalar multiplied into the summed gradient (1/world, loss scale, clip) or null
  int64_t shard;             // elements per rank (multiple of 8)
  int rank, world;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^t
  int zero_grads;            // clear the local gradient shard-sources after use
  int* err;
};

template <typename T>
__global__ void __launch_bounds__(512) lora_rs_adamw_kernel(AdamArgs a) {
  constexpr int VEC = 16 / sizeof(T);
  if (a.world > 1) {
    __threadfence_system();
    if (!rendezvous(a.flags_a, a.rank, a.world, blockIdx.x, a.err, 12)) return;
  }
  const float gs = a.grad_scale != nullptr ? *a.grad_scale : 1.0f;
  const int64_t base = (int64_t)a.rank * a.shard;
  const int64_t nvec = a.shard / VEC;
  const float step = a.lr / a.bc1;
  const float inv_bc2_sqrt = rsqrtf(a.bc2);
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i0 = v * VEC;
    float g[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) g[j] = 0.f;
    for (int r = 0; r < a.world; r++) {
      const T* src = reinterpret_cast<const T*>(a.grads[r]) + base + i0;
      const uint4 raw = a.world > 1 ? ld_relaxed_sys_v4(src) : *reinterpret_cast<const uint4*>(src);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; j++) g[j] += DT<T>::to_f(e[j]);
    }
    __align__(16) T outv[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) {
      const int64_t i = i0 + j;
      const float grad = g[j] * gs;
      float w = a.master[i];
      const float m = a.beta1 * a.exp_avg[i] + (1.f - a.beta1) * grad;
      const float s = a.beta2 * a.exp_avg_sq[i] + (1.f - a.beta2) * grad * grad;
      a.exp_avg[i] = m;
      a.exp_avg_sq[i] = s;
      w -= a.lr * a.weight_decay * w;                       // decoupled weight decay
      w -= step * m / (sqrtf(s) * inv_bc2_sqrt + a.eps);    // sqrt(s / bc2) + eps
      a.master[i] = w;
      outv[j] = DT<T>::from_f(w);
    }
    const uint4 packed = *reinterpret_cast<const uint4*>(outv);
    for (int r = 0; r < a.world; r++)
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.params[r]) + base + i0) = packed;
  }
  if (a.world > 1) {
    __threadfence_system();
    rendezvous(a.flags_b, a.rank, a.world, blockIdx.x, a.err, 13);
  }
}

}  // namespace

// One optimizer step for the flat LoRA parameter space (see the head of this file).
//   grads / params / flags_a / flags_b : device arrays of `world` pointers;  shard % 8 == 0;  blocks <= 64.
//   dtype: DT_F16 / DT_BF16 / DT_F32 of grads and params.  step_t >= 1 is the AdamW step count (bias correction).
IPEX_API int ipex_lora_rs_adamw(const void* grads, const void* params, const void* flags_a, const void* flags_b,
                                float* master, float* exp_avg, float* exp_avg_sq, const float* grad_scale,
                                int64_t shard, int rank, int world, float lr, float beta1, float beta2, float eps,
                                float weight_decay, int step_t, int dtype, int blocks, int* err, void* stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || shard < 0 || (shard % 8) != 0 || step_t < 1 ||
      blocks < 1 || blocks > 64)
    return (int)cudaErrorInvalidValue;
  AdamArgs a;
  a.grads = (const void* const*)grads; a.params = (void* const*)params;
  a.flags_a = (int* const*)flags_a; a.flags_b = (int* const*)flags_b;
  a.master = master; a.exp_avg = exp_avg; a.exp_avg_sq = exp_avg_sq; a.grad_scale = grad_scale;
  a.shard = shard; a.rank = rank; a.world = world;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step_t);
  a.bc2 = 1.f - powf(beta2, (float)step_t);
  a.zero_grads = 0;
  a.err = err;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_BF16) lora_rs_adamw_kernel<__nv_bfloat16><<<blocks, 512, 0, s>>>(a);
  else if (dtype == DT_F16) lora_rs_adamw_kernel<__half><<<blocks, 512, 0, s>>>(a);
  else if (dtype == DT_F32) lora_rs_adamw_kernel<float><<<blocks, 512, 0, s>>>(a);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}
