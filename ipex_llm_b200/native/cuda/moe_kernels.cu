// Mixture-of-experts routing on the device (the expert GEMVs themselves are ipex_moe_gemv in gemv_lowbit.cu).
//
// Reference counterparts: xe_addons.moe_softmax_topk and xe_addons.moe_group_topk as used by
// python/llm/src/ipex_llm/transformers/models/common.py:343-361 (Mixtral / Qwen-MoE routing: softmax over the experts
// in fp32, top-k, optional renormalisation) and models/deepseek.py:274-346 (grouped top-k with a score bias).
// One warp per token; experts are spread over the lanes (E <= 256), top-k (k <= 8) by repeated warp arg-max.
#include "common/utils.cuh"

namespace {

constexpr int kMaxPerLane = 8;  // 256 experts / 32 lanes

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

template <typename T>
__global__ void moe_softmax_topk_kernel(const T* __restrict__ logits, float* __restrict__ probs, float* __restrict__ w,
                                        int64_t* __restrict__ idx, int tokens, int E, int k, int renorm) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const T* row = logits + (size_t)warp * E;
  float v[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; j++) {
    const int e = lane + 32 * j;
    v[j] = e < E ? DT<T>::to_f(row[e]) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; j++) {
    v[j] = (lane + 32 * j) < E ? __expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; j++) {
    v[j] *= inv;
    const int e = lane + 32 * j;
    if (e < E && probs != nullptr) probs[(size_t)warp * E + e] = v[j];
    if (e >= E) v[j] = -1.f;
  }
  float chosen[8];
  int chosen_i[8];
  float tot = 0.f;
  for (int r = 0; r < k; r++) {
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; j++)
      if (v[j] > bv) { bv = v[j]; bi = lane + 32 * j; }
    warp_argmax(bv, bi);
    chosen[r] = bv;
    chosen_i[r] = bi;
    tot += bv;
    if ((bi & 31) == lane) v[bi >> 5] = -1.f;   // remove the winner
  }
  if (lane == 0) {
    const float s = renorm ? 1.0f / tot : 1.0f;
    for (int r = 0; r < k; r++) {
      w[(size_t)warp * k + r] = chosen[r] * s;
      idx[(size_t)warp * k + r] = chosen_i[r];
    }
  }
}

// out[t] = sum_r weights[t, r] * y[t * k + r]   (combining the experts' outputs)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const float* __restrict__ w, const T* __restrict__ residual,
                                   T* __restrict__ out, int tokens, int k, int H) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)tokens * H) return;
  const int t = (int)(i / H), h = (int)(i % H);
  float acc = residual != nullptr ? DT<T>::to_f(residual[i]) : 0.f;
  for (int r = 0; r < k; r++) acc += w[(size_t)t * k + r] * DT<T>::to_f(y[((size_t)t * k + r) * H + h]);
  out[i] = DT<T>::from_f(acc);
}

// DeepSeek-V3 grouped routing, one warp per token: s = sigmoid(score), sb = s + bias; a group's score is the sum of
// its two largest sb; the topk_group best groups stay; the top_k largest sb among them are chosen (descending); the
// weights are the UNBIASED s of the chosen experts, optionally renormalised, times `scale`.
template <typename T>
__global__ void moe_group_topk_kernel(const T* __restrict__ scores, const float* __restrict__ bias,
                                      int64_t* __restrict__ idx, float* __restrict__ w, int tokens, int E, int n_group,
                                      int topk_group, int k, int renorm, float scale) {
  extern __shared__ float sm_gt[];                 // per warp: sb [E] | group score [32] | group kept [32]
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + wib;
  if (tok >= tokens) return;
  float* sb = sm_gt + (size_t)wib * (E + 64);
  float* gscore = sb + E;
  float* gkeep = gscore + 32;
  const int gs = E / n_group;
  float s[kMaxPerLane], v[kMaxPerLane];
#pragma unroll
  for (int j = 0; j < kMaxPerLane; j++) {
    const int i = lane + 32 * j;
    s[j] = 0.f;
    v[j] = -INFINITY;
    if (i < E) {
      s[j] = 1.0f / (1.0f + __expf(-DT<T>::to_f(scores[(size_t)tok * E + i])));
      v[j] = s[j] + bias[i];
      sb[i] = v[j];
    }
  }
  __syncwarp();
  if (lane < n_group) {
    float a = -INFINITY, b = -INFINITY;            // two largest of the group
    for (int i = 0; i < gs; i++) {
      const float x = sb[lane * gs + i];
      if (x > a) { b = a; a = x; } else if (x > b) { b = x; }
    }
    gscore[lane] = a + b;
    gkeep[lane] = 0.f;
  }
  __syncwarp();
  if (lane == 0) {
    for (int r = 0; r < topk_group; r++) {
      int best = -1;
      float bv = -INFINITY;
      for (int g = 0; g < n_group; g++)
        if (gkeep[g] == 0.f && (best < 0 || gscore[g] > bv)) { best = g; bv = gscore[g]; }
      if (best >= 0) gkeep[best] = 1.f;
    }
  }
  __syncwarp();
#pragma unroll
  for (int j = 0; j < kMaxPerLane; j++) {
    const int i = lane + 32 * j;
    if (i >= E || gkeep[i / gs] == 0.f) v[j] = -INFINITY;
  }
  float chosen[8];
  int chosen_i[8];
  float tot = 0.f;
  for (int r = 0; r < k; r++) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; j++)
      if (v[j] > bv) { bv = v[j]; bi = lane + 32 * j; }
    warp_argmax(bv, bi);
    bi = bi == 0x7fffffff ? 0 : bi;
    // the weight is the unbiased score of the winner: its owner broadcasts it
    float sw = 0.f;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < kMaxPerLane; j++)
        if (j == (bi >> 5)) { sw = s[j]; v[j] = -INFINITY; }
    }
    sw = __shfl_sync(0xffffffffu, sw, bi & 31);
    chosen[r] = sw;
    chosen_i[r] = bi;
    tot += sw;
  }
  if (lane == 0) {
    const float f = (renorm ? 1.0f / (tot + 1e-20f) : 1.0f) * scale;
    for (int r = 0; r < k; r++) {
      w[(size_t)tok * k + r] = chosen[r] * f;
      idx[(size_t)tok * k + r] = chosen_i[r];
    }
  }
}

// Stable counting sort of up to kSortMaxSlots (token, choice) slots by expert id, in one CTA.
// order[pos] = slot, ranges[e] = (first pos, count).
constexpr int kSortMaxSlots = 1024;
__global__ void moe_sort_slots_kernel(const int64_t* __restrict__ ids, int slots, int E, int* __restrict__ order,
                                      int* __restrict__ ranges) {
  __shared__ int s_id[kSortMaxSlots];
  __shared__ int s_cnt[256], s_first[256];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int s = tid; s < slots; s += blockDim.x) {
    int e = (int)ids[s];
    e = e < 0 ? 0 : (e >= E ? E - 1 : e);
    s_id[s] = e;
    atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; e++) { s_first[e] = run; run += s_cnt[e]; }
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    ranges[2 * e] = s_first[e];
    ranges[2 * e + 1] = s_cnt[e];
  }
  for (int s = tid; s < slots; s += blockDim.x) {
    const int e = s_id[s];
    int before = 0;
    for (int j = 0; j < s; j++) before += s_id[j] == e;
    order[s_first[e] + before] = s;
  }
}

}  // namespace

// logits [tokens, E] (dtype) -> probs [tokens, E] fp32 (may be null), w [tokens, k] fp32, idx [tokens, k] int64.
IPEX_API int ipex_moe_softmax_topk(const void* logits, float* probs, float* w, int64_t* idx, int tokens, int E, int k,
                                   int renorm, int dtype, void* stream) {
  if (E < 1 || E > 32 * kMaxPerLane || k < 1 || k > 8 || k > E || tokens < 1) return (int)cudaErrorInvalidValue;
  const int threads = 128, blocks = (tokens * 32 + threads - 1) / threads;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16)
    moe_softmax_topk_kernel<__half><<<blocks, threads, 0, s>>>((const __half*)logits, probs, w, idx, tokens, E, k, renorm);
  else if (dtype == DT_BF16)
    moe_softmax_topk_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((const __nv_bfloat16*)logits, probs, w, idx,
                                                                       tokens, E, k, renorm);
  else if (dtype == DT_F32)
    moe_softmax_topk_kernel<float><<<blocks, threads, 0, s>>>((const float*)logits, probs, w, idx, tokens, E, k, renorm);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

// out[t] = (residual[t] +) sum_r w[t, r] * y[t * k + r]
IPEX_API int ipex_moe_combine_add(const void* y, const float* w, const void* residual, void* out, int tokens, int k,
                                  int H, int dtype, void* stream) {
  const int64_t n = (int64_t)tokens * H;
  const int threads = 256, blocks = (int)((n + threads - 1) / threads);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16)
    moe_combine_kernel<__half><<<blocks, threads, 0, s>>>((const __half*)y, w, (const __half*)residual, (__half*)out,
                                                          tokens, k, H);
  else if (dtype == DT_BF16)
    moe_combine_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((const __nv_bfloat16*)y, w,
                                                                  (const __nv_bfloat16*)residual, (__nv_bfloat16*)out,
                                                                  tokens, k, H);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

IPEX_API int ipex_moe_combine(const void* y, const float* w, void* out, int tokens, int k, int H, int dtype,
                              void* stream) {
  return ipex_moe_combine_add(y, w, nullptr, out, tokens, k, H, dtype, stream);
}

// scores [tokens, E] (dtype), bias [E] fp32 -> idx [tokens, k] int64 (descending biased score), w [tokens, k] fp32.
// E <= 256 and divisible by n_group <= 32, topk_group <= n_group, k <= 8.
IPEX_API int ipex_moe_group_topk(const void* scores, const float* bias, int64_t* idx, float* w, int tokens, int E,
                                 int n_group, int topk_group, int k, int renorm, float scale, int dtype, void* stream) {
  if (tokens < 1 || E < 1 || E > 32 * kMaxPerLane || n_group < 1 || n_group > 32 || E % n_group != 0 ||
      topk_group < 1 || topk_group > n_group || k < 1 || k > 8 || k > topk_group * (E / n_group))
    return (int)cudaErrorInvalidValue;
  const int warps = 4, threads = warps * 32, blocks = (tokens + warps - 1) / warps;
  const size_t smem = (size_t)warps * (E + 64) * sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16)
    moe_group_topk_kernel<__half><<<blocks, threads, smem, s>>>((const __half*)scores, bias, idx, w, tokens, E, n_group,
                                                                 topk_group, k, renorm, scale);
  else if (dtype == DT_BF16)
    moe_group_topk_kernel<__nv_bfloat16><<<blocks, threads, smem, s>>>((const __nv_bfloat16*)scores, bias, idx, w,
                                                                        tokens, E, n_group, topk_group, k, renorm,
                                                                        scale);
  else if (dtype == DT_F32)
    moe_group_topk_kernel<float><<<blocks, threads, smem, s>>>((const float*)scores, bias, idx, w, tokens, E, n_group,
                                                                topk_group, k, renorm, scale);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

// Sort `slots` (token, choice) slots by expert on the device: order [slots] int32, ranges [E][2] int32
// (first position, count).  slots <= 1024, E <= 256.
IPEX_API int ipex_moe_sort_slots(const int64_t* expert_ids, int slots, int E, int* order, int* ranges, void* stream) {
  if (slots < 1 || slots > kSortMaxSlots || E < 1 || E > 256) return (int)cudaErrorInvalidValue;
  moe_sort_slots_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(expert_ids, slots, E, order, ranges);
  return (int)cudaGetLastError();
}
