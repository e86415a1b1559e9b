// RWKV recurrences and token-shift mixing, sm_100a.
//
// Counterparts of the reference's closed `xe_linear.rwkv_linear_attention_v4`, `rwkv_linear_attention_v5` and
// `rwkv_time_shift` (python/llm/src/ipex_llm/transformers/xpu_ops.py:40-56; call sites
// python/llm/src/ipex_llm/transformers/models/rwkv4.py:60,96 and models/rwkv5.py:62,102,240).
//
// All three are sequential in time and parallel over (batch, channel): the kernels keep the running state in
// registers (fp32), read each k/v/r element exactly once and write each output once.  The prompt pass is
// therefore one launch per layer instead of T tiny launches, and decode (T = 1) costs one launch as well.
#include "common/utils.cuh"

namespace {

// ---------------------------------------------------------------------------------------------------------
// v4:  wkv_t = (e^{m-p} num + e^{u+k_t-p} v_t) / (e^{m-p} den + e^{u+k_t-p}),  p = max(m, u+k_t)
//      then (num, den, m) <- decayed by w and joined with (k_t, v_t), all in the max-shifted form.
// One thread per (batch, channel); consecutive threads own consecutive channels, so every time step is one
// coalesced row read of k and v.
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) rwkv_wkv_v4_kernel(const float* __restrict__ w, const float* __restrict__ u,
                                                          const T* __restrict__ k, const T* __restrict__ v,
                                                          T* __restrict__ out, float* __restrict__ num,
                                                          float* __restrict__ den, float* __restrict__ mx, int B,
                                                          int Tn, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const float wc = w[c], uc = u[c];
  float a = num[(size_t)b * C + c], d = den[(size_t)b * C + c], m = mx[(size_t)b * C + c];
  const size_t base = (size_t)b * Tn * C + c;
  for (int t = 0; t < Tn; t++) {
    const float kt = DT<T>::to_f(k[base + (size_t)t * C]);
    const float vt = DT<T>::to_f(v[base + (size_t)t * C]);
    const float p = fmaxf(m, uc + kt);
    const float e1 = __expf(m - p), e2 = __expf(uc + kt - p);
    out[base + (size_t)t * C] = DT<T>::from_f((e1 * a + e2 * vt) / (e1 * d + e2));
    const float q = fmaxf(m + wc, kt);
    const float f1 = __expf(m + wc - q), f2 = __expf(kt - q);
    a = f1 * a + f2 * vt;
    d = f1 * d + f2;
    m = q;
  }
  num[(size_t)b * C + c] = a;
  den[(size_t)b * C + c] = d;
  mx[(size_t)b * C + c] = m;
}

// ---------------------------------------------------------------------------------------------------------
// v5 (multi-head, matrix-valued state):  per head, S x S state with rows i (key dim) and columns j (value dim)
//      out_t[j] = sum_i r_t[i] * (u[i] k_t[i] v_t[j] + state[i][j]);   state[i][j] <- k_t[i] v_t[j] + w[i] state[i][j]
// One CTA per (batch, head), thread j owns column j of the state in registers; r_t, k_t are staged in shared
// memory once per step.  r/k/v: [B, H, T, S] fp32, out: [B, T, H, S] fp32, state: [B, H, S, S] fp32 in place.
// ---------------------------------------------------------------------------------------------------------
template <int S>
__global__ void __launch_bounds__(S) rwkv_v5_kernel(const float* __restrict__ w, const float* __restrict__ u,
                                                    const float* __restrict__ r, const float* __restrict__ k,
                                                    const float* __restrict__ v, float* __restrict__ state,
                                                    float* __restrict__ out, int B, int H, int Tn) {
  __shared__ float rs[S], ks[S], ws[S], us[S];
  const int j = threadIdx.x;
  const int h = blockIdx.x, b = blockIdx.y;
  ws[j] = w[h * S + j];
  us[j] = u[h * S + j];
  float st[S];
  float* sp = state + (((size_t)b * H + h) * S) * S;
#pragma unroll
  for (int i = 0; i < S; i++) st[i] = sp[(size_t)i * S + j];
  const size_t in_base = ((size_t)b * H + h) * Tn * S;
  for (int t = 0; t < Tn; t++) {
    __syncthreads();
    rs[j] = r[in_base + (size_t)t * S + j];
    ks[j] = k[in_base + (size_t)t * S + j];
    const float vj = v[in_base + (size_t)t * S + j];
    __syncthreads();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < S; i++) {
      const float kv = ks[i] * vj;
      acc += rs[i] * (us[i] * kv + st[i]);
      st[i] = kv + ws[i] * st[i];
    }
    out[(((size_t)b * Tn + t) * H + h) * S + j] = acc;
  }
#pragma unroll
  for (int i = 0; i < S; i++) sp[(size_t)i * S + j] = st[i];
}

// ---------------------------------------------------------------------------------------------------------
// token shift + mixing:  out[n] = hidden * mix[n] + shifted * (1 - mix[n]) for n < n_mix, where shifted[t] is
// hidden[t-1] for t > 0 and prev (the last hidden row of the previous call, or zeros) for t = 0.
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rwkv_time_shift_kernel(const T* __restrict__ hidden, const T* __restrict__ prev,
                                       const T* __restrict__ mix, T* __restrict__ out, int B, int Tn, int C,
                                       int n_mix) {
  const size_t total = (size_t)B * Tn * C;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % C);
    const size_t bt = idx / C;
    const int t = (int)(bt % Tn), b = (int)(bt / Tn);
    const float x = DT<T>::to_f(hidden[idx]);
    float s = 0.f;
    if (t > 0) s = DT<T>::to_f(hidden[idx - C]);
    else if (prev != nullptr) s = DT<T>::to_f(prev[(size_t)b * C + c]);
    for (int n = 0; n < n_mix; n++) {
      const float mv = DT<T>::to_f(mix[(size_t)n * C + c]);
      out[(size_t)n * total + idx] = DT<T>::from_f(x * mv + s * (1.f - mv));
    }
  }
}

}  // namespace

// time_decay `w` (already -exp(decay)) and time_first `u`: fp32 [C]; k, v, out: [B, T, C] contiguous in `dtype`;
// num/den/max: fp32 [B, C], updated in place.  Returns a cudaError_t.
IPEX_API int ipex_rwkv_wkv_v4(const float* w, const float* u, const void* k, const void* v, void* out, float* num,
                              float* den, float* mx, int B, int T, int C, int dtype, void* stream) {
  if (B < 1 || T < 1 || C < 1 || B > 65535) return (int)cudaErrorInvalidValue;
  dim3 grid((C + 127) / 128, B);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16)
    rwkv_wkv_v4_kernel<__half><<<grid, 128, 0, s>>>(w, u, (const __half*)k, (const __half*)v, (__half*)out, num, den,
                                                     mx, B, T, C);
  else if (dtype == DT_BF16)
    rwkv_wkv_v4_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(w, u, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                            (__nv_bfloat16*)out, num, den, mx, B, T, C);
  else if (dtype == DT_F32)
    rwkv_wkv_v4_kernel<float><<<grid, 128, 0, s>>>(w, u, (const float*)k, (const float*)v, (float*)out, num, den, mx,
                                                    B, T, C);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

// w (= exp(-exp(decay))) and u: fp32 [H, S]; r, k, v: fp32 [B, H, T, S]; state: fp32 [B, H, S, S] in place;
// out: fp32 [B, T, H, S].  S is 32, 64 or 128.  Returns a cudaError_t.
IPEX_API int ipex_rwkv_linear_attention_v5(const float* w, const float* u, const float* r, const float* k,
                                           const float* v, float* state, float* out, int B, int H, int T, int S,
                                           void* stream) {
  if (B < 1 || H < 1 || T < 1 || B > 65535) return (int)cudaErrorInvalidValue;
  dim3 grid(H, B);
  cudaStream_t s = (cudaStream_t)stream;
  switch (S) {
    case 32: rwkv_v5_kernel<32><<<grid, 32, 0, s>>>(w, u, r, k, v, state, out, B, H, T); break;
    case 64: rwkv_v5_kernel<64><<<grid, 64, 0, s>>>(w, u, r, k, v, state, out, B, H, T); break;
    case 128: rwkv_v5_kernel<128><<<grid, 128, 0, s>>>(w, u, r, k, v, state, out, B, H, T); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

// hidden [B, T, C], prev [B, C] or NULL, mix [n_mix, C], out [n_mix, B, T, C]; all `dtype`, contiguous.
IPEX_API int ipex_rwkv_time_shift(const void* hidden, const void* prev, const void* mix, void* out, int B, int T, int C,
                                  int n_mix, int dtype, void* stream) {
  if (B < 1 || T < 1 || C < 1 || n_mix < 1) return (int)cudaErrorInvalidValue;
  const size_t total = (size_t)B * T * C;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16)
    rwkv_time_shift_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)hidden, (const __half*)prev,
                                                          (const __half*)mix, (__half*)out, B, T, C, n_mix);
  else if (dtype == DT_BF16)
    rwkv_time_shift_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)hidden,
                                                                 (const __nv_bfloat16*)prev,
                                                                 (const __nv_bfloat16*)mix, (__nv_bfloat16*)out, B, T,
                                                                 C, n_mix);
  else if (dtype == DT_F32)
    rwkv_time_shift_kernel<float><<<blocks, 256, 0, s>>>((const float*)hidden, (const float*)prev, (const float*)mix,
                                                         (float*)out, B, T, C, n_mix);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}
