// Memory-bound helper kernels: norms, activation*mul, softmax, RoPE, fp8 KV conversion, logits penalty,
// embedding gather, argmax.
//
// Stand-ins for the reference's closed `xe_addons` ops `rms_norm`, `layer_norm`, `mlp_silu_mul_inplaced`,
// `attn_softmax_inplaced`, `rotary_half_inplaced`, `rotary_two_inplaced`, `rotary_*_with_cache_inplaced`,
// `quantize_key_value`, `dequantize_key_value`, `repetition_penalty_logits_process_inplaced`
// (python/llm/src/ipex_llm/transformers/xpu_ops.py:70-162).
#include "common/utils.cuh"

namespace {

template <int N>
struct alignas(16) Pack8 { uint4 v; };

// ------------------------------------------------------------------------------------------------
// RMSNorm / LayerNorm: one CTA per row, 16-byte vector access, fp32 statistics
// ------------------------------------------------------------------------------------------------
template <typename T, bool LAYER>
__global__ void norm_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                            const T* __restrict__ residual, T* __restrict__ y, T* __restrict__ res_out, int H,
                            float eps, float w_offset) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sh[];  // H floats + 64
  float* row = sh;
  float* red = sh + H;
  const size_t base = (size_t)blockIdx.x * H;
  const int tid = threadIdx.x, nt = blockDim.x;
  float s = 0.f, ss = 0.f;
  for (int i = tid; i < H; i += nt) {
    float v = DT<T>::to_f(x[base + i]);
    if (residual != nullptr) {
      v += DT<T>::to_f(residual[base + i]);
      if (res_out != nullptr) res_out[base + i] = DT<T>::from_f(v);
      v = DT<T>::to_f(DT<T>::from_f(v));
    }
    row[i] = v;
    s += v;
    ss += v * v;
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  if ((tid & 31) == 0) { red[tid >> 5] = s; red[32 + (tid >> 5)] = ss; }
  __syncthreads();
  float ts = 0.f, tss = 0.f;
  for (int i = 0; i < (nt + 31) / 32; i++) { ts += red[i]; tss += red[32 + i]; }
  float mean = LAYER ? ts / H : 0.f;
  float var = LAYER ? fmaxf(tss / H - mean * mean, 0.f) : tss / H;
  float rstd = rsqrtf(var + eps);
  for (int i = tid; i < H; i += nt) {
    float v = (row[i] - mean) * rstd;
    if (!LAYER) v = DT<T>::to_f(DT<T>::from_f(v));  // HF casts the normalised value before the weight multiply
    float o = v * ((w != nullptr ? DT<T>::to_f(w[i]) : 1.f) + w_offset);
    if (LAYER && b != nullptr) o += DT<T>::to_f(b[i]);
    y[base + i] = DT<T>::from_f(o);
  }
}

// ------------------------------------------------------------------------------------------------
// act(gate) * up
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, size_t n,
                               int act) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float g = DT<T>::to_f(gate[i]), u = DT<T>::to_f(up[i]);
    float a;
    if (act == 0) {
      a = g / (1.f + __expf(-g));
    } else {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      a = 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
    }
    out[i] = DT<T>::from_f(a * u);
  }
}

// ------------------------------------------------------------------------------------------------
// softmax over the last dimension, in place, fp32 accumulation (one warp per row when cols <= 1024,
// one CTA per row otherwise)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void softmax_kernel(T* __restrict__ x, int cols) {
  extern __shared__ float sh[];
  const size_t base = (size_t)blockIdx.x * cols;
  const int tid = threadIdx.x, nt = blockDim.x;
  float m = -INFINITY;
  for (int i = tid; i < cols; i += nt) m = fmaxf(m, DT<T>::to_f(x[base + i]));
  m = warp_max(m);
  if ((tid & 31) == 0) sh[tid >> 5] = m;
  __syncthreads();
  for (int i = 0; i < (nt + 31) / 32; i++) m = fmaxf(m, sh[i]);
  __syncthreads();
  float s = 0.f;
  for (int i = tid; i < cols; i += nt) s += __expf(DT<T>::to_f(x[base + i]) - m);
  s = warp_sum(s);
  if ((tid & 31) == 0) sh[tid >> 5] = s;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (nt + 31) / 32; i++) tot += sh[i];
  float inv = 1.f / tot;
  for (int i = tid; i < cols; i += nt) x[base + i] = DT<T>::from_f(__expf(DT<T>::to_f(x[base + i]) - m) * inv);
}

// ------------------------------------------------------------------------------------------------
// RoPE in place on strided q / k views [B, H, S, D] (element strides given), cos/sin [B, S, R] fp32 or T.
// interleaved = 0: pairs (i, i + R/2) ("half" / NeoX); 1: pairs (2i, 2i+1) ("two" / GPT-J).
// ------------------------------------------------------------------------------------------------
template <typename T, typename CT>
__global__ void rope_kernel(T* __restrict__ q, T* __restrict__ k, const CT* __restrict__ cosp,
                            const CT* __restrict__ sinp, int B, int Hq, int Hk, int S, int R, int64_t qs_b,
                            int64_t qs_h, int64_t qs_s, int64_t ks_b, int64_t ks_h, int64_t ks_s, int64_t cs_b,
                            int64_t cs_s, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = R / 2;
  const int64_t total = (int64_t)B * (Hq + Hk) * S * half;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int i = (int)(idx % half);
    int64_t r = idx / half;
    int s = (int)(r % S);
    r /= S;
    int h = (int)(r % (Hq + Hk));
    int b = (int)(r / (Hq + Hk));
    T* p;
    if (h < Hq) p = q + b * qs_b + (int64_t)h * qs_h + (int64_t)s * qs_s;
    else p = k + b * ks_b + (int64_t)(h - Hq) * ks_h + (int64_t)s * ks_s;
    const CT* cp = cosp + b * cs_b + (int64_t)s * cs_s;
    const CT* sp = sinp + b * cs_b + (int64_t)s * cs_s;
    int i0, i1;
    float c, sn;
    if (interleaved) {
      i0 = 2 * i; i1 = 2 * i + 1;
      c = DT<CT>::to_f(cp[i]); sn = DT<CT>::to_f(sp[i]);
    } else {
      i0 = i; i1 = i + half;
      c = DT<CT>::to_f(cp[i]); sn = DT<CT>::to_f(sp[i]);
    }
    float x0 = DT<T>::to_f(p[i0]), x1 = DT<T>::to_f(p[i1]);
    p[i0] = DT<T>::from_f(x0 * c - x1 * sn);
    p[i1] = DT<T>::from_f(x1 * c + x0 * sn);
  }
}

// ------------------------------------------------------------------------------------------------
// fp8 e5m2 <-> half conversions for the KV cache (e5m2 = upper byte of fp16, round-to-nearest-even,
// saturating to +-57344)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint8_t f32_to_e5m2(float v) {
  v = fminf(fmaxf(v, -57344.f), 57344.f);
  uint16_t h = __half_as_ushort(__float2half_rn(v));
  uint16_t lsb = (h >> 8) & 1;
  uint32_t r = (uint32_t)h + 0x7F + lsb;
  uint8_t out = (uint8_t)(r >> 8);
  if ((out & 0x7F) > 0x7B) out = (out & 0x80) | 0x7B;  // never round up into inf/nan
  return out;
}
__device__ __forceinline__ float e5m2_to_f32(uint8_t b) { return __half2float(__ushort_as_half((uint16_t)b << 8)); }

template <typename T>
__global__ void kv_quant_kernel(const T* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int D,
                                int64_t src_row_stride_elems, const int64_t* __restrict__ unused) {
  int64_t n = rows * D;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / D;
    int d = (int)(i % D);
    dst[i] = f32_to_e5m2(DT<T>::to_f(src[r * src_row_stride_elems + d]));
  }
}

template <typename T>
__global__ void kv_dequant_kernel(const uint8_t* __restrict__ src, T* __restrict__ dst, int64_t rows, int D,
                                  int64_t src_row_stride) {
  int64_t n = rows * D;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / D;
    int d = (int)(i % D);
    dst[i] = DT<T>::from_f(e5m2_to_f32(src[r * src_row_stride + d]));
  }
}

// ------------------------------------------------------------------------------------------------
// repetition penalty on logits [B, V] for the token ids in ids [B, L]
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rep_penalty_kernel(T* __restrict__ logits, const int64_t* __restrict__ ids, int B, int V, int L,
                                   float penalty) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * L) return;
  int b = idx / L;
  int64_t tok = ids[idx];
  if (tok < 0 || tok >= V) return;
  // idempotent per token only if applied once: skip when an earlier position holds the same id
  for (int j = 0; j < idx % L; j++)
    if (ids[(int64_t)b * L + j] == tok) return;
  float v = DT<T>::to_f(logits[(size_t)b * V + tok]);
  v = v < 0.f ? v * penalty : v / penalty;
  logits[(size_t)b * V + tok] = DT<T>::from_f(v);
}

// ------------------------------------------------------------------------------------------------
// embedding gather (half table) and greedy argmax over logits
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out, int H,
                             float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t tok = ids[blockIdx.x];
  const T* src = table + tok * (int64_t)H;
  T* dst = out + (int64_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    dst[i] = scale == 1.f ? src[i] : DT<T>::from_f(DT<T>::to_f(src[i]) * scale);
}

template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, int64_t* __restrict__ out, int V, int64_t ld) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float bv[32];
  __shared__ int bi[32];
  const T* row = logits + (int64_t)blockIdx.x * ld;
  float best = -INFINITY;
  int besti = 0;
  int done = 0;
  if constexpr (sizeof(T) == 2) {
    // 16-byte loads, a few independent ones per thread (a scalar walk was a chain of ~30 dependent 2-byte loads)
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const int nvec = V / 8;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + (size_t)v * 8);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const float f = DT<T>::to_f(e[j]);
          if (f > best) { best = f; besti = v * 8 + j; }     // ascending index inside a thread: first maximum wins
        }
      }
      done = nvec * 8;
    }
  }
  for (int i = done + threadIdx.x; i < V; i += blockDim.x) {
    float v = DT<T>::to_f(row[i]);
    if (v > best || (v == best && i < besti)) { best = v; besti = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = besti; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x + 31) / 32; w++)
      if (bv[w] > best || (bv[w] == best && bi[w] < besti)) { best = bv[w]; besti = bi[w]; }
    out[blockIdx.x] = besti;
  }
}

template <typename F>
int by_dtype(int dtype, F&& f) {
  if (dtype == DT_F16) return (int)f((__half*)nullptr);
  if (dtype == DT_BF16) return (int)f((__nv_bfloat16*)nullptr);
  if (dtype == DT_F32) return (int)f((float*)nullptr);
  return (int)cudaErrorInvalidValue;
}

}  // namespace

IPEX_API int ipex_rms_norm(const void* x, const void* w, const void* residual, void* y, void* res_out, int64_t rows,
                           int H, float eps, float w_offset, int dtype, int pdl, void* stream) {
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    int threads = H >= 2048 ? 512 : 256;
    size_t smem = (size_t)(H + 64) * sizeof(float);
    auto kern = norm_kernel<T, false>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kern, dim3((unsigned)rows), dim3(threads), smem, (cudaStream_t)stream, pdl != 0,
                         (const T*)x, (const T*)w, (const T*)nullptr, (const T*)residual, (T*)y, (T*)res_out, H, eps,
                         w_offset);
  });
}

IPEX_API int ipex_layer_norm(const void* x, const void* w, const void* b, void* y, int64_t rows, int H, float eps,
                             int dtype, void* stream) {
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    size_t smem = (size_t)(H + 64) * sizeof(float);
    auto kern = norm_kernel<T, true>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kern, dim3((unsigned)rows), dim3(256), smem, (cudaStream_t)stream, false, (const T*)x,
                         (const T*)w, (const T*)b, (const T*)nullptr, (T*)y, (T*)nullptr, H, eps, 0.f);
  });
}

IPEX_API int ipex_act_mul(const void* gate, const void* up, void* out, int64_t n, int act, int dtype, int pdl,
                          void* stream) {
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    return launch_kernel(act_mul_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, pdl != 0, (const T*)gate,
                         (const T*)up, (T*)out, (size_t)n, act);
  });
}

IPEX_API int ipex_softmax_inplace(void* x, int64_t rows, int cols, int dtype, void* stream) {
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    int threads = cols >= 1024 ? 256 : 64;
    softmax_kernel<T><<<(unsigned)rows, threads, 256, (cudaStream_t)stream>>>((T*)x, cols);
    return cudaGetLastError();
  });
}

IPEX_API int ipex_rope_inplace(void* q, void* k, const void* cosp, const void* sinp, int B, int Hq, int Hk, int S,
                               int R, int64_t qs_b, int64_t qs_h, int64_t qs_s, int64_t ks_b, int64_t ks_h,
                               int64_t ks_s, int64_t cs_b, int64_t cs_s, int interleaved, int dtype, int cos_dtype,
                               void* stream) {
  int64_t total = (int64_t)B * (Hq + Hk) * S * (R / 2);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if (cos_dtype == DT_F32) {
      return launch_kernel(rope_kernel<T, float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, false, (T*)q,
                           (T*)k, (const float*)cosp, (const float*)sinp, B, Hq, Hk, S, R, qs_b, qs_h, qs_s, ks_b,
                           ks_h, ks_s, cs_b, cs_s, interleaved);
    }
    return launch_kernel(rope_kernel<T, T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, false, (T*)q, (T*)k,
                         (const T*)cosp, (const T*)sinp, B, Hq, Hk, S, R, qs_b, qs_h, qs_s, ks_b, ks_h, ks_s, cs_b,
                         cs_s, interleaved);
  });
}

IPEX_API int ipex_kv_quant_e5m2(const void* src, void* dst, int64_t rows, int D, int64_t src_row_stride, int dtype,
                                void* stream) {
  int64_t n = rows * D;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (blocks < 1) blocks = 1;
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    kv_quant_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)src, (uint8_t*)dst, rows, D, src_row_stride,
                                                                 nullptr);
    return cudaGetLastError();
  });
}

IPEX_API int ipex_kv_dequant_e5m2(const void* src, void* dst, int64_t rows, int D, int64_t src_row_stride, int dtype,
                                  void* stream) {
  int64_t n = rows * D;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (blocks < 1) blocks = 1;
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    kv_dequant_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (T*)dst, rows, D,
                                                                   src_row_stride);
    return cudaGetLastError();
  });
}

IPEX_API int ipex_repetition_penalty(void* logits, const void* ids, int B, int V, int L, float penalty, int dtype,
                                     void* stream) {
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    int n = B * L;
    rep_penalty_kernel<T><<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((T*)logits, (const int64_t*)ids, B, V, L,
                                                                             penalty);
    return cudaGetLastError();
  });
}

IPEX_API int ipex_embedding(const void* ids, const void* table, void* out, int64_t n_tokens, int H, float scale,
                            int dtype, int pdl, void* stream) {
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    return launch_kernel(embed_kernel<T>, dim3((unsigned)n_tokens), dim3(256), 0, (cudaStream_t)stream, pdl != 0,
                         (const int64_t*)ids, (const T*)table, (T*)out, H, scale);
  });
}

IPEX_API int ipex_argmax(const void* logits, void* out, int rows, int V, int64_t ld, int dtype, int pdl, void* stream) {
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    return launch_kernel(argmax_kernel<T>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, pdl != 0,
                         (const T*)logits, (int64_t*)out, V, ld);
  });
}
