// GPU quantizers (dense weight -> device tile layout) and dequantizers (tile layout / canonical blocks -> dense).
//
// * quantize: what the reference does on the host through `ggml_quantize_tensor`
//   (python/llm/src/ipex_llm/transformers/low_bit_linear.py:104-175) followed by `ggml_q_format_convet_cpu2xpu`
//   (:178-233) happens here in one pass on the GPU: a warp owns one block, finds the scale with shuffles and
//   writes codes and scales directly in tile order.  Arithmetic mirrors native/host/quant_core.cpp operation
//   by operation (no fused multiply-add) so that CPU- and GPU-quantized weights are bit-identical for the
//   integer formats.
// * dequantize: the reference's `xe_linear.dequant` (QLoRA backward, :534-538) and
//   `xe_linear.dequantize_rows` (quantized embedding rows, embedding.py:220-222).
#include "common/utils.cuh"
#include <cuda_fp8.h>

namespace {

__constant__ float c_nf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
                                0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
                                0.7229568362236023f, 1.0f};
__constant__ float c_fp4[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
__constant__ float c_nf3[8] = {-1.0f, -0.5350227355957031f, -0.2469314038753510f, 0.0f,
                               0.1833375245332718f, 0.3819939494132996f, 0.6229856610298157f, 1.0f};
__constant__ int c_magic_slot[8] = {0, 4, 1, 5, 2, 6, 3, 7};

__device__ __forceinline__ int pair_row(int r) { return (r & 7) * 2 + (r >> 3); }

__device__ __forceinline__ int nearest_sorted(const float* table, int n, float v) {
  int lo = 0, hi = n - 1;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (table[mid] <= v) lo = mid; else hi = mid;
  }
  return (v - table[lo] <= table[hi] - v) ? lo : hi;
}

// kinds for the 4-bit quantizer
enum { Q4_SYM = 0, Q4_ASYM = 1, Q4_NF4 = 2, Q4_FP4 = 3 };

template <typename T, int KIND>
__global__ void quantize_4bit_kernel(const T* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t cols,
                                     int64_t ld) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t Np = ceil_to_i64(rows, 16), Kp = ceil_to_i64(cols, 128);
  const int64_t groups_per_row = cols / 64;
  const int64_t total = rows * groups_per_row;
  uint8_t* codes = dst;
  uint16_t* scales = reinterpret_cast<uint16_t*>(dst + Np * Kp / 2);
  uint16_t* mins = scales + Np * (Kp / 64);
  const int64_t kt = Kp / 128;
  __shared__ uint8_t sq[8][64];
  uint8_t* myq = sq[threadIdx.x >> 5];
  for (int64_t gi = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5); gi < total;
       gi += (int64_t)gridDim.x * warps_per_block) {
    const int64_t r = gi / groups_per_row, b = gi % groups_per_row;
    const T* p = src + r * ld + b * 64;
    const float v0 = DT<T>::to_f(p[lane]), v1 = DT<T>::to_f(p[lane + 32]);
    float d = 0.f, mn = 0.f;
    if (KIND == Q4_ASYM) {
      float lo = fminf(v0, v1), hi = fmaxf(v0, v1);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      d = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
      mn = lo;
    } else {
      // (|v|, index) arg-max with first-index tie break, as the serial host loop does
      float a0 = fabsf(v0), a1 = fabsf(v1);
      float best = a0;
      int bi = lane;
      if (a1 > a0) { best = a1; bi = lane + 32; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      const float cand = (bi & 32) ? v1 : v0;
      const float maxv = __shfl_sync(0xffffffffu, cand, bi & 31);
      if (KIND == Q4_SYM) d = __fdiv_rn(maxv, -8.0f);
      else if (KIND == Q4_NF4) d = best;
      else d = __fdiv_rn(best, 6.0f);
    }
    const __half dh = __float2half_rn(d);
    uint8_t q0, q1;
    if (KIND == Q4_SYM) {
      const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
      int a = (int)__fadd_rn(__fmul_rn(v0, id), 8.5f), c = (int)__fadd_rn(__fmul_rn(v1, id), 8.5f);
      q0 = (uint8_t)min(15, max(0, a));
      q1 = (uint8_t)min(15, max(0, c));
    } else if (KIND == Q4_ASYM) {
      const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
      int a = (int)__fadd_rn(__fmul_rn(__fsub_rn(v0, mn), id), 0.5f);
      int c = (int)__fadd_rn(__fmul_rn(__fsub_rn(v1, mn), id), 0.5f);
      q0 = (uint8_t)min(15, max(0, a));
      q1 = (uint8_t)min(15, max(0, c));
    } else {
      const float ds = __half2float(dh);
      const float id = ds != 0.f ? __fdiv_rn(1.0f, ds) : 0.f;
      const float s0 = __fmul_rn(v0, id), s1 = __fmul_rn(v1, id);
      if (KIND == Q4_NF4) {
        q0 = (uint8_t)nearest_sorted(c_nf4, 16, s0);
        q1 = (uint8_t)nearest_sorted(c_nf4, 16, s1);
      } else {
        q0 = (uint8_t)(nearest_sorted(c_fp4, 8, fabsf(s0)) | (s0 < 0.f ? 8 : 0));
        q1 = (uint8_t)(nearest_sorted(c_fp4, 8, fabsf(s1)) | (s1 < 0.f ? 8 : 0));
      }
    }
    myq[lane] = q0;
    myq[lane + 32] = q1;
    __syncwarp();
    const int64_t tile = (r / 16) * kt + b / 2;
    const int grp = (int)(b & 1), rr = (int)(r % 16);
    if (lane < 8) {
      uint32_t word = 0;
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int slot = (KIND == Q4_SYM || KIND == Q4_ASYM) ? c_magic_slot[k] : k;
        word |= (uint32_t)myq[8 * lane + k] << (4 * slot);
      }
      const int t = lane >> 1, u = lane & 1;
      *reinterpret_cast<uint32_t*>(codes + tile * 1024 + rr * 64 + t * 16 + grp * 8 + u * 4) = word;
    }
    if (lane == 0) {
      scales[(tile * 2 + grp) * 16 + pair_row(rr)] = __half_as_ushort(dh);
      if (KIND == Q4_ASYM) mins[(tile * 2 + grp) * 16 + pair_row(rr)] = __half_as_ushort(__float2half_rn(mn));
    }
    __syncwarp();
  }
}

// kinds for the 8-bit quantizer
enum { Q8_E4M3 = 0, Q8_E5M2 = 1, Q8_INT8 = 2 };

template <typename T, int KIND>
__global__ void quantize_8bit_kernel(const T* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t cols,
                                     int64_t ld) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t Np = ceil_to_i64(rows, 16), Kp = ceil_to_i64(cols, 128);
  constexpr int QK = KIND == Q8_INT8 ? 64 : 128;
  constexpr int PER = QK / 32;
  const int64_t blocks_per_row = cols / QK;
  const int64_t total = rows * blocks_per_row;
  const int64_t kt = Kp / 64;
  uint8_t* codes = dst;
  for (int64_t gi = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5); gi < total;
       gi += (int64_t)gridDim.x * warps_per_block) {
    const int64_t r = gi / blocks_per_row, b = gi % blocks_per_row;
    const T* p = src + r * ld + b * QK + lane * PER;
    float v[PER];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < PER; i++) { v[i] = DT<T>::to_f(p[i]); amax = fmaxf(amax, fabsf(v[i])); }
    amax = warp_max(amax);
    const int rr = (int)(r % 16);
    if (KIND == Q8_INT8) {
      const float d = __fdiv_rn(amax, 127.0f);
      const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
      uint16_t pk = 0;
#pragma unroll
      for (int i = 0; i < PER; i++) {
        int q = min(127, max(-128, __float2int_rn(__fmul_rn(v[i], id))));
        pk |= (uint16_t)((uint8_t)(int8_t)q) << (8 * i);
      }
      const int64_t tile = (r / 16) * kt + b;
      *reinterpret_cast<uint16_t*>(codes + tile * 1024 + rr * 64 + lane * 2) = pk;
      if (lane == 0) {
        uint16_t* scales = reinterpret_cast<uint16_t*>(dst + Np * Kp);
        scales[tile * 16 + pair_row(rr)] = __half_as_ushort(__float2half_rn(d));
      }
    } else {
      const float fmax = KIND == Q8_E4M3 ? 448.0f : 57344.0f;
      const float d = __fdiv_rn(amax, fmax);
      const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
      uint32_t pk = 0;
#pragma unroll
      for (int i = 0; i < PER; i++) {
        const float s = __fmul_rn(v[i], id);
        uint8_t c = (uint8_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, KIND == Q8_E4M3 ? __NV_E4M3 : __NV_E5M2);
        pk |= (uint32_t)c << (8 * i);
      }
      // 4 consecutive k per lane: k = 4*lane .. 4*lane+3 of the 128-block -> 64-k tile (lane / 16)
      const int64_t tile = (r / 16) * kt + 2 * b + (lane >> 4);
      *reinterpret_cast<uint32_t*>(codes + tile * 1024 + rr * 64 + (lane & 15) * 4) = pk;
      if (lane == 0) {
        float* scales = reinterpret_cast<float*>(dst + Np * Kp);
        scales[((r / 16) * (Kp / 128) + b) * 16 + pair_row(rr)] = d;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// tile layout -> dense [rows, cols] (row-major, leading dimension ld).  One thread per 8 weights.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void dequant_tiled_kernel(const uint8_t* __restrict__ w, T* __restrict__ out, int64_t rows, int64_t cols,
                                     int64_t ld, int wf, const float* __restrict__ lut) {
  const int64_t Np = ceil_to_i64(rows, 16), Kp = ceil_to_i64(cols, 128);
  const int64_t octs_per_row = cols / 8;
  const int64_t total = rows * octs_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / octs_per_row;
    const int64_t k0 = (i % octs_per_row) * 8;
    const int rr = (int)(r % 16);
    float vals[8];
    if (wf == WF_SYM_INT4 || wf == WF_ASYM_INT4 || wf == WF_LUT4) {
      const int64_t kt = Kp / 128;
      const int64_t tile = (r / 16) * kt + k0 / 128;
      const int kin = (int)(k0 % 128);
      const int grp = kin / 64, k64 = kin % 64;
      const int t = k64 / 16, u = (k64 % 16) / 8;
      const uint32_t word = *reinterpret_cast<const uint32_t*>(w + tile * 1024 + rr * 64 + t * 16 + grp * 8 + u * 4);
      const uint16_t* scales = reinterpret_cast<const uint16_t*>(w + Np * Kp / 2);
      const float d = __half2float(__ushort_as_half(scales[(tile * 2 + grp) * 16 + pair_row(rr)]));
      float mn = 0.f;
      if (wf == WF_ASYM_INT4) {
        const uint16_t* mins = scales + Np * (Kp / 64);
        mn = __half2float(__ushort_as_half(mins[(tile * 2 + grp) * 16 + pair_row(rr)]));
      }
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int slot = wf == WF_LUT4 ? k : c_magic_slot[k];
        const int q = (word >> (4 * slot)) & 0xF;
        vals[k] = wf == WF_SYM_INT4 ? (float)(q - 8) * d : (wf == WF_ASYM_INT4 ? (float)q * d + mn : lut[q] * d);
      }
    } else {
      const int64_t kt = Kp / 64;
      const int64_t tile = (r / 16) * kt + k0 / 64;
      const uint2 raw = *reinterpret_cast<const uint2*>(w + tile * 1024 + rr * 64 + (k0 % 64));
      const uint8_t* bytes = reinterpret_cast<const uint8_t*>(&raw);
      float d;
      if (wf == WF_INT8) {
        const uint16_t* scales = reinterpret_cast<const uint16_t*>(w + Np * Kp);
        d = __half2float(__ushort_as_half(scales[tile * 16 + pair_row(rr)]));
      } else {
        const float* scales = reinterpret_cast<const float*>(w + Np * Kp);
        d = scales[((r / 16) * (Kp / 128) + k0 / 128) * 16 + pair_row(rr)];
      }
#pragma unroll
      for (int k = 0; k < 8; k++) {
        float c;
        if (wf == WF_INT8) c = (float)(int8_t)bytes[k];
        else {
          __half_raw h = __nv_cvt_fp8_to_halfraw(bytes[k], wf == WF_FP8_E4M3 ? __NV_E4M3 : __NV_E5M2);
          c = __half2float(*reinterpret_cast<__half*>(&h));
        }
        vals[k] = c * d;
      }
    }
    T* dst = out + r * ld + k0;
    if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      // the thread's 8 outputs as 16-byte stores (one for 16-bit outputs, two for fp32)
      __align__(16) T o8[8];
#pragma unroll
      for (int k = 0; k < 8; k++) o8[k] = DT<T>::from_f(vals[k]);
#pragma unroll
      for (int v = 0; v < (int)(sizeof(T) * 8 / 16); v++)
        reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(o8)[v];
    } else {
#pragma unroll
      for (int k = 0; k < 8; k++) dst[k] = DT<T>::from_f(vals[k]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// canonical block decoders (one thread per block) for the qtypes without a tile layout, and for embedding rows
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float ldh(const uint8_t* p) {
  uint16_t h = (uint16_t)p[0] | ((uint16_t)p[1] << 8);
  return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ float minifloat(int c, int mbits, int bias) {
  int e = c >> mbits, m = c & ((1 << mbits) - 1);
  if (e == 0) return ldexpf((float)m, 1 - bias - mbits);
  return ldexpf((float)((1 << mbits) + m), e - bias - mbits);
}
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int* d, int* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
  else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// qtype ids as in quant/qtypes.py
template <typename T>
__device__ void decode_block(const uint8_t* y, T* x, int qtype) {
  auto put = [&](int i, float v) { x[i] = DT<T>::from_f(v); };
  switch (qtype) {
    case 2: {  // sym_int4
      float d = ldh(y);
      for (int j = 0; j < 32; j++) { put(j, (float)((y[2 + j] & 0xF) - 8) * d); put(j + 32, (float)((y[2 + j] >> 4) - 8) * d); }
    } break;
    case 3: case 34: {  // asym_int4
      float d = ldh(y), m = ldh(y + 2);
      for (int j = 0; j < 32; j++) { put(j, (float)(y[4 + j] & 0xF) * d + m); put(j + 32, (float)(y[4 + j] >> 4) * d + m); }
    } break;
    case 6: {  // sym_int5
      float d = ldh(y);
      uint32_t qh = y[2] | (y[3] << 8) | (y[4] << 16) | ((uint32_t)y[5] << 24);
      for (int j = 0; j < 16; j++) {
        int a = (y[6 + j] & 0xF) | (((qh >> j) & 1) << 4), b = (y[6 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
        put(j, (float)(a - 16) * d); put(j + 16, (float)(b - 16) * d);
      }
    } break;
    case 7: {  // asym_int5
      float d = ldh(y), m = ldh(y + 2);
      uint32_t qh = y[4] | (y[5] << 8) | (y[6] << 16) | ((uint32_t)y[7] << 24);
      for (int j = 0; j < 16; j++) {
        int a = (y[8 + j] & 0xF) | (((qh >> j) & 1) << 4), b = (y[8 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
        put(j, (float)a * d + m); put(j + 16, (float)b * d + m);
      }
    } break;
    case 8: {  // sym_int8
      float d = ldh(y);
      for (int i = 0; i < 64; i++) put(i, (float)(int8_t)y[2 + i] * d);
    } break;
    case 10: case 16: {  // nf4 / fp4
      float d = ldh(y);
      for (int j = 0; j < 32; j++) {
        int a = y[2 + j] & 0xF, b = y[2 + j] >> 4;
        float va = qtype == 10 ? c_nf4[a] : ((a & 8) ? -c_fp4[a & 7] : c_fp4[a & 7]);
        float vb = qtype == 10 ? c_nf4[b] : ((b & 8) ? -c_fp4[b & 7] : c_fp4[b & 7]);
        put(j, va * d); put(j + 32, vb * d);
      }
    } break;
    case 11: {  // nf3
      float d = ldh(y);
      for (int i = 0; i < 64; i++) {
        int bit = 3 * i;
        uint32_t v = y[2 + (bit >> 3)];
        if ((bit >> 3) + 1 < 24) v |= (uint32_t)y[2 + (bit >> 3) + 1] << 8;
        put(i, c_nf3[(v >> (bit & 7)) & 7] * d);
      }
    } break;
    case 29: case 30: {  // fp6 (e3m2)
      float d = ldh(y);
      for (int g = 0; g < 16; g++) {
        uint32_t pack = y[2 + 3 * g] | (y[2 + 3 * g + 1] << 8) | (y[2 + 3 * g + 2] << 16);
        for (int k = 0; k < 4; k++) {
          uint32_t c = (pack >> (6 * k)) & 63;
          float m = minifloat(c & 31, 2, 3) * d;
          put(4 * g + k, (c & 32) ? -m : m);
        }
      }
    } break;
    case 15: case 19: {  // fp8 e4m3 / e5m2, 128-block with fp32 scale
      float d;
      memcpy(&d, y, 4);
      for (int i = 0; i < 128; i++) {
        int c = y[4 + i] & 0x7f;
        float m = (qtype == 15 ? (c < 127 ? minifloat(c, 3, 7) : 0.f) : (c < 124 ? minifloat(c, 2, 15) : 0.f)) * d;
        put(i, (y[4 + i] & 0x80) ? -m : m);
      }
    } break;
    case 27: {  // q4_k
      float d = ldh(y), dmin = ldh(y + 2);
      const uint8_t* sc = y + 4;
      const uint8_t* q = y + 16;
      int is = 0;
      for (int j = 0; j < 256; j += 64) {
        int s, m;
        scale_min_k4(is, sc, &s, &m);
        float d1 = d * s, m1 = dmin * m;
        scale_min_k4(is + 1, sc, &s, &m);
        float d2 = d * s, m2 = dmin * m;
        for (int l = 0; l < 32; l++) { put(j + l, d1 * (q[l] & 0xF) - m1); put(j + 32 + l, d2 * (q[l] >> 4) - m2); }
        q += 32; is += 2;
      }
    } break;
    case 28: {  // q5_k
      float d = ldh(y), dmin = ldh(y + 2);
      const uint8_t* sc = y + 4;
      const uint8_t* qh = y + 16;
      const uint8_t* ql = y + 48;
      int is = 0;
      uint8_t u1 = 1, u2 = 2;
      for (int j = 0; j < 256; j += 64) {
        int s, m;
        scale_min_k4(is, sc, &s, &m);
        float d1 = d * s, m1 = dmin * m;
        scale_min_k4(is + 1, sc, &s, &m);
        float d2 = d * s, m2 = dmin * m;
        for (int l = 0; l < 32; l++) {
          put(j + l, d1 * ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1);
          put(j + 32 + l, d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2);
        }
        ql += 32; is += 2; u1 <<= 2; u2 <<= 2;
      }
    } break;
    case 26: {  // q6_k
      const uint8_t* ql = y;
      const uint8_t* qh = y + 128;
      const int8_t* sc = reinterpret_cast<const int8_t*>(y + 192);
      float d = ldh(y + 208);
      int o = 0;
      for (int n = 0; n < 256; n += 128) {
        for (int l = 0; l < 32; l++) {
          int is = l / 16;
          int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
          int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
          int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
          int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
          put(o + l, d * sc[is] * q1); put(o + l + 32, d * sc[is + 2] * q2);
          put(o + l + 64, d * sc[is + 4] * q3); put(o + l + 96, d * sc[is + 6] * q4);
        }
        o += 128; ql += 64; qh += 32; sc += 8;
      }
    } break;
    case 23: {  // q2_k
      const uint8_t* sc = y;
      const uint8_t* q = y + 16;
      float d = ldh(y + 80), dmin = ldh(y + 82);
      int is = 0, o = 0;
      for (int n = 0; n < 256; n += 128) {
        int shift = 0;
        for (int j = 0; j < 4; j++) {
          uint8_t s = sc[is++];
          float dl = d * (s & 0xF), ml = dmin * (s >> 4);
          for (int l = 0; l < 16; l++) put(o++, dl * ((q[l] >> shift) & 3) - ml);
          s = sc[is++];
          dl = d * (s & 0xF); ml = dmin * (s >> 4);
          for (int l = 0; l < 16; l++) put(o++, dl * ((q[l + 16] >> shift) & 3) - ml);
          shift += 2;
        }
        q += 32;
      }
    } break;
    default: break;
  }
}

template <typename T>
__global__ void dequant_blocks_kernel(const uint8_t* __restrict__ src, T* __restrict__ dst, int64_t nblocks, int qk,
                                      int ts, int qtype) {
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (int64_t)gridDim.x * blockDim.x)
    decode_block<T>(src + b * ts, dst + b * qk, qtype);
}

// rows of a canonical [vocab, dim] table selected by ids -> out [n, dim]
template <typename T>
__global__ void dequant_rows_kernel(const int64_t* __restrict__ ids, const uint8_t* __restrict__ table,
                                    T* __restrict__ out, int64_t n, int dim, int qk, int ts, int qtype) {
  const int bpr = dim / qk;
  const int64_t total = n * bpr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / bpr;
    const int b = (int)(i % bpr);
    decode_block<T>(table + (ids[row] * bpr + b) * ts, out + row * dim + (int64_t)b * qk, qtype);
  }
}

template <typename F>
int by_dtype3(int dtype, F&& f) {
  if (dtype == DT_F16) return (int)f((__half*)nullptr);
  if (dtype == DT_BF16) return (int)f((__nv_bfloat16*)nullptr);
  if (dtype == DT_F32) return (int)f((float*)nullptr);
  return (int)cudaErrorInvalidValue;
}

}  // namespace

// Dense [rows, cols] (leading dimension ld, dtype) -> device tile layout of weight family `wf` (plus `lut_kind`
// for WF_LUT4: 0 = nf4, 1 = fp4).  `dst` must be zero-filled and hold ipex_device_bytes(rows, cols, qtype) bytes.
IPEX_API int ipex_quantize_to_tiles(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld, int wf,
                                    int lut_kind, int dtype, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t work = rows * (cols / 64);
  int blocks = (int)((work + 7) / 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  return by_dtype3(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    const T* p = (const T*)src;
    uint8_t* d = (uint8_t*)dst;
    switch (wf) {
      case WF_SYM_INT4: quantize_4bit_kernel<T, Q4_SYM><<<blocks, 256, 0, s>>>(p, d, rows, cols, ld); break;
      case WF_ASYM_INT4: quantize_4bit_kernel<T, Q4_ASYM><<<blocks, 256, 0, s>>>(p, d, rows, cols, ld); break;
      case WF_LUT4:
        if (lut_kind == 0) quantize_4bit_kernel<T, Q4_NF4><<<blocks, 256, 0, s>>>(p, d, rows, cols, ld);
        else quantize_4bit_kernel<T, Q4_FP4><<<blocks, 256, 0, s>>>(p, d, rows, cols, ld);
        break;
      case WF_FP8_E4M3: quantize_8bit_kernel<T, Q8_E4M3><<<blocks, 256, 0, s>>>(p, d, rows, cols, ld); break;
      case WF_FP8_E5M2: quantize_8bit_kernel<T, Q8_E5M2><<<blocks, 256, 0, s>>>(p, d, rows, cols, ld); break;
      case WF_INT8: quantize_8bit_kernel<T, Q8_INT8><<<blocks, 256, 0, s>>>(p, d, rows, cols, ld); break;
      default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
  });
}

IPEX_API int ipex_dequantize_tiles(const void* w, void* out, int64_t rows, int64_t cols, int64_t ld, int wf,
                                   const float* lut, int dtype, void* stream) {
  const int64_t work = rows * (cols / 8);
  int blocks = (int)((work + 255) / 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (blocks < 1) blocks = 1;
  return by_dtype3(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    dequant_tiled_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)w, (T*)out, rows, cols, ld, wf,
                                                                      lut);
    return cudaGetLastError();
  });
}

IPEX_API int ipex_dequantize_blocks(const void* src, void* dst, int64_t nblocks, int qk, int ts, int qtype, int dtype,
                                    void* stream) {
  int blocks = (int)((nblocks + 127) / 128);
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (blocks < 1) blocks = 1;
  return by_dtype3(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    dequant_blocks_kernel<T><<<blocks, 128, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (T*)dst, nblocks, qk, ts,
                                                                       qtype);
    return cudaGetLastError();
  });
}

IPEX_API int ipex_dequantize_rows(const void* ids, const void* table, void* out, int64_t n, int dim, int qk, int ts,
                                  int qtype, int dtype, void* stream) {
  const int64_t work = n * (dim / qk);
  int blocks = (int)((work + 127) / 128);
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (blocks < 1) blocks = 1;
  return by_dtype3(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    dequant_rows_kernel<T><<<blocks, 128, 0, (cudaStream_t)stream>>>((const int64_t*)ids, (const uint8_t*)table,
                                                                     (T*)out, n, dim, qk, ts, qtype);
    return cudaGetLastError();
  });
}
