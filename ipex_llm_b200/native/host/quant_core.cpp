// quant_core.cpp — CPU implementation of the low-bit block formats (see quant_core.h).
//
// Canonical block layouts (what save_low_bit serializes), per block of QK weights:
//   sym_int4  (QK 64): [fp16 d][32 B qs]        q = min(15, int(x/d + 8.5)), d = signed_absmax / -8,
//                                               byte j = q[j] | q[j+32] << 4          (ggml q4_0 with QK=64)
//   asym_int4 (QK 64): [fp16 d][fp16 m][32 B]   x ~ q*d + m                           (ggml q4_1 with QK=64)
//   sym_int5  (QK 32): [fp16 d][u32 qh][16 B]   5th bits in qh                        (ggml q5_0)
//   asym_int5 (QK 32): [fp16 d][fp16 m][u32 qh][16 B]                                 (ggml q5_1)
//   sym_int8  (QK 64): [fp16 d][64 x int8]      d = absmax / 127                      (ggml q8_0 with QK=64)
//   nf4       (QK 64): [fp16 absmax][32 B]      nibble = index into the NF4 code book, same nibble order as sym_int4
//   nf3       (QK 64): [fp16 absmax][24 B]      3-bit indices, code i at bit 3*i
//   fp4       (QK 64): [fp16 d][32 B]           e2m1 codes, d = absmax / 6
//   fp6       (QK 64): [fp16 d][48 B]           e3m2 codes (bias 3, max 28), 4 codes per 3 bytes
//   fp8_e4m3  (QK 128): [fp32 d][128 B]         d = absmax / 448
//   fp8_e5m2  (QK 128): [fp32 d][128 B]         d = absmax / 57344
//   q4_k / q5_k / q6_k / q2_k (QK 256): the ggml k-quant super-blocks
// The first five are bit-compatible with what is recoverable from the reference's
// python/llm/src/ipex_llm/utils/convert_chatglm.py:88-172; the others are defined here.
#include "quant_core.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

namespace {

// ----------------------------------------------------------------------------------------------
// fp16 <-> fp32 (bit exact, round-to-nearest-even)
// ----------------------------------------------------------------------------------------------
inline float fp16_to_fp32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { e++; man <<= 1; } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t fp32_to_fp16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t mant = x & 0x007fffffu;
  int32_t exp = (int32_t)((x >> 23) & 0xff);
  if (exp == 255) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0));
  int32_t e = exp - 127 + 15;
  if (e >= 31) return (uint16_t)(sign | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    mant |= 0x00800000u;
    int shift = 14 - e;
    uint32_t half = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half & 1))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)e << 10) | (mant >> 13);
  uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
  return (uint16_t)(sign | half);
}

// Block scales and minima: a value beyond the fp16 range is stored as the largest finite fp16, so such a block clips
// instead of decoding to inf / NaN.
inline void put_f16(uint8_t* p, float v) {
  if (v > 65504.0f) v = 65504.0f;
  else if (v < -65504.0f) v = -65504.0f;
  uint16_t h = fp32_to_fp16(v);
  memcpy(p, &h, 2);
}
inline float get_f16(const uint8_t* p) { uint16_t h; memcpy(&h, p, 2); return fp16_to_fp32(h); }
inline void put_f32(uint8_t* p, float v) { memcpy(p, &v, 4); }
inline float get_f32(const uint8_t* p) { float v; memcpy(&v, p, 4); return v; }

// ----------------------------------------------------------------------------------------------
// small float code books
// ----------------------------------------------------------------------------------------------
const float kNF4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                        -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                        0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
                        0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
                        0.7229568362236023f, 1.0f};
// 8-level normal-float code book (quantiles of N(0,1) normalised to [-1,1], zero included).
const float kNF3[8] = {-1.0f, -0.5350227355957031f, -0.2469314038753510f, 0.0f,
                       0.1833375245332718f, 0.3819939494132996f, 0.6229856610298157f, 1.0f};
// e2m1 magnitudes; code = sign<<3 | idx.
const float kFP4[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

inline int nearest_code(const float* table, int n, float v) {
  // table ascending
  int lo = 0, hi = n - 1;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (table[mid] <= v) lo = mid; else hi = mid;
  }
  return (v - table[lo] <= table[hi] - v) ? lo : hi;
}

// generic tiny-float encode/decode (no inf/nan; saturating), used for fp6 e3m2 and fp8.
template <int EBITS, int MBITS, int BIAS>
struct MiniFloat {
  static constexpr int kCodes = 1 << (EBITS + MBITS);  // magnitudes
  static float decode_mag(int c) {
    int e = c >> MBITS, m = c & ((1 << MBITS) - 1);
    if (e == 0) return std::ldexp((float)m, 1 - BIAS - MBITS);
    return std::ldexp((float)((1 << MBITS) + m), e - BIAS - MBITS);
  }
};

struct Tables {
  float fp6[32];      // e3m2 magnitudes, ascending
  float e4m3[127];    // e4m3 magnitudes 0..0x7e (0x7f is NaN in the OCP format)
  float e5m2[124];    // e5m2 magnitudes 0..0x7b (0x7c.. are inf/nan)
  float e4m3_byte[256], e5m2_byte[256];   // signed value of every code byte (codes without a finite value: 0)
  float fp6_signed[64];                   // signed value of every 6-bit code
  Tables() {
    for (int i = 0; i < 32; i++) fp6[i] = MiniFloat<3, 2, 3>::decode_mag(i);
    for (int i = 0; i < 127; i++) e4m3[i] = MiniFloat<4, 3, 7>::decode_mag(i);
    for (int i = 0; i < 124; i++) e5m2[i] = MiniFloat<5, 2, 15>::decode_mag(i);
    for (int c = 0; c < 64; c++) fp6_signed[c] = (c & 32) ? -fp6[c & 31] : fp6[c & 31];
    for (int b = 0; b < 256; b++) {
      int c = b & 0x7f;
      float m4 = c < 127 ? e4m3[c] : 0.0f, m5 = c < 124 ? e5m2[c] : 0.0f;
      e4m3_byte[b] = (b & 0x80) ? -m4 : m4;
      e5m2_byte[b] = (b & 0x80) ? -m5 : m5;
    }
  }
};
const Tables& tables() { static Tables t; return t; }

inline uint8_t encode_signed(const float* mags, int n, float v) {
  int c = nearest_code(mags, n, std::fabs(v));
  return (uint8_t)c;
}

// ----------------------------------------------------------------------------------------------
// per-qtype geometry
// ----------------------------------------------------------------------------------------------
struct QInfo { int qk; int ts; };

QInfo qinfo(int qtype) {
  switch (qtype) {
    case QT_SYM_INT4: return {64, 34};
    case QT_ASYM_INT4: return {64, 36};
    case QT_WOQ_INT4: return {64, 36};
    case QT_SYM_INT5: return {32, 22};
    case QT_ASYM_INT5: return {32, 24};
    case QT_SYM_INT8: return {64, 66};
    case QT_NF4: return {64, 34};
    case QT_NF3: return {64, 26};
    case QT_FP4: return {64, 34};
    case QT_FP6: return {64, 50};
    case QT_FP6_K: return {64, 50};
    case QT_FP8_E4M3: return {128, 132};
    case QT_FP8_E5M2: return {128, 132};
    case QT_Q2_K: return {256, 84};
    case QT_Q4_K: return {256, 144};
    case QT_Q5_K: return {256, 176};
    case QT_Q6_K: return {256, 210};
    // code-book super-blocks: geometry only; their codecs live in quant/iq_codebooks.py (the grids come from
    // the gguf package at run time), so ipex_qtype_supported() stays 0 for them
    case QT_IQ2_XXS: return {256, 66};
    case QT_IQ2_XS: return {256, 74};
    case QT_IQ1_S: return {256, 50};
    case QT_IQ1_M: return {256, 56};
    // per-output-channel round-to-nearest containers: one code byte (or nibble pair) per weight
    case QT_SYM_INT8_RTN: return {1, 1};
    case QT_SYM_INT4_RTN: return {2, 1};
    case QT_ASYM_INT4_RTN: return {2, 1};
    default: return {0, 0};
  }
}

// ----------------------------------------------------------------------------------------------
// block quantizers. w = optional importance weights for the block (NULL = uniform).
// ----------------------------------------------------------------------------------------------
inline float wsel(const float* w, int i) { return w ? w[i] : 1.0f; }

void q_sym_int4(const float* x, uint8_t* y, const float* w, bool search, int64_t* hist) {
  const int QK = 64;
  float amax = 0.f, maxv = 0.f;
  for (int i = 0; i < QK; i++) { float a = std::fabs(x[i]); if (a > amax) { amax = a; maxv = x[i]; } }
  float best_d = maxv / -8.0f;
  if ((search || w) && amax > 0) {
    // try a few scales around the default, keep the (weighted) least-squares best
    double best_err = 1e300;
    float base = best_d;
    for (int s = -4; s <= 6; s++) {
      float d = base * (1.0f + 0.03f * (float)s);
      float id = d ? 1.0f / d : 0.f;
      double err = 0;
      for (int i = 0; i < QK; i++) {
        int q = std::min(15, std::max(0, (int)(x[i] * id + 8.5f)));
        float r = (float)(q - 8) * d - x[i];
        err += (double)wsel(w, i) * r * r;
      }
      if (err < best_err) { best_err = err; best_d = d; }
    }
  }
  // as in ggml: codes are computed against the fp32 scale, the stored scale is its fp16 rounding
  put_f16(y, best_d);
  const float d = best_d;
  const float id = d ? 1.0f / d : 0.0f;
  uint8_t q[QK];
  for (int i = 0; i < QK; i++) {
    int v = (int)(x[i] * id + 8.5f);
    q[i] = (uint8_t)std::min(15, std::max(0, v));
    if (hist) hist[q[i]]++;
  }
  for (int j = 0; j < 32; j++) y[2 + j] = (uint8_t)(q[j] | (q[j + 32] << 4));
}

void dq_sym_int4(const uint8_t* y, float* x) {
  float d = get_f16(y);
  for (int j = 0; j < 32; j++) {
    x[j] = (float)((int)(y[2 + j] & 0xF) - 8) * d;
    x[j + 32] = (float)((int)(y[2 + j] >> 4) - 8) * d;
  }
}

void q_asym_int4(const float* x, uint8_t* y, const float* w, bool search, int64_t* hist) {
  const int QK = 64;
  float mn = x[0], mx = x[0];
  for (int i = 1; i < QK; i++) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
  float d = (mx - mn) / 15.0f;
  (void)search; (void)w;
  put_f16(y, d);
  put_f16(y + 2, mn);
  const float ms = mn;
  float id = d ? 1.0f / d : 0.0f;
  uint8_t q[QK];
  for (int i = 0; i < QK; i++) {
    int v = (int)((x[i] - ms) * id + 0.5f);
    q[i] = (uint8_t)std::min(15, std::max(0, v));
    if (hist) hist[q[i]]++;
  }
  for (int j = 0; j < 32; j++) y[4 + j] = (uint8_t)(q[j] | (q[j + 32] << 4));
}

void dq_asym_int4(const uint8_t* y, float* x) {
  float d = get_f16(y), m = get_f16(y + 2);
  for (int j = 0; j < 32; j++) {
    x[j] = (float)(y[4 + j] & 0xF) * d + m;
    x[j + 32] = (float)(y[4 + j] >> 4) * d + m;
  }
}

void q_sym_int5(const float* x, uint8_t* y, const float*, bool, int64_t*) {
  const int QK = 32;
  float amax = 0.f, maxv = 0.f;
  for (int i = 0; i < QK; i++) { float a = std::fabs(x[i]); if (a > amax) { amax = a; maxv = x[i]; } }
  float d = maxv / -16.0f;
  put_f16(y, d);
  float id = d ? 1.0f / d : 0.0f;
  uint32_t qh = 0;
  for (int j = 0; j < 16; j++) {
    int a = std::min(31, std::max(0, (int)(x[j] * id + 16.5f)));
    int b = std::min(31, std::max(0, (int)(x[j + 16] * id + 16.5f)));
    y[6 + j] = (uint8_t)((a & 0xF) | ((b & 0xF) << 4));
    qh |= (uint32_t)((a >> 4) & 1) << j;
    qh |= (uint32_t)((b >> 4) & 1) << (j + 16);
  }
  memcpy(y + 2, &qh, 4);
}

void dq_sym_int5(const uint8_t* y, float* x) {
  float d = get_f16(y);
  uint32_t qh; memcpy(&qh, y + 2, 4);
  for (int j = 0; j < 16; j++) {
    int a = (y[6 + j] & 0xF) | (((qh >> j) & 1) << 4);
    int b = (y[6 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
    x[j] = (float)(a - 16) * d;
    x[j + 16] = (float)(b - 16) * d;
  }
}

void q_asym_int5(const float* x, uint8_t* y, const float*, bool, int64_t*) {
  const int QK = 32;
  float mn = x[0], mx = x[0];
  for (int i = 1; i < QK; i++) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
  put_f16(y, (mx - mn) / 31.0f);
  put_f16(y + 2, mn);
  float d = get_f16(y), m = get_f16(y + 2);
  float id = d ? 1.0f / d : 0.0f;
  uint32_t qh = 0;
  for (int j = 0; j < 16; j++) {
    int a = std::min(31, std::max(0, (int)((x[j] - m) * id + 0.5f)));
    int b = std::min(31, std::max(0, (int)((x[j + 16] - m) * id + 0.5f)));
    y[8 + j] = (uint8_t)((a & 0xF) | ((b & 0xF) << 4));
    qh |= (uint32_t)((a >> 4) & 1) << j;
    qh |= (uint32_t)((b >> 4) & 1) << (j + 16);
  }
  memcpy(y + 4, &qh, 4);
}

void dq_asym_int5(const uint8_t* y, float* x) {
  float d = get_f16(y), m = get_f16(y + 2);
  uint32_t qh; memcpy(&qh, y + 4, 4);
  for (int j = 0; j < 16; j++) {
    int a = (y[8 + j] & 0xF) | (((qh >> j) & 1) << 4);
    int b = (y[8 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
    x[j] = (float)a * d + m;
    x[j + 16] = (float)b * d + m;
  }
}

void q_sym_int8(const float* x, uint8_t* y, const float*, bool, int64_t*) {
  const int QK = 64;
  float amax = 0.f;
  for (int i = 0; i < QK; i++) amax = std::max(amax, std::fabs(x[i]));
  float d = amax / 127.0f;
  put_f16(y, d);
  float id = d ? 1.0f / d : 0.0f;
  for (int i = 0; i < QK; i++) {
    int v = (int)std::nearbyint(x[i] * id);
    ((int8_t*)y)[2 + i] = (int8_t)std::min(127, std::max(-128, v));
  }
}

void dq_sym_int8(const uint8_t* y, float* x) {
  float d = get_f16(y);
  for (int i = 0; i < 64; i++) x[i] = (float)((const int8_t*)y)[2 + i] * d;
}

template <bool NF>
void q_lut4(const float* x, uint8_t* y, const float* w, bool search, int64_t* hist) {
  const int QK = 64;
  (void)w; (void)search;
  float amax = 0.f;
  for (int i = 0; i < QK; i++) amax = std::max(amax, std::fabs(x[i]));
  float d = NF ? amax : amax / 6.0f;
  put_f16(y, d);
  d = get_f16(y);
  float id = d ? 1.0f / d : 0.0f;
  uint8_t q[QK];
  for (int i = 0; i < QK; i++) {
    float v = x[i] * id;
    if (NF) {
      q[i] = (uint8_t)nearest_code(kNF4, 16, v);
    } else {
      int c = nearest_code(kFP4, 8, std::fabs(v));
      q[i] = (uint8_t)(c | (v < 0 ? 8 : 0));
    }
    if (hist) hist[q[i]]++;
  }
  for (int j = 0; j < 32; j++) y[2 + j] = (uint8_t)(q[j] | (q[j + 32] << 4));
}

inline float fp4_value(int c) { float m = kFP4[c & 7]; return (c & 8) ? -m : m; }

// signed value of all 16 codes: the decoders index it instead of branching on the (random) sign bit
struct Fp4Signed {
  float v[16];
  Fp4Signed() { for (int c = 0; c < 16; c++) v[c] = fp4_value(c); }
};
inline const float* fp4_signed() { static Fp4Signed t; return t.v; }

template <bool NF>
void dq_lut4(const uint8_t* y, float* x) {
  float d = get_f16(y);
  const float* lut = NF ? kNF4 : fp4_signed();
  for (int j = 0; j < 32; j++) {
    int a = y[2 + j] & 0xF, b = y[2 + j] >> 4;
    x[j] = lut[a] * d;
    x[j + 32] = lut[b] * d;
  }
}

void q_nf3(const float* x, uint8_t* y, const float*, bool, int64_t*) {
  const int QK = 64;
  float amax = 0.f;
  for (int i = 0; i < QK; i++) amax = std::max(amax, std::fabs(x[i]));
  put_f16(y, amax);
  float d = get_f16(y);
  float id = d ? 1.0f / d : 0.0f;
  memset(y + 2, 0, 24);
  for (int i = 0; i < QK; i++) {
    uint32_t c = (uint32_t)nearest_code(kNF3, 8, x[i] * id);
    int bit = 3 * i;
    y[2 + (bit >> 3)] |= (uint8_t)(c << (bit & 7));
    if ((bit & 7) > 5) y[2 + (bit >> 3) + 1] |= (uint8_t)(c >> (8 - (bit & 7)));
  }
}

void dq_nf3(const uint8_t* y, float* x) {
  float d = get_f16(y);
  for (int i = 0; i < 64; i++) {
    int bit = 3 * i;
    uint32_t v = y[2 + (bit >> 3)];
    if ((bit >> 3) + 1 < 24) v |= (uint32_t)y[2 + (bit >> 3) + 1] << 8;
    x[i] = kNF3[(v >> (bit & 7)) & 7] * d;
  }
}

// fp6: e3m2, codes = sign<<5 | mag(5 bits); four codes per three bytes, little endian bit stream.
void q_fp6(const float* x, uint8_t* y, const float* w, bool search, int64_t*) {
  const int QK = 64;
  const float* mags = tables().fp6;
  float amax = 0.f;
  for (int i = 0; i < QK; i++) amax = std::max(amax, std::fabs(x[i]));
  float best_d = amax / 28.0f;
  if (search && amax > 0) {
    double best_err = 1e300;
    float base = best_d;
    for (int s = 0; s <= 8; s++) {
      float d = fp16_to_fp32(fp32_to_fp16(base * (1.0f - 0.025f * (float)s)));
      float id = d ? 1.0f / d : 0.f;
      double err = 0;
      for (int i = 0; i < QK; i++) {
        float v = x[i] * id;
        float r = mags[nearest_code(mags, 32, std::fabs(v))] * d - std::fabs(x[i]);
        err += (double)wsel(w, i) * r * r;
      }
      if (err < best_err) { best_err = err; best_d = d; }
    }
  }
  put_f16(y, best_d);
  float d = get_f16(y);
  float id = d ? 1.0f / d : 0.0f;
  for (int g = 0; g < 16; g++) {
    uint32_t pack = 0;
    for (int k = 0; k < 4; k++) {
      float v = x[4 * g + k] * id;
      uint32_t c = (uint32_t)nearest_code(mags, 32, std::fabs(v)) | (v < 0 ? 32u : 0u);
      pack |= c << (6 * k);
    }
    y[2 + 3 * g] = (uint8_t)pack;
    y[2 + 3 * g + 1] = (uint8_t)(pack >> 8);
    y[2 + 3 * g + 2] = (uint8_t)(pack >> 16);
  }
}

void dq_fp6(const uint8_t* y, float* x) {
  const float* val = tables().fp6_signed;
  float d = get_f16(y);
  for (int g = 0; g < 16; g++) {
    uint32_t pack = y[2 + 3 * g] | ((uint32_t)y[2 + 3 * g + 1] << 8) | ((uint32_t)y[2 + 3 * g + 2] << 16);
    for (int k = 0; k < 4; k++) x[4 * g + k] = val[(pack >> (6 * k)) & 63] * d;
  }
}

template <bool E4M3>
void q_fp8(const float* x, uint8_t* y, const float* w, bool search, int64_t*) {
  const int QK = 128;
  const float* mags = E4M3 ? tables().e4m3 : tables().e5m2;
  const int ncodes = E4M3 ? 127 : 124;
  const float fmax = E4M3 ? 448.0f : 57344.0f;
  float amax = 0.f;
  for (int i = 0; i < QK; i++) amax = std::max(amax, std::fabs(x[i]));
  float best_d = amax / fmax;
  if (search && E4M3 && amax > 0) {
    double best_err = 1e300;
    float base = best_d;
    for (int s = 0; s <= 6; s++) {
      float d = base * (1.0f - 0.02f * (float)s);
      float id = 1.0f / d;
      double err = 0;
      for (int i = 0; i < QK; i++) {
        float r = mags[nearest_code(mags, ncodes, std::fabs(x[i] * id))] * d - std::fabs(x[i]);
        err += (double)wsel(w, i) * r * r;
      }
      if (err < best_err) { best_err = err; best_d = d; }
    }
  }
  put_f32(y, best_d);
  float id = best_d ? 1.0f / best_d : 0.0f;
  for (int i = 0; i < QK; i++) {
    float v = x[i] * id;
    uint8_t c = encode_signed(mags, ncodes, v);
    y[4 + i] = (uint8_t)(c | (v < 0 ? 0x80 : 0));
  }
}

template <bool E4M3>
void dq_fp8(const uint8_t* y, float* x) {
  // one table look-up per byte: the sign of a weight is random, so a branch on it mispredicts half of the time
  const float* val = E4M3 ? tables().e4m3_byte : tables().e5m2_byte;
  float d = get_f32(y);
  for (int i = 0; i < 128; i++) x[i] = val[y[4 + i]] * d;
}

// ---------------------------- k-quants (ggml super-block layouts) ------------------------------
// Scale and minimum of one k-quant sub-block: codes 0..nmax, value = scale * code + min with min <= 0 (the formats
// store -min as an unsigned multiple of dmin).  Starts from the min / max fit, then tries code grids that are a little
// finer than the range (the largest values clip, the bulk gets smaller steps): for every assignment the scale and
// the minimum are re-fitted by weighted least squares and the pair with the smallest weighted error is kept.
// `w` are importance weights of the elements (NULL = all equal).  Returns the scale, *neg_min = -min.
float fit_scale_min(int n, int nmax, const float* x, const float* w, float* neg_min) {
  float mn = x[0], mx = x[0];
  for (int i = 1; i < n; i++) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
  if (mn > 0) mn = 0;
  if (!(mx > mn)) { *neg_min = -mn; return 0.f; }
  float best_s = (mx - mn) / (float)nmax, best_m = mn;
  double best_err = 0;
  for (int i = 0; i < n; i++) {
    int l = std::min(nmax, std::max(0, (int)std::nearbyint((x[i] - best_m) / best_s)));
    double e = (double)best_s * l + best_m - x[i];
    best_err += wsel(w, i) * e * e;
  }
  int L[64];
  for (int step = 1; step <= 10; step++) {
    float iscale = ((float)nmax + 0.15f * (float)step) / (mx - mn);
    double sw = 0, sl = 0, sl2 = 0, sx = 0, sxl = 0;
    for (int i = 0; i < n; i++) {
      int l = std::min(nmax, std::max(0, (int)std::nearbyint(iscale * (x[i] - mn))));
      L[i] = l;
      double wi = wsel(w, i);
      sw += wi; sl += wi * l; sl2 += wi * l * l; sx += wi * x[i]; sxl += wi * x[i] * l;
    }
    double det = sw * sl2 - sl * sl;
    if (det <= 0) continue;
    double sc = (sw * sxl - sx * sl) / det, m = (sl2 * sx - sl * sxl) / det;
    if (m > 0) { m = 0; sc = sl2 > 0 ? sxl / sl2 : 0; }
    if (sc <= 0) continue;
    double err = 0;
    for (int i = 0; i < n; i++) { double e = sc * L[i] + m - x[i]; err += wsel(w, i) * e * e; }
    if (err < best_err) { best_err = err; best_s = (float)sc; best_m = (float)m; }
  }
  *neg_min = -best_m;
  return best_s;
}

// q4_k: [fp16 d][fp16 dmin][12 B scales/mins 6-bit][128 B qs]
inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
  else { *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

inline void set_scale_min_k4(int j, uint8_t* q, uint8_t ls, uint8_t lm) {
  if (j < 4) { q[j] = (uint8_t)((q[j] & 0xC0) | ls); q[j + 4] = (uint8_t)((q[j + 4] & 0xC0) | lm); }
  else {
    q[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
    q[j - 4] = (uint8_t)((q[j - 4] & 63) | ((ls >> 4) << 6));
    q[j] = (uint8_t)((q[j] & 63) | ((lm >> 4) << 6));
  }
}

void dq_q4_k(const uint8_t* y, float* x) {
  float d = get_f16(y), dmin = get_f16(y + 2);
  const uint8_t* sc = y + 4;
  const uint8_t* q = y + 16;
  int is = 0;
  for (int j = 0; j < 256; j += 64) {
    uint8_t s, m;
    get_scale_min_k4(is + 0, sc, &s, &m);
    float d1 = d * s, m1 = dmin * m;
    get_scale_min_k4(is + 1, sc, &s, &m);
    float d2 = d * s, m2 = dmin * m;
    for (int l = 0; l < 32; l++) x[j + l] = d1 * (q[l] & 0xF) - m1;
    for (int l = 0; l < 32; l++) x[j + 32 + l] = d2 * (q[l] >> 4) - m2;
    q += 32; is += 2;
  }
}

void q_q4_k(const float* x, uint8_t* y, const float* w, bool, int64_t*) {
  float scales[8], mins[8];
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; j++) {
    scales[j] = fit_scale_min(32, 15, x + 32 * j, w ? w + 32 * j : nullptr, &mins[j]);
    max_scale = std::max(max_scale, scales[j]);
    max_min = std::max(max_min, mins[j]);
  }
  float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
  float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
  memset(y + 4, 0, 12);
  for (int j = 0; j < 8; j++) {
    uint8_t ls = (uint8_t)std::min(63, (int)std::nearbyint(inv_scale * scales[j]));
    uint8_t lm = (uint8_t)std::min(63, (int)std::nearbyint(inv_min * mins[j]));
    set_scale_min_k4(j, y + 4, ls, lm);
  }
  put_f16(y, max_scale / 63.f);
  put_f16(y + 2, max_min / 63.f);
  float d = get_f16(y), dmin = get_f16(y + 2);
  uint8_t L[256];
  for (int j = 0; j < 8; j++) {
    uint8_t s, m;
    get_scale_min_k4(j, y + 4, &s, &m);
    float dd = d * s, dm = dmin * m;
    for (int l = 0; l < 32; l++) {
      int v = dd ? (int)std::nearbyint((x[32 * j + l] + dm) / dd) : 0;
      L[32 * j + l] = (uint8_t)std::min(15, std::max(0, v));
    }
  }
  uint8_t* q = y + 16;
  for (int j = 0; j < 256; j += 64) {
    for (int l = 0; l < 32; l++) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
    q += 32;
  }
}

// q5_k: [fp16 d][fp16 dmin][12 B scales][32 B qh][128 B qs]
void dq_q5_k(const uint8_t* y, float* x) {
  float d = get_f16(y), dmin = get_f16(y + 2);
  const uint8_t* sc = y + 4;
  const uint8_t* qh = y + 16;
  const uint8_t* ql = y + 48;
  int is = 0;
  uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 256; j += 64) {
    uint8_t s, m;
    get_scale_min_k4(is + 0, sc, &s, &m);
    float d1 = d * s, m1 = dmin * m;
    get_scale_min_k4(is + 1, sc, &s, &m);
    float d2 = d * s, m2 = dmin * m;
    for (int l = 0; l < 32; l++) x[j + l] = d1 * ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
    for (int l = 0; l < 32; l++) x[j + 32 + l] = d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
    ql += 32; is += 2; u1 <<= 2; u2 <<= 2;
  }
}

void q_q5_k(const float* x, uint8_t* y, const float* w, bool, int64_t*) {
  float scales[8], mins[8];
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; j++) {
    scales[j] = fit_scale_min(32, 31, x + 32 * j, w ? w + 32 * j : nullptr, &mins[j]);
    max_scale = std::max(max_scale, scales[j]);
    max_min = std::max(max_min, mins[j]);
  }
  float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
  float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
  memset(y + 4, 0, 12);
  for (int j = 0; j < 8; j++) {
    uint8_t ls = (uint8_t)std::min(63, (int)std::nearbyint(inv_scale * scales[j]));
    uint8_t lm = (uint8_t)std::min(63, (int)std::nearbyint(inv_min * mins[j]));
    set_scale_min_k4(j, y + 4, ls, lm);
  }
  put_f16(y, max_scale / 63.f);
  put_f16(y + 2, max_min / 63.f);
  float d = get_f16(y), dmin = get_f16(y + 2);
  uint8_t L[256];
  for (int j = 0; j < 8; j++) {
    uint8_t s, m;
    get_scale_min_k4(j, y + 4, &s, &m);
    float dd = d * s, dm = dmin * m;
    for (int l = 0; l < 32; l++) {
      int v = dd ? (int)std::nearbyint((x[32 * j + l] + dm) / dd) : 0;
      L[32 * j + l] = (uint8_t)std::min(31, std::max(0, v));
    }
  }
  uint8_t* qh = y + 16;
  uint8_t* ql = y + 48;
  memset(qh, 0, 32);
  uint8_t m1 = 1, m2 = 2;
  for (int n = 0; n < 256; n += 64) {
    for (int j = 0; j < 32; j++) {
      int l1 = L[n + j], l2 = L[n + j + 32];
      if (l1 > 15) { l1 -= 16; qh[j] |= m1; }
      if (l2 > 15) { l2 -= 16; qh[j] |= m2; }
      ql[j] = (uint8_t)(l1 | (l2 << 4));
    }
    m1 <<= 2; m2 <<= 2; ql += 32;
  }
}

// q6_k: [128 B ql][64 B qh][16 x int8 scales][fp16 d]
void dq_q6_k(const uint8_t* y, float* x) {
  const uint8_t* ql = y;
  const uint8_t* qh = y + 128;
  const int8_t* sc = (const int8_t*)(y + 192);
  float d = get_f16(y + 208);
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; l++) {
      int is = l / 16;
      int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
      int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      x[l] = d * sc[is + 0] * q1;
      x[l + 32] = d * sc[is + 2] * q2;
      x[l + 64] = d * sc[is + 4] * q3;
      x[l + 96] = d * sc[is + 6] * q4;
    }
    x += 128; ql += 64; qh += 32; sc += 8;
  }
}

void q_q6_k(const float* x, uint8_t* y, const float*, bool, int64_t*) {
  float scales[16];
  float max_abs_scale = 0, max_scale = 0;
  for (int ib = 0; ib < 16; ib++) {
    float amax = 0, maxv = 0;
    for (int l = 0; l < 16; l++) { float a = std::fabs(x[16 * ib + l]); if (a > amax) { amax = a; maxv = x[16 * ib + l]; } }
    scales[ib] = maxv / -32.0f;
    if (std::fabs(scales[ib]) > max_abs_scale) { max_abs_scale = std::fabs(scales[ib]); max_scale = scales[ib]; }
  }
  int8_t* sc = (int8_t*)(y + 192);
  if (max_abs_scale == 0) { memset(y, 0, 210); return; }
  float iscale = -128.f / max_scale;
  put_f16(y + 208, 1.0f / iscale);
  float d = get_f16(y + 208);
  uint8_t L[256];
  for (int ib = 0; ib < 16; ib++) {
    sc[ib] = (int8_t)std::min(127, std::max(-128, (int)std::nearbyint(iscale * scales[ib])));
    float dd = d * sc[ib];
    for (int l = 0; l < 16; l++) {
      int v = dd ? (int)std::nearbyint(x[16 * ib + l] / dd) : 0;
      L[16 * ib + l] = (uint8_t)(std::min(31, std::max(-32, v)) + 32);
    }
  }
  uint8_t* ql = y;
  uint8_t* qh = y + 128;
  for (int j = 0; j < 256; j += 128) {
    for (int l = 0; l < 32; l++) {
      uint8_t q1 = L[j + l] & 0xF, q2 = L[j + l + 32] & 0xF, q3 = L[j + l + 64] & 0xF, q4 = L[j + l + 96] & 0xF;
      ql[l] = (uint8_t)(q1 | (q3 << 4));
      ql[l + 32] = (uint8_t)(q2 | (q4 << 4));
      qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) | ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
    }
    ql += 64; qh += 32;
  }
}

// q2_k: [16 B scales(4b scale | 4b min)][64 B qs][fp16 d][fp16 dmin]
void dq_q2_k(const uint8_t* y, float* x) {
  const uint8_t* sc = y;
  const uint8_t* q = y + 16;
  float d = get_f16(y + 80), dmin = get_f16(y + 82);
  int is = 0;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; j++) {
      uint8_t s = sc[is++];
      float dl = d * (s & 0xF), ml = dmin * (s >> 4);
      for (int l = 0; l < 16; l++) *x++ = dl * ((q[l] >> shift) & 3) - ml;
      s = sc[is++];
      dl = d * (s & 0xF); ml = dmin * (s >> 4);
      for (int l = 0; l < 16; l++) *x++ = dl * ((q[l + 16] >> shift) & 3) - ml;
      shift += 2;
    }
    q += 32;
  }
}

void q_q2_k(const float* x, uint8_t* y, const float* w, bool, int64_t*) {
  float scales[16], mins[16];
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 16; j++) {
    scales[j] = fit_scale_min(16, 3, x + 16 * j, w ? w + 16 * j : nullptr, &mins[j]);
    max_scale = std::max(max_scale, scales[j]);
    max_min = std::max(max_min, mins[j]);
  }
  put_f16(y + 80, max_scale / 15.f);
  put_f16(y + 82, max_min / 15.f);
  float d = get_f16(y + 80), dmin = get_f16(y + 82);
  uint8_t L[256];
  for (int j = 0; j < 16; j++) {
    int ls = max_scale > 0 ? std::min(15, (int)std::nearbyint(15.f / max_scale * scales[j])) : 0;
    int lm = max_min > 0 ? std::min(15, (int)std::nearbyint(15.f / max_min * mins[j])) : 0;
    y[j] = (uint8_t)(ls | (lm << 4));
    float dd = d * ls, dm = dmin * lm;
    for (int l = 0; l < 16; l++) {
      int v = dd ? (int)std::nearbyint((x[16 * j + l] + dm) / dd) : 0;
      L[16 * j + l] = (uint8_t)std::min(3, std::max(0, v));
    }
  }
  uint8_t* q = y + 16;
  for (int j = 0; j < 256; j += 128) {
    for (int l = 0; l < 32; l++)
      q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    q += 32;
  }
}

typedef void (*qfn)(const float*, uint8_t*, const float*, bool, int64_t*);
typedef void (*dqfn)(const uint8_t*, float*);

struct Codec { qfn q; dqfn dq; };

Codec codec(int qtype) {
  switch (qtype) {
    case QT_SYM_INT4: return {q_sym_int4, dq_sym_int4};
    case QT_ASYM_INT4: case QT_WOQ_INT4: return {q_asym_int4, dq_asym_int4};
    case QT_SYM_INT5: return {q_sym_int5, dq_sym_int5};
    case QT_ASYM_INT5: return {q_asym_int5, dq_asym_int5};
    case QT_SYM_INT8: return {q_sym_int8, dq_sym_int8};
    case QT_NF4: return {q_lut4<true>, dq_lut4<true>};
    case QT_FP4: return {q_lut4<false>, dq_lut4<false>};
    case QT_NF3: return {q_nf3, dq_nf3};
    case QT_FP6: case QT_FP6_K: return {q_fp6, dq_fp6};
    case QT_FP8_E4M3: return {q_fp8<true>, dq_fp8<true>};
    case QT_FP8_E5M2: return {q_fp8<false>, dq_fp8<false>};
    case QT_Q2_K: return {q_q2_k, dq_q2_k};
    case QT_Q4_K: return {q_q4_k, dq_q4_k};
    case QT_Q5_K: return {q_q5_k, dq_q5_k};
    case QT_Q6_K: return {q_q6_k, dq_q6_k};
    default: return {nullptr, nullptr};
  }
}

inline int64_t ceil_to(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// nibble slot (0..7) inside a 32-bit word for the k-th of 8 consecutive weights.
// "magic" order pairs (w0,w1) in bits [0:4) and [16:20) so that a masked word is directly a pair
// of fp16/bf16 magic-number operands; "natural" order keeps weight k at bit 4k (byte = pair).
inline int nibble_slot(bool magic, int k) {
  static const int kMagic[8] = {0, 4, 1, 5, 2, 6, 3, 7};
  return magic ? kMagic[k] : k;
}

}  // namespace

extern "C" {

int ggml_qk_size(int qtype) { return qinfo(qtype).qk; }
int ggml_type_size(int qtype) { return qinfo(qtype).ts; }
int ipex_qtype_supported(int qtype) { return codec(qtype).q != nullptr; }
int ipex_quant_core_version(void) { return 1; }

size_t ggml_quantize_tensor(const float* src, void* dst, int qtype, size_t n, int k, int64_t* hist,
                            int scale_search) {
  QInfo qi = qinfo(qtype);
  Codec c = codec(qtype);
  if (!c.q || qi.qk == 0 || k % qi.qk != 0) return 0;
  int64_t nb = (int64_t)(n / qi.qk);
  uint8_t* out = (uint8_t*)dst;
  if (hist) {
    for (int64_t b = 0; b < nb; b++) c.q(src + b * qi.qk, out + b * qi.ts, nullptr, scale_search != 0, hist);
  } else {
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) c.q(src + b * qi.qk, out + b * qi.ts, nullptr, scale_search != 0, nullptr);
  }
  return (size_t)nb * qi.ts;
}

size_t ggml_quantize_tensor_with_weights(const float* src, void* dst, int qtype, int nrow, int n_per_row,
                                         int64_t* hist, const float* imatrix) {
  QInfo qi = qinfo(qtype);
  Codec c = codec(qtype);
  if (!c.q || qi.qk == 0 || n_per_row % qi.qk != 0) return 0;
  (void)hist;
  int64_t bpr = n_per_row / qi.qk;
  uint8_t* out = (uint8_t*)dst;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < nrow; r++) {
    for (int64_t b = 0; b < bpr; b++) {
      const float* w = imatrix ? imatrix + b * qi.qk : nullptr;
      c.q(src + (r * bpr + b) * qi.qk, out + (r * bpr + b) * qi.ts, w, true, nullptr);
    }
  }
  return (size_t)nrow * bpr * qi.ts;
}

size_t ggml_quantize_tensor_rtn(const float* src, void* dst, float* scale, int qtype, size_t n, int k,
                                int64_t* hist, int scale_search) {
  (void)hist; (void)scale_search;
  int64_t rows = (int64_t)(n / k);
  if (qtype == QT_SYM_INT8_RTN) {
    int8_t* out = (int8_t*)dst;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      const float* x = src + r * k;
      float amax = 0;
      for (int i = 0; i < k; i++) amax = std::max(amax, std::fabs(x[i]));
      float d = amax / 127.f, id = d ? 1.f / d : 0.f;
      scale[r] = d;
      for (int i = 0; i < k; i++) out[r * k + i] = (int8_t)std::min(127, std::max(-127, (int)std::nearbyint(x[i] * id)));
    }
    return (size_t)rows * k;
  }
  if (qtype == QT_SYM_INT4_RTN || qtype == QT_ASYM_INT4_RTN) {
    uint8_t* out = (uint8_t*)dst;
    bool asym = qtype == QT_ASYM_INT4_RTN;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      const float* x = src + r * k;
      float mn = x[0], mx = x[0], amax = 0;
      for (int i = 0; i < k; i++) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); amax = std::max(amax, std::fabs(x[i])); }
      float d, m;
      if (asym) { d = (mx - mn) / 15.f; m = mn; scale[2 * r] = d; scale[2 * r + 1] = m; }
      else { d = amax / 7.f; m = -8.f * d; scale[r] = d; }
      float id = d ? 1.f / d : 0.f;
      for (int i = 0; i < k; i += 2) {
        int a = std::min(15, std::max(0, (int)std::nearbyint((x[i] - m) * id)));
        int b = std::min(15, std::max(0, (int)std::nearbyint((x[i + 1] - m) * id)));
        out[(r * k + i) / 2] = (uint8_t)(a | (b << 4));
      }
    }
    return (size_t)rows * k / 2;
  }
  return 0;
}

void ggml_dequantize(const void* src, float* dst, size_t k, int qtype) {
  QInfo qi = qinfo(qtype);
  Codec c = codec(qtype);
  if (!c.dq) return;
  int64_t nb = (int64_t)(k / qi.qk);
  const uint8_t* in = (const uint8_t*)src;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; b++) c.dq(in + b * qi.ts, dst + b * qi.qk);
}

void ggml_dequantize_q4_0(const void* src, float* dst, size_t k) { ggml_dequantize(src, dst, k, QT_SYM_INT4); }

// ----------------------------------------------------------------------------------------------
// device layout
//
// 4-bit family (sym_int4, asym_int4, nf4, fp4), logical [rows, cols], rows padded to 16 (Np) and
// cols padded to 128 (Kp):
//   plane 0, codes : [Np/16][Kp/128] tiles of 1024 B; tile = [16 rows][64 B]; a row's 64 B are four
//            16-B lane slots t=0..3; slot t = [8 B: k = 16t..16t+15 of the first 64-group]
//            [8 B: the same k range of the second 64-group]; every 32-bit word packs 8 consecutive
//            weights (nibble order: "magic" for the integer types, natural for the code-book types).
//   plane 1, scales: fp16 [Np/16][Kp/128][2 groups][8 row pairs][2] -> index ((tile*2+grp)*16 + (r%8)*2 + r/8)
//   plane 2, mins  : same as scales (asym_int4 only)
// Padding blocks carry scale 0. This is the layout the sm_100a GEMV (mma fragments) and the tcgen05
// GEMM dequant stage read with 16-byte loads.
//
// 8-bit family (fp8_e4m3, fp8_e5m2, sym_int8): rows padded to 16, cols padded to 128:
//   plane 0, codes : [Np/16][Kp/64] tiles of 1024 B; tile = [16 rows][64 B], bytes in k order
//   plane 1, scales: fp8: fp32 [Np/16][Kp/128][16 rows(pair order)]; sym_int8: fp16 [Np/16][Kp/64][16 rows(pair order)]
//
// Every other qtype keeps the canonical bytes on the device (generic kernels decode blocks directly).
// ----------------------------------------------------------------------------------------------
static bool is_4bit_tiled(int q) { return q == QT_SYM_INT4 || q == QT_ASYM_INT4 || q == QT_NF4 || q == QT_FP4; }
static bool is_8bit_tiled(int q) { return q == QT_FP8_E4M3 || q == QT_FP8_E5M2 || q == QT_SYM_INT8; }

size_t ipex_device_bytes(int64_t rows, int64_t cols, int qtype) {
  QInfo qi = qinfo(qtype);
  if (qi.qk == 0) return 0;
  int64_t Np = ceil_to(rows, 16), Kp = ceil_to(cols, 128);
  if (is_4bit_tiled(qtype)) {
    size_t planes = qtype == QT_ASYM_INT4 ? 2 : 1;
    return (size_t)(Np * Kp / 2) + planes * (size_t)(Np * (Kp / 64) * 2);
  }
  if (is_8bit_tiled(qtype)) {
    if (qtype == QT_SYM_INT8) return (size_t)(Np * Kp) + (size_t)(Np * (Kp / 64) * 2);
    return (size_t)(Np * Kp) + (size_t)(Np * (Kp / 128) * 4);
  }
  return (size_t)(rows * cols / qi.qk) * qi.ts;
}

static inline int pair_row(int r) { return (r & 7) * 2 + (r >> 3); }

int ggml_q_format_convet_cpu2xpu(const void* src_, void* dst_, int64_t rows, int64_t cols, int qtype) {
  QInfo qi = qinfo(qtype);
  if (qi.qk == 0 || cols % qi.qk != 0) return -1;
  const uint8_t* src = (const uint8_t*)src_;
  uint8_t* dst = (uint8_t*)dst_;
  size_t total = ipex_device_bytes(rows, cols, qtype);
  int64_t Np = ceil_to(rows, 16), Kp = ceil_to(cols, 128);
  if (is_4bit_tiled(qtype)) {
    const bool asym = qtype == QT_ASYM_INT4;
    const bool magic = qtype == QT_SYM_INT4 || qtype == QT_ASYM_INT4;
    const int hdr = asym ? 4 : 2;
    memset(dst, 0, total);
    if (magic && !asym) {
      // padded sym blocks must decode to 0 even before the zero scale is applied
      memset(dst, 0x88, (size_t)(Np * Kp / 2));
    }
    uint8_t* codes = dst;
    uint16_t* scales = (uint16_t*)(dst + Np * Kp / 2);
    uint16_t* mins = scales + Np * (Kp / 64);
    int64_t kt = Kp / 128;
    int64_t bpr = cols / 64;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      for (int64_t b = 0; b < bpr; b++) {
        const uint8_t* blk = src + (r * bpr + b) * qi.ts;
        int64_t tile = (r / 16) * kt + b / 2;
        int grp = (int)(b & 1);
        int rr = (int)(r % 16);
        uint16_t d; memcpy(&d, blk, 2);
        scales[(tile * 2 + grp) * 16 + pair_row(rr)] = d;
        if (asym) { uint16_t m; memcpy(&m, blk + 2, 2); mins[(tile * 2 + grp) * 16 + pair_row(rr)] = m; }
        const uint8_t* qs = blk + hdr;
        uint8_t* row = codes + tile * 1024 + rr * 64;
        for (int t = 0; t < 4; t++) {
          for (int u = 0; u < 2; u++) {
            uint32_t word = 0;
            for (int k = 0; k < 8; k++) {
              int kk = 16 * t + 8 * u + k;  // weight index inside the 64-group
              uint32_t q = kk < 32 ? (qs[kk] & 0xFu) : (uint32_t)(qs[kk - 32] >> 4);
              word |= q << (4 * nibble_slot(magic, k));
            }
            memcpy(row + t * 16 + grp * 8 + u * 4, &word, 4);
          }
        }
      }
    }
    return 0;
  }
  if (is_8bit_tiled(qtype)) {
    memset(dst, 0, total);
    uint8_t* codes = dst;
    int64_t kt = Kp / 64;
    const bool i8 = qtype == QT_SYM_INT8;
    int64_t bpr = cols / qi.qk;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      int rr = (int)(r % 16);
      for (int64_t b = 0; b < bpr; b++) {
        const uint8_t* blk = src + (r * bpr + b) * qi.ts;
        if (i8) {
          uint16_t* scales = (uint16_t*)(dst + Np * Kp);
          memcpy(&scales[((r / 16) * kt + b) * 16 + pair_row(rr)], blk, 2);
          memcpy(codes + ((r / 16) * kt + b) * 1024 + rr * 64, blk + 2, 64);
        } else {
          float* scales = (float*)(dst + Np * Kp);
          memcpy(&scales[((r / 16) * (Kp / 128) + b) * 16 + pair_row(rr)], blk, 4);
          memcpy(codes + ((r / 16) * kt + 2 * b) * 1024 + rr * 64, blk + 4, 64);
          memcpy(codes + ((r / 16) * kt + 2 * b + 1) * 1024 + rr * 64, blk + 68, 64);
        }
      }
    }
    return 0;
  }
  memcpy(dst, src, total);
  return 0;
}

int ggml_q_format_convet_xpu2cpu(const void* src_, void* dst_, int64_t rows, int64_t cols, int qtype) {
  QInfo qi = qinfo(qtype);
  if (qi.qk == 0 || cols % qi.qk != 0) return -1;
  const uint8_t* src = (const uint8_t*)src_;
  uint8_t* dst = (uint8_t*)dst_;
  int64_t Np = ceil_to(rows, 16), Kp = ceil_to(cols, 128);
  if (is_4bit_tiled(qtype)) {
    const bool asym = qtype == QT_ASYM_INT4;
    const bool magic = qtype == QT_SYM_INT4 || qtype == QT_ASYM_INT4;
    const int hdr = asym ? 4 : 2;
    const uint8_t* codes = src;
    const uint16_t* scales = (const uint16_t*)(src + Np * Kp / 2);
    const uint16_t* mins = scales + Np * (Kp / 64);
    int64_t kt = Kp / 128;
    int64_t bpr = cols / 64;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      for (int64_t b = 0; b < bpr; b++) {
        uint8_t* blk = dst + (r * bpr + b) * qi.ts;
        int64_t tile = (r / 16) * kt + b / 2;
        int grp = (int)(b & 1);
        int rr = (int)(r % 16);
        memcpy(blk, &scales[(tile * 2 + grp) * 16 + pair_row(rr)], 2);
        if (asym) memcpy(blk + 2, &mins[(tile * 2 + grp) * 16 + pair_row(rr)], 2);
        uint8_t q[64];
        const uint8_t* row = codes + tile * 1024 + rr * 64;
        for (int t = 0; t < 4; t++)
          for (int u = 0; u < 2; u++) {
            uint32_t word; memcpy(&word, row + t * 16 + grp * 8 + u * 4, 4);
            for (int k = 0; k < 8; k++) q[16 * t + 8 * u + k] = (uint8_t)((word >> (4 * nibble_slot(magic, k))) & 0xF);
          }
        for (int j = 0; j < 32; j++) blk[hdr + j] = (uint8_t)(q[j] | (q[j + 32] << 4));
      }
    }
    return 0;
  }
  if (is_8bit_tiled(qtype)) {
    const uint8_t* codes = src;
    int64_t kt = Kp / 64;
    const bool i8 = qtype == QT_SYM_INT8;
    int64_t bpr = cols / qi.qk;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      int rr = (int)(r % 16);
      for (int64_t b = 0; b < bpr; b++) {
        uint8_t* blk = dst + (r * bpr + b) * qi.ts;
        if (i8) {
          const uint16_t* scales = (const uint16_t*)(src + Np * Kp);
          memcpy(blk, &scales[((r / 16) * kt + b) * 16 + pair_row(rr)], 2);
          memcpy(blk + 2, codes + ((r / 16) * kt + b) * 1024 + rr * 64, 64);
        } else {
          const float* scales = (const float*)(src + Np * Kp);
          memcpy(blk, &scales[((r / 16) * (Kp / 128) + b) * 16 + pair_row(rr)], 4);
          memcpy(blk + 4, codes + ((r / 16) * kt + 2 * b) * 1024 + rr * 64, 64);
          memcpy(blk + 68, codes + ((r / 16) * kt + 2 * b + 1) * 1024 + rr * 64, 64);
        }
      }
    }
    return 0;
  }
  memcpy(dst, src, (size_t)(rows * cols / qi.qk) * qi.ts);
  return 0;
}

void ggml_compute_forward_mul_mat_q_fp32(const int64_t* src0_ne, const void* src0, int qtype,
                                         const int64_t* src1_ne, const float* src1, float* result) {
  const int64_t K = src0_ne[0], N = src0_ne[1], M = src1_ne[1];
  QInfo qi = qinfo(qtype);
  Codec c = codec(qtype);
  if (!c.dq || K % qi.qk != 0) return;
  const int64_t bpr = K / qi.qk;
  const uint8_t* w = (const uint8_t*)src0;
#pragma omp parallel
  {
    std::vector<float> row((size_t)K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; n++) {
      for (int64_t b = 0; b < bpr; b++) c.dq(w + (n * bpr + b) * qi.ts, row.data() + b * qi.qk);
      for (int64_t m = 0; m < M; m++) {
        const float* x = src1 + m * K;
        float acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
        int64_t k = 0;
        for (; k + 4 <= K; k += 4) {
          acc0 += x[k] * row[k]; acc1 += x[k + 1] * row[k + 1];
          acc2 += x[k + 2] * row[k + 2]; acc3 += x[k + 3] * row[k + 3];
        }
        for (; k < K; k++) acc0 += x[k] * row[k];
        result[m * N + n] = (acc0 + acc1) + (acc2 + acc3);
      }
    }
  }
}

double ipex_quantize_mse(const float* src, int qtype, size_t n, int k) {
  QInfo qi = qinfo(qtype);
  Codec c = codec(qtype);
  if (!c.q || k % qi.qk != 0) return -1.0;
  int64_t nb = (int64_t)(n / qi.qk);
  double total = 0;
#pragma omp parallel for reduction(+ : total) schedule(static)
  for (int64_t b = 0; b < nb; b++) {
    uint8_t buf[256];
    float out[256];
    c.q(src + b * qi.qk, buf, nullptr, false, nullptr);
    c.dq(buf, out);
    double e = 0;
    for (int i = 0; i < qi.qk; i++) { double r = (double)out[i] - src[b * qi.qk + i]; e += r * r; }
    total += e;
  }
  return total / (double)n;
}

}  // extern "C"
