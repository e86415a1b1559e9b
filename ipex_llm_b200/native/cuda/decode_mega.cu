// One decode step of a llama-architecture model as ONE persistent kernel (sm_100a).
//
// The reference runs a token through the Hugging Face module tree: per layer an RMSNorm kernel, the qkv low-bit
// linear, rotary, KV quantize/append, sdp, o_proj, a second norm, the fused MLP kernel and down_proj
// (python/llm/src/ipex_llm/transformers/models/llama.py:129-206, models/common.py:145-201, low_bit_linear.py:606-715),
// each a separate launch that starts its weight stream cold.  At batch 1 a B200 streams a 7B int4 layer in ~16 us, so
// launch gaps, cold starts and tails cost more than the work.  Here the whole step is one cooperative launch with
// one CTA per SM:
//   * a producer warp walks the CTA's share of EVERY projection's weight tiles, layer after layer, with
//     cp.async.bulk into one ring of shared-memory stages: the HBM stream never drains between ops, and while the
//     consumers sit in a grid barrier or run the attention the next ops' weights keep landing;
//   * eight consumer warps each own whole stages (8 KB of codes of one 16-row tile): a stage is decoded and
//     multiplied by one warp with the tensor cores (weights are the A operand; symmetric int4 runs on the s8
//     instruction against activations quantised to 15-bit hi/lo pairs that occupy two B columns per token, fp8
//     e4m3 on the f16 instruction), partial tiles meet in shared-memory accumulators and the warp that draws a
//     tile's last ticket applies the epilogue (bias, residual, act(gate) * up, arg-max key of the logits);
//   * attention (rotary, KV append with optional e5m2 storage, split-KV softmax(QK^T)V) runs in the same kernel
//     on the tensor cores with the query heads of a kv head as one MMA dimension;
//   * ops are separated by grid-wide barriers (one arrival counter, bounded spins);
//   * with tensor parallelism the row-parallel projections push their fp32 partial tiles straight into every
//     peer's buffer over NVLink and each CTA reduces the rows it owns once the peers' flags arrive: the all-reduce
//     costs one NVLink latency and no launch; the vocabulary-parallel lm_head exchanges one arg-max key per rank.
// Every wait (mbarrier, ticket, grid barrier, peer flag) is bounded; on expiry the kernel records a code in *err,
// raises the abort word and every role leaves.  Error codes: 31 producer, 32 consumer stage, 33 tile buffer,
// 34 grid barrier, 35 peer flag, 36 arg-max exchange.
#include <cuda_fp8.h>

#include <type_traits>

#include "common/utils.cuh"

namespace {

#ifndef IPEX_MEGA_CW
#define IPEX_MEGA_CW 8
#endif
#ifndef IPEX_MEGA_CPS4
#define IPEX_MEGA_CPS4 8
#endif
constexpr int kCW = IPEX_MEGA_CW;           // consumer warps
constexpr int kCThreads = kCW * 32;
constexpr int kThreads = kCThreads + 32;    // + producer warp
constexpr int kCPS4 = IPEX_MEGA_CPS4;       // 128-k chunks of a 4-bit row tile per stage (8-bit: half as many)
constexpr int kSpin = 1 << 22;             // mbarrier / ticket polls (tens of ns each)
constexpr int kSpinGlobal = 1 << 20;       // polls that cross L2 or NVLink (about a microsecond each)
constexpr int kNB = 8;                      // tile accumulators in flight
constexpr int kStageBytes = kCPS4 * 1088;   // kCPS4 x (1024 + 64) for 4-bit chunks; 8-bit stages are a little smaller
constexpr int kPad = 64;                    // extra bytes per staged int8 activation row (bank spread)
constexpr int kMaxM = 4;                    // sequences per step
constexpr int WFK_I8 = 0, WFK_FP8 = 1;      // weight families of this kernel

struct MegaLayer {
  const uint8_t* w_qkv;
  const uint8_t* w_o;
  const uint8_t* w_gu;
  const uint8_t* w_down;
  const void* ln1;
  const void* ln2;
  const void* b_qkv;
  const void* b_o;
  void* kcache;
  void* vcache;
};

struct MegaArgs {
  const MegaLayer* layers;
  const void* embed;
  const void* final_norm;
  const uint8_t* w_lm;
  const float* cosp;
  const float* sinp;
  long long* tokens;          // [B] in: token ids; out: arg-max of this step
  int* past_len;              // [B] advanced by one at the end
  void* h0;
  void* h1;
  void* qkv;
  void* attn;
  void* act;
  void* logits;
  float* attn_scratch;        // [B*Hkv*nsplit][16][D+2]
  int* attn_counters;         // [B*Hkv] zero between launches
  unsigned long long* amax;   // [B] zero between launches
  unsigned int* barrier;      // [2] zero between launches
  int* abort_word;            // global abort flag (zero between launches)
  int* err;
  long long c_b, c_h, c_s;    // KV cache strides in elements
  int n_layers, B, H, I, Nqkv, Hq, Hkv, D, V, R;
  int ld_logits;
  int nsplit, stages, kv_fp8;
  float eps, norm_offset, scale;
  // tensor parallel (tp_world == 1: unused)
  int tp_rank, tp_world, tp_npad, vocab_offset;
  float* const* tp_bufs;                 // [world] -> rank's partial buffer [2][world][kMaxM][tp_npad] fp32
  int* const* tp_flags;                  // [world] -> rank's flags [2][world][grid]
  unsigned long long* const* tp_keys;    // [world] -> rank's key buffer [world][kMaxM]
  int* const* tp_kflags;                 // [world] -> rank's key flags [world]
  int* tp_epoch;                         // device int, advanced by the kernel
  long long* prof;                       // optional [grid][8] cycle counters (null = off): x staging, stage waits,
                                         // stage math, grid barriers, attention, producer stalls, producer total, all
};

// ---------------------------------------------------------------------------------------------------------------
// small PTX helpers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_s) {
  const uint32_t addr = smem_u32(bar);
  uint32_t done = 0;
  for (int i = 0; i < kSpin; i++) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (i >= 4) {
      __nanosleep(i < 64 ? 20 : 100);
      if ((i & 63) == 0 && *abort_s) return false;
    }
  }
  *abort_s = 1;
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCThreads) : "memory"); }

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_s32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// D = A * B + {c0, c1, c0, c1}: the two accumulator seeds of a token (hi, lo) start rows g and g + 8 alike
__device__ __forceinline__ void mma_s8_seed(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1, int c0, int c1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename CT>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if constexpr (sizeof(CT) == 2 && std::is_same<CT, __nv_bfloat16>::value) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ float act_apply(float g) { return g / (1.0f + __expf(-g)); }

__device__ __forceinline__ uint8_t to_e5m2(float v) {
  v = fminf(fmaxf(v, -57344.f), 57344.f);
  uint16_t h = __half_as_ushort(__float2half_rn(v));
  uint32_t r = (uint32_t)h + 0x7F + ((h >> 8) & 1);
  uint8_t o = (uint8_t)(r >> 8);
  if ((o & 0x7F) > 0x7B) o = (o & 0x80) | 0x7B;
  return o;
}

template <typename CT>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (std::is_same<CT, __nv_bfloat16>::value) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// orderable 64-bit key of (value, index): larger value wins, ties go to the smaller index
__device__ __forceinline__ unsigned long long amax_key(float v, int idx) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)idx);
}

// ---------------------------------------------------------------------------------------------------------------
// shared-memory context
// ---------------------------------------------------------------------------------------------------------------
struct Ctx {
  uint8_t* ring;
  uint64_t* full_bar;
  uint64_t* empty_bar;
  uint8_t* phase;      // x staging (GEMV ops) / attention scratch, aliased
  float* red;          // [kNB][2][128]
  int* red_cnt;        // [kNB]
  int* red_gen;        // [kNB]
  float* scratch;      // [64]
  float* dxs;          // [kMaxM]
  volatile int* abort_s;
  int* bcast;          // [4] small broadcast slots
  int stages;
  long long* prof;     // this CTA's counters or null
};

struct OpInfo {
  const uint8_t* w;
  int N, K, RT, kind;      // kind: 0 qkv, 1 o_proj, 2 gate/up, 3 down, 4 lm_head
  const void* x;
  int ldx;
  const void* norm_w;
  const void* bias;
  const void* residual;
  void* y;
  int ldy;
};

__device__ __forceinline__ OpInfo get_op(const MegaArgs& a, int q) {
  OpInfo o;
  const int L = a.n_layers;
  o.norm_w = nullptr; o.bias = nullptr; o.residual = nullptr; o.RT = 1;
  if (q == 4 * L) {
    o.w = a.w_lm; o.N = a.V; o.K = a.H; o.kind = 4; o.x = a.h0; o.ldx = a.H; o.norm_w = a.final_norm;
    o.y = a.logits; o.ldy = a.ld_logits;
    return o;
  }
  const MegaLayer& ly = a.layers[q >> 2];
  switch (q & 3) {
    case 0:
      o.w = ly.w_qkv; o.N = a.Nqkv; o.K = a.H; o.kind = 0; o.x = a.h0; o.ldx = a.H; o.norm_w = ly.ln1;
      o.bias = ly.b_qkv; o.y = a.qkv; o.ldy = a.Nqkv;
      break;
    case 1:
      o.w = ly.w_o; o.N = a.H; o.K = a.Hq * a.D; o.kind = 1; o.x = a.attn; o.ldx = a.Hq * a.D;
      o.bias = ly.b_o; o.residual = a.h0; o.y = a.h1; o.ldy = a.H;
      break;
    case 2:
      o.w = ly.w_gu; o.N = 2 * a.I; o.K = a.H; o.kind = 2; o.RT = 2; o.x = a.h1; o.ldx = a.H; o.norm_w = ly.ln2;
      o.y = a.act; o.ldy = a.I;
      break;
    default:
      o.w = ly.w_down; o.N = a.H; o.K = a.I; o.kind = 3; o.x = a.act; o.ldx = a.I; o.residual = a.h1; o.y = a.h0;
      o.ldy = a.H;
      break;
  }
  return o;
}

template <int WFK>
struct Geo {
  static constexpr int CB = WFK == WFK_I8 ? 1024 : 2048;   // code bytes per 128-k chunk of a row tile
  static constexpr int CPS = WFK == WFK_I8 ? kCPS4 : kCPS4 / 2;   // chunks per stage
};

// ---------------------------------------------------------------------------------------------------------------
// activation staging
// ---------------------------------------------------------------------------------------------------------------
// int8 path: token m becomes two byte rows (2m: hi, 2m+1: lo) in the octet order (k0,k4,k1,k5 | k2,k6,k3,k7) of the
// masked weight words, a per-token scale and per-(64-group, token) accumulator seeds (-8 sum hi, -8 sum lo).
template <typename T>
__device__ void stage_x_i8(const MegaArgs& a, const OpInfo& op, const Ctx& c, int Kp) {
  const int tid = threadIdx.x;
  const int M = a.B;
  const T* x = reinterpret_cast<const T*>(op.x);
  const T* nw = reinterpret_cast<const T*>(op.norm_w);
  const int nvec = op.K / 8;
  const int groups = Kp / 64;
  const int stride = Kp + kPad;
  int8_t* xq = reinterpret_cast<int8_t*>(c.phase);
  int2* seeds = reinterpret_cast<int2*>(c.phase + (size_t)2 * M * stride);
  for (int i = tid; i < groups * kMaxM; i += kCThreads)
    if ((i & (kMaxM - 1)) >= M) seeds[i] = make_int2(0, 0);
  for (int m = 0; m < M; m++) {
    const T* xr = x + (size_t)m * op.ldx;
    float ss = 0.f, mx = 0.f;
    for (int v = tid; v < nvec; v += kCThreads) {
      const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(xr + v * 8));
      const T* e = reinterpret_cast<const T*>(&raw);
      uint4 wraw = make_uint4(0, 0, 0, 0);
      if (nw != nullptr) wraw = *reinterpret_cast<const uint4*>(nw + v * 8);
      const T* we = reinterpret_cast<const T*>(&wraw);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float f = DT<T>::to_f(e[j]);
        ss += f * f;
        if (nw != nullptr) f *= DT<T>::to_f(we[j]) + a.norm_offset;
        mx = fmaxf(mx, fabsf(f));
      }
    }
    ss = warp_sum(ss);
    mx = warp_max(mx);
    if ((tid & 31) == 0) { c.scratch[tid >> 5] = ss; c.scratch[kCW + (tid >> 5)] = mx; }
    consumer_sync();
    float tot = 0.f, amax = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; w++) { tot += c.scratch[w]; amax = fmaxf(amax, c.scratch[kCW + w]); }
    const float rstd = nw != nullptr ? rsqrtf(tot / (float)op.K + a.eps) : 1.0f;
    amax *= rstd;
    const float dx = amax > 0.f ? amax / 16383.f : 1.0f;
    const float inv = rstd / dx;
    if (tid == 0) c.dxs[m] = dx;
    consumer_sync();
    int8_t* xh = xq + (size_t)(2 * m) * stride;
    int8_t* xl = xq + (size_t)(2 * m + 1) * stride;
    for (int v0 = 0; v0 < Kp / 8; v0 += kCThreads) {
      const int v = v0 + tid;
      int sh = 0, sl = 0;
      if (v < Kp / 8) {
        uint32_t ph[2] = {0, 0}, pl[2] = {0, 0};
        if (v < nvec) {
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(xr + v * 8));
          const T* e = reinterpret_cast<const T*>(&raw);
          uint4 wraw = make_uint4(0, 0, 0, 0);
          if (nw != nullptr) wraw = *reinterpret_cast<const uint4*>(nw + v * 8);
          const T* we = reinterpret_cast<const T*>(&wraw);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            float f = DT<T>::to_f(e[j]);
            if (nw != nullptr) f *= DT<T>::to_f(we[j]) + a.norm_offset;
            int xi = __float2int_rn(f * inv);
            xi = max(-16383, min(16383, xi));
            const int hi = xi >> 7, lo = xi & 127;
            sh += hi;
            sl += lo;
            const int pos = ((j & 2) ? 4 : 0) + ((j & 1) ? 2 : 0) + ((j & 4) ? 1 : 0);
            ph[pos >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (pos & 3));
            pl[pos >> 2] |= (uint32_t)lo << (8 * (pos & 3));
          }
        }
        *reinterpret_cast<uint2*>(xh + v * 8) = make_uint2(ph[0], ph[1]);
        *reinterpret_cast<uint2*>(xl + v * 8) = make_uint2(pl[0], pl[1]);
      }
      // 8 consecutive octets (= 8 consecutive lanes) form a 64-group
      sh += __shfl_xor_sync(0xffffffffu, sh, 1); sl += __shfl_xor_sync(0xffffffffu, sl, 1);
      sh += __shfl_xor_sync(0xffffffffu, sh, 2); sl += __shfl_xor_sync(0xffffffffu, sl, 2);
      sh += __shfl_xor_sync(0xffffffffu, sh, 4); sl += __shfl_xor_sync(0xffffffffu, sl, 4);
      if ((tid & 7) == 0 && v < Kp / 8) seeds[(v >> 3) * kMaxM + m] = make_int2(-8 * sh, -8 * sl);
    }
  }
}

// fp8-weight path: token m becomes two e4m3 byte rows in natural k order (2m: hi = e4m3(v), 2m+1: lo = e4m3(v - hi))
// with v = x / dxs[m]; hi + lo carries about 8 bits of mantissa, and both rows run against the fp8 weight codes on
// the fp8 tensor-core instruction as two B columns of the same MMA.  RMS norm fused, zero padded to Kp.
template <typename T>
__device__ void stage_x_f8(const MegaArgs& a, const OpInfo& op, const Ctx& c, int Kp) {
  const int tid = threadIdx.x;
  const int M = a.B;
  const T* x = reinterpret_cast<const T*>(op.x);
  const T* nw = reinterpret_cast<const T*>(op.norm_w);
  const int nvec = op.K / 8;
  const int stride = Kp + kPad;
  uint8_t* xq = c.phase;
  for (int m = 0; m < M; m++) {
    const T* xr = x + (size_t)m * op.ldx;
    float ss = 0.f, mx = 0.f;
    for (int v = tid; v < nvec; v += kCThreads) {
      const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(xr + v * 8));
      const T* e = reinterpret_cast<const T*>(&raw);
      uint4 wraw = make_uint4(0, 0, 0, 0);
      if (nw != nullptr) wraw = *reinterpret_cast<const uint4*>(nw + v * 8);
      const T* we = reinterpret_cast<const T*>(&wraw);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float f = DT<T>::to_f(e[j]);
        ss += f * f;
        if (nw != nullptr) f *= DT<T>::to_f(we[j]) + a.norm_offset;
        mx = fmaxf(mx, fabsf(f));
      }
    }
    ss = warp_sum(ss);
    mx = warp_max(mx);
    float* sc = c.scratch + (m & 1) * 2 * kCW;
    if ((tid & 31) == 0) { sc[tid >> 5] = ss; sc[kCW + (tid >> 5)] = mx; }
    consumer_sync();
    float tot = 0.f, amax = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; w++) { tot += sc[w]; amax = fmaxf(amax, sc[kCW + w]); }
    const float rstd = nw != nullptr ? rsqrtf(tot / (float)op.K + a.eps) : 1.0f;
    amax *= rstd;
    const float dx = amax > 0.f ? amax / 448.f : 1.0f;
    const float inv = rstd / dx;
    if (tid == 0) c.dxs[m] = dx;
    uint8_t* xh = xq + (size_t)(2 * m) * stride;
    uint8_t* xl = xq + (size_t)(2 * m + 1) * stride;
    for (int v = tid; v < Kp / 8; v += kCThreads) {
      uint32_t ph[2] = {0, 0}, pl[2] = {0, 0};
      if (v < nvec) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(xr + v * 8));
        const T* e = reinterpret_cast<const T*>(&raw);
        uint4 wraw = make_uint4(0, 0, 0, 0);
        if (nw != nullptr) wraw = *reinterpret_cast<const uint4*>(nw + v * 8);
        const T* we = reinterpret_cast<const T*>(&wraw);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          float f0 = DT<T>::to_f(e[j]), f1 = DT<T>::to_f(e[j + 1]);
          if (nw != nullptr) {
            f0 *= DT<T>::to_f(we[j]) + a.norm_offset;
            f1 *= DT<T>::to_f(we[j + 1]) + a.norm_offset;
          }
          f0 *= inv;
          f1 *= inv;
          const __nv_fp8x2_storage_t h = __nv_cvt_float2_to_fp8x2(make_float2(f0, f1), __NV_SATFINITE, __NV_E4M3);
          const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(h, __NV_E4M3);
          const float r0 = f0 - __half2float(__ushort_as_half(hr.x)), r1 = f1 - __half2float(__ushort_as_half(hr.y));
          const __nv_fp8x2_storage_t l = __nv_cvt_float2_to_fp8x2(make_float2(r0, r1), __NV_SATFINITE, __NV_E4M3);
          ph[j >> 2] |= (uint32_t)h << (16 * ((j >> 1) & 1));
          pl[j >> 2] |= (uint32_t)l << (16 * ((j >> 1) & 1));
        }
      }
      *reinterpret_cast<uint2*>(xh + v * 8) = make_uint2(ph[0], ph[1]);
      *reinterpret_cast<uint2*>(xl + v * 8) = make_uint2(pl[0], pl[1]);
    }
  }
}

// Single-pass staging for K <= 8 * kCThreads * kNVMax: every thread keeps its slices of the token row (and of the
// norm weight) in registers, so the row is read from L2 once and the statistics (sum of squares, largest magnitude)
// are reduced while the data waits in registers.  I8: same output as stage_x_i8; otherwise same as stage_x_f16.
constexpr int kNVMax = 6;
template <typename T, bool I8>
__device__ void stage_x_fast(const MegaArgs& a, const OpInfo& op, const Ctx& c, int Kp) {
  const int tid = threadIdx.x;
  const int M = a.B;
  const T* x = reinterpret_cast<const T*>(op.x);
  const T* nw = reinterpret_cast<const T*>(op.norm_w);
  const int nvec = op.K / 8, pvec = Kp / 8;
  const int groups = Kp / 64;
  const int stride = I8 ? Kp + kPad : Kp + 8;
  int8_t* xq = reinterpret_cast<int8_t*>(c.phase);
  int2* seeds = reinterpret_cast<int2*>(c.phase + (size_t)2 * M * (Kp + kPad));
  if (I8) {
    for (int i = tid; i < groups * kMaxM; i += kCThreads)
      if ((i & (kMaxM - 1)) >= M) seeds[i] = make_int2(0, 0);
  }
  uint4 wv[kNVMax];
#pragma unroll
  for (int i = 0; i < kNVMax; i++) {
    const int v = tid + i * kCThreads;
    wv[i] = make_uint4(0, 0, 0, 0);
    if (nw != nullptr && v < nvec) wv[i] = *reinterpret_cast<const uint4*>(nw + v * 8);
  }
  for (int m = 0; m < M; m++) {
    const T* xr = x + (size_t)m * op.ldx;
    uint4 xv[kNVMax];
#pragma unroll
    for (int i = 0; i < kNVMax; i++) {
      const int v = tid + i * kCThreads;
      xv[i] = make_uint4(0, 0, 0, 0);
      if (v < nvec) xv[i] = __ldcg(reinterpret_cast<const uint4*>(xr + v * 8));
    }
    float ss = 0.f, mx = 0.f;
#pragma unroll
    for (int i = 0; i < kNVMax; i++) {
      const T* e = reinterpret_cast<const T*>(&xv[i]);
      const T* we = reinterpret_cast<const T*>(&wv[i]);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float f = DT<T>::to_f(e[j]);
        ss += f * f;
        if (nw != nullptr) f *= DT<T>::to_f(we[j]) + a.norm_offset;
        mx = fmaxf(mx, fabsf(f));
      }
    }
    ss = warp_sum(ss);
    mx = warp_max(mx);
    float* sc = c.scratch + (m & 1) * 2 * kCW;
    if ((tid & 31) == 0) { sc[tid >> 5] = ss; sc[kCW + (tid >> 5)] = mx; }
    consumer_sync();
    float tot = 0.f, amax = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; w++) { tot += sc[w]; amax = fmaxf(amax, sc[kCW + w]); }
    const float rstd = nw != nullptr ? rsqrtf(tot / (float)op.K + a.eps) : 1.0f;
    if constexpr (I8) {
      amax *= rstd;
      const float dx = amax > 0.f ? amax / 16383.f : 1.0f;
      const float inv = rstd / dx;
      if (tid == 0) c.dxs[m] = dx;
      int8_t* xh = xq + (size_t)(2 * m) * stride;
      int8_t* xl = xq + (size_t)(2 * m + 1) * stride;
#pragma unroll
      for (int i = 0; i < kNVMax; i++) {
        const int v = tid + i * kCThreads;
        if (i * kCThreads < pvec) {     // uniform over the CTA: the shuffles below need whole warps
          int sh = 0, sl = 0;
          uint32_t ph[2] = {0, 0}, pl[2] = {0, 0};
          const T* e = reinterpret_cast<const T*>(&xv[i]);
          const T* we = reinterpret_cast<const T*>(&wv[i]);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            float f = DT<T>::to_f(e[j]);
            if (nw != nullptr) f *= DT<T>::to_f(we[j]) + a.norm_offset;
            int xi = __float2int_rn(f * inv);
            xi = max(-16383, min(16383, xi));
            const int hi = xi >> 7, lo = xi & 127;
            sh += hi;
            sl += lo;
            const int pos = ((j & 2) ? 4 : 0) + ((j & 1) ? 2 : 0) + ((j & 4) ? 1 : 0);
            ph[pos >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (pos & 3));
            pl[pos >> 2] |= (uint32_t)lo << (8 * (pos & 3));
          }
          if (v < pvec) {
            *reinterpret_cast<uint2*>(xh + v * 8) = make_uint2(ph[0], ph[1]);
            *reinterpret_cast<uint2*>(xl + v * 8) = make_uint2(pl[0], pl[1]);
          }
          sh += __shfl_xor_sync(0xffffffffu, sh, 1); sl += __shfl_xor_sync(0xffffffffu, sl, 1);
          sh += __shfl_xor_sync(0xffffffffu, sh, 2); sl += __shfl_xor_sync(0xffffffffu, sl, 2);
          sh += __shfl_xor_sync(0xffffffffu, sh, 4); sl += __shfl_xor_sync(0xffffffffu, sl, 4);
          if ((tid & 7) == 0 && v < pvec) seeds[(v >> 3) * kMaxM + m] = make_int2(-8 * sh, -8 * sl);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// one stage (up to CPS chunks of one 16-row tile) by one warp -> acc[4] = (row g, col 2t), (row g, col 2t+1),
// (row g+8, col 2t), (row g+8, col 2t+1) in token columns
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void stage_mma_i8(const uint8_t* st, int nch, int c0, const Ctx& c, int M, int Kp,
                                             float (&acc)[4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr uint32_t kM = 0x0F0F0F0Fu;
  const uint8_t* sc = st + kCPS4 * 1024;
  const int stride = Kp + kPad;
  const bool has_x = g < 2 * M;
  const int8_t* xrow = reinterpret_cast<const int8_t*>(c.phase) + (size_t)g * stride + 16 * t;
  const int2* seeds = reinterpret_cast<const int2*>(c.phase + (size_t)2 * M * stride);
  float a0 = 0.f, a1 = 0.f;   // token t: rows g and g + 8
#pragma unroll 4
  for (int ch = 0; ch < nch; ch++) {
    const int cg = c0 + ch;
    const uint8_t* tp = st + ch * 1024;
    const uint4 qa = *reinterpret_cast<const uint4*>(tp + g * 64 + t * 16);
    const uint4 qb = *reinterpret_cast<const uint4*>(tp + (g + 8) * 64 + t * 16);
    const uint32_t s0 = *reinterpret_cast<const uint32_t*>(sc + ch * 64 + (0 * 16 + 2 * g) * 2);
    const uint32_t s1 = *reinterpret_cast<const uint32_t*>(sc + ch * 64 + (1 * 16 + 2 * g) * 2);
    uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
    if (has_x) {
      xa = *reinterpret_cast<const uint4*>(xrow + cg * 128);
      xb = *reinterpret_cast<const uint4*>(xrow + cg * 128 + 64);
    }
    const int2 sd0 = seeds[(2 * cg) * kMaxM + t];
    const int2 sd1 = seeds[(2 * cg + 1) * kMaxM + t];
    int c0v[4], c1v[4];
    mma_s8_seed(c0v, qa.x & kM, qb.x & kM, (qa.x >> 4) & kM, (qb.x >> 4) & kM, xa.x, xa.y, sd0.x, sd0.y);
    mma_s8_seed(c1v, qa.z & kM, qb.z & kM, (qa.z >> 4) & kM, (qb.z >> 4) & kM, xb.x, xb.y, sd1.x, sd1.y);
    mma_s8(c0v, qa.y & kM, qb.y & kM, (qa.y >> 4) & kM, (qb.y >> 4) & kM, xa.z, xa.w);
    mma_s8(c1v, qa.w & kM, qb.w & kM, (qa.w >> 4) & kM, (qb.w >> 4) & kM, xb.z, xb.w);
    const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
    const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));
    a0 += d0.x * (float)(c0v[0] * 128 + c0v[1]) + d1.x * (float)(c1v[0] * 128 + c1v[1]);
    a1 += d0.y * (float)(c0v[2] * 128 + c0v[3]) + d1.y * (float)(c1v[2] * 128 + c1v[3]);
  }
  // to token columns: lane t holds token t -> column t of the tile (columns 2t, 2t+1 convention of the fp8 path is
  // not used here; the caller reads acc[0] = row g, acc[2] = row g + 8 for token t)
  const float dx = t < M ? c.dxs[t] : 0.f;
  acc[0] = a0 * dx; acc[1] = 0.f; acc[2] = a1 * dx; acc[3] = 0.f;
}

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// fp8 e4m3 weights against the e4m3 (hi, lo) activation rows on the fp8 tensor-core instruction: no conversion of
// the codes at all.  A 128-k chunk is two [16 rows][64 B] tiles in natural k order; a lane's 16 bytes of a weight
// row and the same 16 bytes of an activation row form the operands of two m16n8k32 MMAs (the contraction order of
// the instruction is permuted the same way on both sides, which leaves the sum unchanged).  Columns 2t / 2t+1 of the
// accumulator are the hi / lo parts of token t; the block's fp32 scale is applied once per 128 k.
__device__ __forceinline__ void stage_mma_fp8(const uint8_t* st, int nch, int c0, const Ctx& c, int M, int Kp,
                                              float (&acc)[4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint8_t* sc = st + (kCPS4 / 2) * 2048;
  const int stride = Kp + kPad;
  const bool has_x = g < 2 * M;
  const uint8_t* xrow = c.phase + (size_t)g * stride + 16 * t;
  float a0 = 0.f, a1 = 0.f;
#pragma unroll 2
  for (int ch = 0; ch < nch; ch++) {
    const int cg = c0 + ch;
    const uint8_t* tp = st + ch * 2048 + g * 64 + t * 16;
    const uint4 qa0 = *reinterpret_cast<const uint4*>(tp);
    const uint4 qb0 = *reinterpret_cast<const uint4*>(tp + 512);
    const uint4 qa1 = *reinterpret_cast<const uint4*>(tp + 1024);
    const uint4 qb1 = *reinterpret_cast<const uint4*>(tp + 1536);
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
    if (has_x) {
      x0 = *reinterpret_cast<const uint4*>(xrow + cg * 128);
      x1 = *reinterpret_cast<const uint4*>(xrow + cg * 128 + 64);
    }
    const float2 d = *reinterpret_cast<const float2*>(sc + ch * 64 + 2 * g * 4);
    float c0v[4] = {0.f, 0.f, 0.f, 0.f}, c1v[4] = {0.f, 0.f, 0.f, 0.f};
    mma_e4m3(c0v, qa0.x, qb0.x, qa0.y, qb0.y, x0.x, x0.y);
    mma_e4m3(c1v, qa1.x, qb1.x, qa1.y, qb1.y, x1.x, x1.y);
    mma_e4m3(c0v, qa0.z, qb0.z, qa0.w, qb0.w, x0.z, x0.w);
    mma_e4m3(c1v, qa1.z, qb1.z, qa1.w, qb1.w, x1.z, x1.w);
    a0 += d.x * ((c0v[0] + c0v[1]) + (c1v[0] + c1v[1]));
    a1 += d.y * ((c0v[2] + c0v[3]) + (c1v[2] + c1v[3]));
  }
  const float dx = t < M ? c.dxs[t] : 0.f;
  acc[0] = a0 * dx; acc[1] = 0.f; acc[2] = a1 * dx; acc[3] = 0.f;
}

// ---------------------------------------------------------------------------------------------------------------
// grid barrier (consumer threads only); false on expiry / abort
// ---------------------------------------------------------------------------------------------------------------
__device__ bool grid_barrier(const MegaArgs& a, const Ctx& c, unsigned int& epoch) {
  epoch++;
  long long tb0 = 0;
  if (c.prof != nullptr && threadIdx.x == 0) tb0 = clock64();
  consumer_sync();
  if (threadIdx.x == 0) {
    red_release_gpu_add(a.barrier, 1u);
    const unsigned int target = epoch * gridDim.x;
    bool arrived = false;
    for (int i = 0; i < kSpinGlobal; i++) {
      if (ld_acquire_gpu_u32(a.barrier) >= target) { arrived = true; break; }
      if (i > 16384) __nanosleep(200);
      if ((i & 1023) == 1023 && (*c.abort_s || *(volatile int*)a.abort_word)) break;
    }
    if (!arrived) {
      atomicCAS(a.err, 0, 34);
      *c.abort_s = 1;
      *(volatile int*)a.abort_word = 1;
    }
    if (c.prof != nullptr) c.prof[3] += clock64() - tb0;
  }
  consumer_sync();
  return *c.abort_s == 0;
}

// ---------------------------------------------------------------------------------------------------------------
// GEMV op, consumer side
// ---------------------------------------------------------------------------------------------------------------
struct TpState {
  int epoch_base;   // value of *tp_epoch at kernel start
  int rp_ops;       // row-parallel ops completed in this launch
};

template <typename T>
__device__ __forceinline__ void finalize_tile(const MegaArgs& a, const OpInfo& op, float* rbuf, int grp, int lane,
                                              int tp_parity) {
  const int M = a.B;
  T* y = reinterpret_cast<T*>(op.y);
  if (op.RT == 2) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int i = lane + 32 * j;          // [16 rows][8 cols]
      const int row = i >> 3, col = i & 7;
      float gsum = atomicExch(&rbuf[i], 0.f), usum = atomicExch(&rbuf[128 + i], 0.f);
      const int n = grp * 16 + row;
      if (col < M && n < a.I) y[(size_t)col * op.ldy + n] = DT<T>::from_f(act_apply(gsum) * usum);
    }
    return;
  }
  const bool row_parallel = a.tp_world > 1 && (op.kind == 1 || op.kind == 3);
  unsigned long long best[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = lane + 32 * j;
    const int row = i >> 3, col = i & 7;
    float sv = atomicExch(&rbuf[i], 0.f);
    const int n = grp * 16 + row;
    best[j] = 0ull;
    if (col < M && n < op.N) {
      if (row_parallel) {
        // this rank's fp32 partial goes to slot [parity][tp_rank] of every rank's buffer
        for (int rk = 0; rk < a.tp_world; rk++) {
          float* dst = a.tp_bufs[rk] + ((size_t)(tp_parity * a.tp_world + a.tp_rank) * kMaxM + col) * a.tp_npad;
          dst[n] = sv;
        }
      } else {
        if (op.bias != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(op.bias)[n]);
        if (op.residual != nullptr)
          sv += DT<T>::to_f(__ldcg(reinterpret_cast<const T*>(op.residual) + (size_t)col * a.H + n));
        const T out = DT<T>::from_f(sv);
        y[(size_t)col * op.ldy + n] = out;
        if (op.kind == 4) best[j] = amax_key(DT<T>::to_f(out), n + a.vocab_offset);
      }
    }
  }
  if (op.kind == 4) {
    // column (token) = i & 7 = lane & 7 for every j: reduce over j, then over the lanes that share lane & 7
    unsigned long long b = best[0];
#pragma unroll
    for (int j = 1; j < 4; j++) b = best[j] > b ? best[j] : b;
#pragma unroll
    for (int o = 8; o < 32; o <<= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
      b = other > b ? other : b;
    }
    if (lane < M && b != 0ull) atomicMax(a.amax + lane, b);
  }
}

template <typename T, int WFK>
__device__ bool consume_op(const MegaArgs& a, const OpInfo& op, const Ctx& c, int start, int& it0, int& g0,
                           TpState& tp, const void* next_norm_w, int next_norm_k) {
  constexpr int CPS = Geo<WFK>::CPS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int M = a.B;
  const int Kp = (int)ceil_to_i64(op.K, 128), Np = (int)ceil_to_i64(op.N, 16);
  const int chunks = Kp / 128;
  const int spt = (chunks + CPS - 1) / CPS;
  const int RT = op.RT;
  const int ngroups = (Np / 16) / RT;
  const int grid = gridDim.x;
  const int rel = ((int)blockIdx.x - start + grid) % grid;
  const int my_groups = rel < ngroups ? (ngroups - rel + grid - 1) / grid : 0;
  const int per_group = RT * spt;
  const int nst = my_groups * per_group;
  const bool row_parallel = a.tp_world > 1 && (op.kind == 1 || op.kind == 3);
  const int tp_parity = (tp.epoch_base + tp.rp_ops) & 1;

  const bool prof = c.prof != nullptr && tid == 0;
  long long tp0 = 0;
  if (prof) tp0 = clock64();
  // The NEXT op's norm weight is first touched one op from now, by every CTA at once, right after a grid barrier:
  // ask L2 for it now (a few lines per CTA) so that its staging pass does not open with an HBM miss.
  if (next_norm_w != nullptr) {
    const int lines = (next_norm_k * (int)sizeof(T) + 127) / 128;
    for (int i = blockIdx.x * kCThreads + tid; i < lines; i += gridDim.x * kCThreads)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t*>(next_norm_w) + (size_t)i * 128));
  }
  if constexpr (WFK == WFK_I8) {
    if (Kp <= 8 * kCThreads * kNVMax) stage_x_fast<T, true>(a, op, c, Kp);
    else stage_x_i8<T>(a, op, c, Kp);
  } else {
    stage_x_f8<T>(a, op, c, Kp);
  }
  consumer_sync();
  if (prof) c.prof[0] += clock64() - tp0;

  const int j0 = (warp - (it0 % kCW) + kCW) % kCW;
  for (int j = j0; j < nst; j += kCW) {
    const int gi = j / per_group;
    const int rem = j - gi * per_group;
    const int r = rem / spt, sp = rem - r * spt;
    const int grp = rel + gi * grid;
    const int itj = it0 + j;
    const int slot = itj % c.stages;
    if (prof) tp0 = clock64();
    if (!mbar_wait(&c.full_bar[slot], (uint32_t)(itj / c.stages) & 1u, c.abort_s)) {
      atomicCAS(a.err, 0, 32);
      return false;
    }
    if (prof) { const long long now = clock64(); c.prof[1] += now - tp0; tp0 = now; }
    const int c0 = sp * CPS;
    const int nch = min(CPS, chunks - c0);
    const uint8_t* st = c.ring + (size_t)slot * kStageBytes;
    float acc[4];
    if constexpr (WFK == WFK_I8) stage_mma_i8(st, nch, c0, c, M, Kp, acc);
    else stage_mma_fp8(st, nch, c0, c, M, Kp, acc);
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty_bar[slot]);
    if (prof) { const long long now = clock64(); c.prof[2] += now - tp0; tp0 = now; }

    // ---- partial tile -> shared accumulator of the tile group; last ticket finalises ----
    const int giter = g0 + gi;
    const int b = giter % kNB;
    {
      volatile int* genp = c.red_gen + b;
      bool ready = false;
      for (int i = 0; i < kSpin; i++) {
        if (*genp == giter / kNB) { ready = true; break; }
        __nanosleep(32);
        if ((i & 63) == 63 && *c.abort_s) break;
      }
      if (!ready) {
        atomicCAS(a.err, 0, 33);
        *c.abort_s = 1;
        return false;
      }
    }
    float* rbuf = c.red + (size_t)b * 256;
    float* rp = rbuf + r * 128;
    if (t < M) {      // both weight families leave token t's rows g / g + 8 in acc[0] / acc[2]
      atomicAdd(&rp[g * 8 + t], acc[0]);
      atomicAdd(&rp[(g + 8) * 8 + t], acc[2]);
    }
    __threadfence_block();
    __syncwarp();
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(c.red_cnt + b, 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket == per_group - 1) {
      __threadfence_block();
      finalize_tile<T>(a, op, rbuf, grp, lane, tp_parity);
      __threadfence_block();
      __syncwarp();
      if (lane == 0) {
        c.red_cnt[b] = 0;
        __threadfence_block();
        *(volatile int*)(c.red_gen + b) = giter / kNB + 1;
      }
    }
    if (prof) c.prof[6] += clock64() - tp0;
  }
  it0 += nst;
  g0 += my_groups;

  if (row_parallel) {
    // ---- all-reduce of the rows this CTA owns: flags out, wait for the peers' flags, sum, epilogue ----
    const int epoch = tp.epoch_base + tp.rp_ops + 1;
    consumer_sync();
    if (tid < a.tp_world) {
      __threadfence_system();
      st_release_sys_s32(a.tp_flags[tid] + (size_t)(tp_parity * a.tp_world + a.tp_rank) * grid + blockIdx.x, epoch);
    }
    if (tid < a.tp_world) {
      const int* f = a.tp_flags[a.tp_rank] + (size_t)(tp_parity * a.tp_world + tid) * grid + blockIdx.x;
      bool ok = false;
      for (int i = 0; i < kSpinGlobal; i++) {
        if (ld_acquire_sys_s32(f) >= epoch) { ok = true; break; }
        if (i > 8) __nanosleep(20);
        if ((i & 255) == 255 && (*c.abort_s || *(volatile int*)a.abort_word)) break;
      }
      if (!ok) {
        atomicCAS(a.err, 0, 35);
        *c.abort_s = 1;
        *(volatile int*)a.abort_word = 1;
      }
    }
    consumer_sync();
    if (*c.abort_s) return false;
    T* y = reinterpret_cast<T*>(op.y);
    const float* src = a.tp_bufs[a.tp_rank] + (size_t)tp_parity * a.tp_world * kMaxM * a.tp_npad;
    for (int idx = tid; idx < my_groups * 16 * M; idx += kCThreads) {
      const int gi = idx / (16 * M);
      const int rem = idx - gi * 16 * M;
      const int col = rem / 16, row = rem % 16;
      const int n = (rel + gi * grid) * 16 + row;
      if (n < op.N) {
        float sv = 0.f;
        for (int rk = 0; rk < a.tp_world; rk++) sv += ld_relaxed_sys_f32(src + ((size_t)rk * kMaxM + col) * a.tp_npad + n);
        if (op.bias != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(op.bias)[n]);
        if (op.residual != nullptr)
          sv += DT<T>::to_f(__ldcg(reinterpret_cast<const T*>(op.residual) + (size_t)col * a.H + n));
        y[(size_t)col * op.ldy + n] = DT<T>::from_f(sv);
      }
    }
    tp.rp_ops++;
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------------------
// attention phase: rotary + KV append + split-KV attention of one (sequence, kv head, split) per CTA pass
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float rope_half(const float* cosp, const float* sinp, int pos, int R, int e, float v,
                                           float partner) {
  const int half = R / 2;
  const int j = e < half ? e : e - half;
  const float cs = cosp[(int64_t)pos * half + j], sn = sinp[(int64_t)pos * half + j];
  return e < half ? v * cs - partner * sn : v * cs + partner * sn;
}

template <typename T, bool FP8, int D, bool HI>
__device__ bool attention_phase(const MegaArgs& a, const MegaLayer& ly, const Ctx& c) {
  using CT = typename std::conditional<FP8, __half, T>::type;   // MMA operand type
  constexpr int ROWS = HI ? 16 : 8;
  constexpr int DQ = D / 4;                  // head dims per lane quarter
  constexpr int KSTEPS = D / 16;             // k16 steps of Q K^T
  constexpr int KW = FP8 ? DQ / 4 : DQ / 2;  // 32-bit words of a K row per lane
  constexpr int MB = D / 16;                 // 16-row d blocks of O^T
  constexpr int QS = D + 8;                  // padded row of the staged Q (elements)
  constexpr float kLog2e = 1.4426950408889634f;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = a.Hq / a.Hkv;
  const int nitems = a.B * a.Hkv * a.nsplit;
  const int esz = FP8 ? 1 : 2;

  // shared scratch (aliases the activation staging area)
  CT* Qs = reinterpret_cast<CT*>(c.phase);                                   // [16][QS]
  float* Osm = reinterpret_cast<float*>(c.phase + 16 * QS * sizeof(CT));     // [ROWS][D]
  float* mls = Osm + ROWS * D;                                               // [kCW][16][2]
  float* Msm = mls + kCW * 32;                                               // [16]
  float* Lsm = Msm + 16;                                                     // [16]
  float* wsm = Lsm + 16;                                                     // [16][nsplit] merge weights

  for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
    const int sp = item % a.nsplit;
    const int kvh = (item / a.nsplit) % a.Hkv;
    const int b = item / (a.nsplit * a.Hkv);
    const int past = a.past_len[b];
    const int total = past + 1;
    int chunk = (total + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + 31) & ~31;
    const int t0 = sp * chunk;
    const int t1 = min(total, t0 + chunk);
    const T* qkv = reinterpret_cast<const T*>(a.qkv) + (size_t)b * a.Nqkv;
    uint8_t* kc = reinterpret_cast<uint8_t*>(ly.kcache) + ((int64_t)b * a.c_b + (int64_t)kvh * a.c_h) * esz;
    uint8_t* vc = reinterpret_cast<uint8_t*>(ly.vcache) + ((int64_t)b * a.c_b + (int64_t)kvh * a.c_h) * esz;
    const int64_t rowb = a.c_s * esz;       // bytes between consecutive tokens

    consumer_sync();   // previous item's shared state is dead
    // ---- the split that holds position `past` rotates and appends the new K / V row ----
    if (past >= t0 && past < t0 + chunk) {
      for (int idx = tid; idx < 2 * D; idx += kCThreads) {
        const bool isv = idx >= D;
        const int e = isv ? idx - D : idx;
        const T* src = qkv + (size_t)(a.Hq + (isv ? a.Hkv : 0) + kvh) * D;
        float v = DT<T>::to_f(__ldcg(src + e));
        if (!isv && e < a.R) {
          const int half = a.R / 2;
          const float partner = DT<T>::to_f(__ldcg(src + (e < half ? e + half : e - half)));
          v = rope_half(a.cosp, a.sinp, past, a.R, e, v, partner);
        }
        uint8_t* dstc = (isv ? vc : kc) + (int64_t)past * rowb;
        if constexpr (FP8) dstc[e] = to_e5m2(v);
        else reinterpret_cast<T*>(dstc)[e] = DT<T>::from_f(v);
      }
    }
    // ---- stage rotated Q rows (rounded to the activation type like the stand-alone kernel), zero the rest ----
    for (int idx = tid; idx < ROWS * D; idx += kCThreads) {
      const int r = idx / D, e = idx % D;
      float v = 0.f;
      if (r < G) {
        const T* src = qkv + (size_t)(kvh * G + r) * D;
        v = DT<T>::to_f(__ldcg(src + e));
        if (e < a.R) {
          const int half = a.R / 2;
          const float partner = DT<T>::to_f(__ldcg(src + (e < half ? e + half : e - half)));
          v = rope_half(a.cosp, a.sinp, past, a.R, e, v, partner);
        }
        v = DT<T>::to_f(DT<T>::from_f(v));
      }
      if constexpr (std::is_same<CT, __nv_bfloat16>::value) Qs[r * QS + e] = __float2bfloat16_rn(v);
      else Qs[r * QS + e] = __float2half_rn(v);
    }
    for (int idx = tid; idx < ROWS * D; idx += kCThreads) Osm[idx] = 0.f;
    __threadfence();     // the appended row is read back below through L2 by other warps of this CTA
    consumer_sync();

    // ---- Q fragments: lane (g, t) keeps Q[g][DQ t .. DQ t + DQ) (and row g + 8) ----
    uint32_t qlo[2 * KSTEPS], qhi[HI ? 2 * KSTEPS : 1];
#pragma unroll
    for (int j = 0; j < 2 * KSTEPS; j++) {
      qlo[j] = *reinterpret_cast<const uint32_t*>(Qs + g * QS + DQ * t + 2 * j);
      if constexpr (HI) qhi[j] = *reinterpret_cast<const uint32_t*>(Qs + (g + 8) * QS + DQ * t + 2 * j);
    }

    float o[MB][HI ? 8 : 4];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
#pragma unroll
      for (int i = 0; i < (HI ? 8 : 4); i++) o[mb][i] = 0.f;
    float m_lo = -INFINITY, l_lo = 0.f, m_hi = -INFINITY, l_hi = 0.f;   // rows g and g + 8, log2 domain

    const int nblk = t1 > t0 ? (t1 - t0 + 31) / 32 : 0;
    for (int blk = warp; blk < nblk; blk += kCW) {
      const int base = t0 + 32 * blk;
      // ---- V words of both 16-token steps are requested before the Q K^T math so that one memory latency
      //      covers K and V (fp8 caches; 16-bit caches would need 64 registers and load in place) ----
      constexpr bool kPrefV = FP8 && (!HI || D == 64);
      constexpr int VW = kPrefV ? (D / 32) * 4 : 1;
      uint32_t vw[2][VW];
      if constexpr (kPrefV) {
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
          const int tk = base + 16 * ks + 2 * t;
#pragma unroll
          for (int q4 = 0; q4 < 4; q4++) {
            const int tok = min(tk + (q4 & 1) + (q4 >> 1) * 8, t1 - 1);
            const uint8_t* vp = vc + (int64_t)tok * rowb + 4 * g;
#pragma unroll
            for (int cc = 0; cc < D / 32; cc++)
              vw[ks][cc * 4 + q4] = __ldcg(reinterpret_cast<const uint32_t*>(vp + 32 * cc));
          }
        }
      }
      // ---- S = Q K^T for 32 tokens (4 sub-blocks of 8) ----
      float s[4][4];
#pragma unroll
      for (int sb = 0; sb < 4; sb++) {
        const int tok = min(base + 8 * sb + g, t1 - 1);
        const uint8_t* kp = kc + (int64_t)tok * rowb + (size_t)DQ * t * esz;
        uint32_t kw[KW];
#pragma unroll
        for (int i = 0; i < KW / 4; i++) {
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(kp) + i);
          kw[4 * i] = v.x; kw[4 * i + 1] = v.y; kw[4 * i + 2] = v.z; kw[4 * i + 3] = v.w;
        }
        s[sb][0] = s[sb][1] = s[sb][2] = s[sb][3] = 0.f;
#pragma unroll
        for (int j = 0; j < KSTEPS; j++) {
          uint32_t b0, b1;
          if constexpr (FP8) {
            b0 = __byte_perm(kw[j], 0, 0x1404);
            b1 = __byte_perm(kw[j], 0, 0x3424);
          } else {
            b0 = kw[2 * j];
            b1 = kw[2 * j + 1];
          }
          uint32_t h0 = 0u, h1 = 0u;
          if constexpr (HI) { h0 = qhi[2 * j]; h1 = qhi[2 * j + 1]; }
          mma_16816<CT>(s[sb], qlo[2 * j], h0, qlo[2 * j + 1], h1, b0, b1);
        }
      }
      // ---- scale, mask, online softmax (log2 domain) ----
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int sb = 0; sb < 4; sb++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const bool valid = base + 8 * sb + 2 * t + e < t1;
          s[sb][e] = valid ? s[sb][e] * (a.scale * kLog2e) : -INFINITY;
          s[sb][2 + e] = valid ? s[sb][2 + e] * (a.scale * kLog2e) : -INFINITY;
          mx_lo = fmaxf(mx_lo, s[sb][e]);
          mx_hi = fmaxf(mx_hi, s[sb][2 + e]);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);   // finite: every block has a valid token
      const float corr_lo = exp2f(m_lo - mn_lo), corr_hi = exp2f(m_hi - mn_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
      for (int sb = 0; sb < 4; sb++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          s[sb][e] = exp2f(s[sb][e] - mn_lo);
          ps_lo += s[sb][e];
          if constexpr (HI) {
            s[sb][2 + e] = exp2f(s[sb][2 + e] - mn_hi);
            ps_hi += s[sb][2 + e];
          }
        }
      }
      l_lo = l_lo * corr_lo + ps_lo;
      l_hi = l_hi * corr_hi + ps_hi;
      // O^T columns of this lane are query rows 2t, 2t+1 (and 8+2t, 9+2t): fetch their correction factors
      {
        const float f0 = __shfl_sync(0xffffffffu, corr_lo, 8 * t);
        const float f1 = __shfl_sync(0xffffffffu, corr_lo, 8 * t + 4);
        float f2 = 1.f, f3 = 1.f;
        if constexpr (HI) {
          f2 = __shfl_sync(0xffffffffu, corr_hi, 8 * t);
          f3 = __shfl_sync(0xffffffffu, corr_hi, 8 * t + 4);
        }
#pragma unroll
        for (int mb = 0; mb < MB; mb++) {
          o[mb][0] *= f0; o[mb][1] *= f1; o[mb][2] *= f0; o[mb][3] *= f1;
          if constexpr (HI) { o[mb][4] *= f2; o[mb][5] *= f3; o[mb][6] *= f2; o[mb][7] *= f3; }
        }
      }
      // ---- O^T += V^T P^T, two k16 steps of 16 tokens ----
#pragma unroll
      for (int ks = 0; ks < 2; ks++) {
        const uint32_t pb0 = pack2<CT>(s[2 * ks][0], s[2 * ks][1]);
        const uint32_t pb1 = pack2<CT>(s[2 * ks + 1][0], s[2 * ks + 1][1]);
        uint32_t ph0 = 0, ph1 = 0;
        if constexpr (HI) {
          ph0 = pack2<CT>(s[2 * ks][2], s[2 * ks][3]);
          ph1 = pack2<CT>(s[2 * ks + 1][2], s[2 * ks + 1][3]);
        }
        const int tk = base + 16 * ks + 2 * t;
        const uint8_t* v0 = vc + (int64_t)min(tk, t1 - 1) * rowb;
        const uint8_t* v1 = vc + (int64_t)min(tk + 1, t1 - 1) * rowb;
        const uint8_t* v2 = vc + (int64_t)min(tk + 8, t1 - 1) * rowb;
        const uint8_t* v3 = vc + (int64_t)min(tk + 9, t1 - 1) * rowb;
        if constexpr (FP8) {
          // word c of a token = bytes d = 32c + 4g + {0,1,2,3}; d block (c, e01): rows g -> d = 32c+4g+e01,
          // rows g+8 -> d = 32c+4g+e01+2
#pragma unroll
          for (int cc = 0; cc < D / 32; cc++) {
            uint32_t w0, w1, w2, w3;
            if constexpr (kPrefV) {
              w0 = vw[ks][cc * 4 + 0]; w1 = vw[ks][cc * 4 + 1]; w2 = vw[ks][cc * 4 + 2]; w3 = vw[ks][cc * 4 + 3];
            } else {
              w0 = __ldcg(reinterpret_cast<const uint32_t*>(v0 + 32 * cc + 4 * g));
              w1 = __ldcg(reinterpret_cast<const uint32_t*>(v1 + 32 * cc + 4 * g));
              w2 = __ldcg(reinterpret_cast<const uint32_t*>(v2 + 32 * cc + 4 * g));
              w3 = __ldcg(reinterpret_cast<const uint32_t*>(v3 + 32 * cc + 4 * g));
            }
            const uint32_t e0 = __byte_perm(w0, 0, 0x2404), e1 = __byte_perm(w1, 0, 0x2404);
            const uint32_t e2 = __byte_perm(w2, 0, 0x2404), e3 = __byte_perm(w3, 0, 0x2404);
            const uint32_t o0 = w0 & 0xFF00FF00u, o1 = w1 & 0xFF00FF00u;
            const uint32_t o2 = w2 & 0xFF00FF00u, o3 = w3 & 0xFF00FF00u;
            // e01 = 0: bytes 0 (row g) and 2 (row g+8) -> even words; e01 = 1: bytes 1 and 3 -> odd words
            {
              const uint32_t a0 = __byte_perm(e0, e1, 0x5410), a1 = __byte_perm(e0, e1, 0x7632);
              const uint32_t a2 = __byte_perm(e2, e3, 0x5410), a3 = __byte_perm(e2, e3, 0x7632);
              float* oc = o[2 * cc];
              mma_16816<CT>(*reinterpret_cast<float(*)[4]>(oc), a0, a1, a2, a3, pb0, pb1);
              if constexpr (HI) mma_16816<CT>(*reinterpret_cast<float(*)[4]>(oc + 4), a0, a1, a2, a3, ph0, ph1);
            }
            {
              const uint32_t a0 = __byte_perm(o0, o1, 0x5410), a1 = __byte_perm(o0, o1, 0x7632);
              const uint32_t a2 = __byte_perm(o2, o3, 0x5410), a3 = __byte_perm(o2, o3, 0x7632);
              float* oc = o[2 * cc + 1];
              mma_16816<CT>(*reinterpret_cast<float(*)[4]>(oc), a0, a1, a2, a3, pb0, pb1);
              if constexpr (HI) mma_16816<CT>(*reinterpret_cast<float(*)[4]>(oc + 4), a0, a1, a2, a3, ph0, ph1);
            }
          }
        } else {
          // word c of a token = elements d = 16c + 2g + {0,1}; d block c: rows g -> d = 16c+2g, rows g+8 -> +1
#pragma unroll
          for (int cc = 0; cc < D / 16; cc++) {
            const uint32_t w0 = __ldcg(reinterpret_cast<const uint32_t*>(v0 + (16 * cc + 2 * g) * 2));
            const uint32_t w1 = __ldcg(reinterpret_cast<const uint32_t*>(v1 + (16 * cc + 2 * g) * 2));
            const uint32_t w2 = __ldcg(reinterpret_cast<const uint32_t*>(v2 + (16 * cc + 2 * g) * 2));
            const uint32_t w3 = __ldcg(reinterpret_cast<const uint32_t*>(v3 + (16 * cc + 2 * g) * 2));
            const uint32_t a0 = __byte_perm(w0, w1, 0x5410), a1 = __byte_perm(w0, w1, 0x7632);
            const uint32_t a2 = __byte_perm(w2, w3, 0x5410), a3 = __byte_perm(w2, w3, 0x7632);
            float* oc = o[cc];
            mma_16816<CT>(*reinterpret_cast<float(*)[4]>(oc), a0, a1, a2, a3, pb0, pb1);
            if constexpr (HI) mma_16816<CT>(*reinterpret_cast<float(*)[4]>(oc + 4), a0, a1, a2, a3, ph0, ph1);
          }
        }
      }
    }

    // ---- merge the warps of this CTA ----
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (t == 0) {
      mls[(warp * 16 + g) * 2] = m_lo;
      mls[(warp * 16 + g) * 2 + 1] = l_lo;
      mls[(warp * 16 + g + 8) * 2] = HI ? m_hi : -INFINITY;
      mls[(warp * 16 + g + 8) * 2 + 1] = HI ? l_hi : 0.f;
    }
    consumer_sync();
    if (tid < 16) {
      float mm = -INFINITY;
      for (int w = 0; w < kCW; w++) mm = fmaxf(mm, mls[(w * 16 + tid) * 2]);
      float ll = 0.f;
      for (int w = 0; w < kCW; w++) {
        const float mw = mls[(w * 16 + tid) * 2];
        if (mw > -INFINITY) ll += mls[(w * 16 + tid) * 2 + 1] * exp2f(mw - mm);
      }
      Msm[tid] = mm;
      Lsm[tid] = ll;
    }
    consumer_sync();
    if (nblk > warp) {
      // this warp's O^T columns are query rows 2t, 2t+1 (and +8)
      float f[HI ? 4 : 2];
#pragma unroll
      for (int i = 0; i < (HI ? 4 : 2); i++) {
        const int row = 2 * t + (i & 1) + (i >> 1) * 8;
        const float mw = mls[(warp * 16 + row) * 2];
        f[i] = mw > -INFINITY ? exp2f(mw - Msm[row]) : 0.f;
      }
#pragma unroll
      for (int mb = 0; mb < MB; mb++) {
        int d_lo, d_hi;   // head dim of fragment rows g and g + 8
        if constexpr (FP8) {
          const int cc = mb >> 1, e01 = mb & 1;
          d_lo = 32 * cc + 4 * g + e01;
          d_hi = d_lo + 2;
        } else {
          d_lo = 16 * mb + 2 * g;
          d_hi = d_lo + 1;
        }
        atomicAdd(&Osm[(2 * t) * D + d_lo], o[mb][0] * f[0]);
        atomicAdd(&Osm[(2 * t + 1) * D + d_lo], o[mb][1] * f[1]);
        atomicAdd(&Osm[(2 * t) * D + d_hi], o[mb][2] * f[0]);
        atomicAdd(&Osm[(2 * t + 1) * D + d_hi], o[mb][3] * f[1]);
        if constexpr (HI) {
          atomicAdd(&Osm[(8 + 2 * t) * D + d_lo], o[mb][4] * f[2]);
          atomicAdd(&Osm[(9 + 2 * t) * D + d_lo], o[mb][5] * f[3]);
          atomicAdd(&Osm[(8 + 2 * t) * D + d_hi], o[mb][6] * f[2]);
          atomicAdd(&Osm[(9 + 2 * t) * D + d_hi], o[mb][7] * f[3]);
        }
      }
    }
    consumer_sync();

    T* outp = reinterpret_cast<T*>(a.attn) + (size_t)b * a.Hq * D + (size_t)kvh * G * D;
    if (a.nsplit == 1) {
      for (int idx = tid; idx < G * D; idx += kCThreads) {
        const int r = idx / D;
        const float ll = Lsm[r];
        outp[idx] = DT<T>::from_f(ll > 0.f ? Osm[idx] / ll : 0.f);
      }
      continue;
    }
    // ---- partial of this split -> scratch; the last split to arrive merges ----
    constexpr int PS = D + 2;
    float* part = a.attn_scratch + ((size_t)(b * a.Hkv + kvh) * a.nsplit) * 16 * PS;
    float* mine = part + (size_t)sp * 16 * PS;
    for (int idx = tid; idx < G * D; idx += kCThreads) {
      const int r = idx / D, e = idx % D;
      mine[r * PS + e] = Osm[idx];
    }
    if (tid < G) {
      mine[tid * PS + D] = Msm[tid];
      mine[tid * PS + D + 1] = Lsm[tid];
    }
    __threadfence();
    consumer_sync();
    if (tid == 0) {
      const int ticket = atomicAdd(a.attn_counters + b * a.Hkv + kvh, 1);
      c.bcast[0] = ticket == a.nsplit - 1;
    }
    consumer_sync();
    if (!c.bcast[0]) continue;
    __threadfence();
    if (tid < G) {
      float mm = -INFINITY;
      for (int s2 = 0; s2 < a.nsplit; s2++) mm = fmaxf(mm, __ldcg(part + ((size_t)s2 * 16 + tid) * PS + D));
      float ll = 0.f;
      for (int s2 = 0; s2 < a.nsplit; s2++) {
        const float ms = __ldcg(part + ((size_t)s2 * 16 + tid) * PS + D);
        const float w = ms > -INFINITY ? exp2f(ms - mm) : 0.f;
        wsm[tid * a.nsplit + s2] = w;
        ll += __ldcg(part + ((size_t)s2 * 16 + tid) * PS + D + 1) * w;
      }
      Lsm[tid] = ll;
    }
    consumer_sync();
    for (int idx = tid; idx < G * D; idx += kCThreads) {
      const int r = idx / D, e = idx % D;
      float av = 0.f;
      for (int s2 = 0; s2 < a.nsplit; s2++) {
        const float w = wsm[r * a.nsplit + s2];
        if (w > 0.f) av += __ldcg(part + ((size_t)s2 * 16 + r) * PS + e) * w;
      }
      const float ll = Lsm[r];
      outp[idx] = DT<T>::from_f(ll > 0.f ? av / ll : 0.f);
    }
    if (tid == 0) a.attn_counters[b * a.Hkv + kvh] = 0;
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------------------------
template <typename T, int WFK, bool FP8KV, int D, bool HI>
__global__ void __launch_bounds__(kThreads, 1) decode_mega_kernel(const __grid_constant__ MegaArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int CB = Geo<WFK>::CB, CPS = Geo<WFK>::CPS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  Ctx c;
  c.stages = a.stages;
  c.ring = smem_raw;
  size_t off = (size_t)a.stages * kStageBytes;
  c.full_bar = reinterpret_cast<uint64_t*>(smem_raw + off);
  c.empty_bar = c.full_bar + a.stages;
  off += (size_t)2 * a.stages * sizeof(uint64_t);
  off = (off + 15) & ~(size_t)15;
  c.red = reinterpret_cast<float*>(smem_raw + off);
  off += (size_t)kNB * 256 * sizeof(float);
  c.red_cnt = reinterpret_cast<int*>(smem_raw + off);
  c.red_gen = c.red_cnt + kNB;
  off += 2 * kNB * sizeof(int);
  c.scratch = reinterpret_cast<float*>(smem_raw + off);
  off += 64 * sizeof(float);
  c.dxs = reinterpret_cast<float*>(smem_raw + off);
  off += 8 * sizeof(float);
  c.abort_s = reinterpret_cast<volatile int*>(smem_raw + off);
  c.bcast = reinterpret_cast<int*>(smem_raw + off) + 1;
  off += 8 * sizeof(int);
  off = (off + 127) & ~(size_t)127;
  c.phase = smem_raw + off;
  c.prof = a.prof != nullptr ? a.prof + (size_t)blockIdx.x * 8 : nullptr;
  const long long t_start = c.prof != nullptr ? clock64() : 0;

  if (tid == 0) {
    for (int s = 0; s < a.stages; s++) {
      mbar_init(&c.full_bar[s], 1);
      mbar_init(&c.empty_bar[s], 1);
    }
    *c.abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int L = a.n_layers;
  const int grid = gridDim.x;

  if (warp == kCW) {
    // ---------------- producer: the weight tiles of every projection, in op order ----------------
    // PL lanes share the work in lock step: one pass of the loop body (index arithmetic, wait for the slot, two bulk
    // copies) issues PL consecutive stages, one per lane, and the lanes meet before the next pass.  Issue order is
    // therefore kept up to a window of PL stages.  That matters: consumer warps own different stages and run ahead
    // of each other, and the parity of an mbarrier phase cannot tell "one use ahead" from "two uses ahead"; with
    // stages issued (almost) in order a consumer can reach use n of a slot only after use n-1 of that slot, issued
    // at least (ring depth - consumer warps) stages earlier, has landed.  PL = 1 for rings too shallow for that.
    const int PL = a.stages >= kCW + 8 ? 4 : 1;
    if (lane < PL) {
      int it0 = 0, start = 0;
      bool ok = true;
      long long stall = 0;
      for (int q = 0; q <= 4 * L && ok; q++) {
        const OpInfo op = get_op(a, q);
        const int Kp = (int)ceil_to_i64(op.K, 128), Np = (int)ceil_to_i64(op.N, 16);
        const int chunks = Kp / 128;
        const int spt = (chunks + CPS - 1) / CPS;
        const int ngroups = (Np / 16) / op.RT;
        const uint8_t* codes = op.w;
        const uint8_t* scales = op.w + (WFK == WFK_I8 ? (size_t)Np * Kp / 2 : (size_t)Np * Kp);
        const int rel = ((int)blockIdx.x - start + grid) % grid;
        const int my_groups = rel < ngroups ? (ngroups - rel + grid - 1) / grid : 0;
        const int per_group = op.RT * spt;
        const int nst = my_groups * per_group;
        for (int base = 0; base < nst && ok; base += PL) {
          const int j = base + lane;
          if (j < nst) {
          const int gi = j / per_group;
          const int rem = j - gi * per_group;
          const int r = rem / spt, sp = rem - r * spt;
          const int tile = (rel + gi * grid) * op.RT + r;
          const int it = it0 + j;
          const int round = it / a.stages;
          const int slot = it - round * a.stages;
          if (round > 0) {
            const long long w0 = c.prof != nullptr ? clock64() : 0;
            if (!mbar_wait(&c.empty_bar[slot], (uint32_t)(round - 1) & 1u, c.abort_s)) {
              atomicCAS(a.err, 0, 31);
              ok = false;
            }
            if (c.prof != nullptr) stall += clock64() - w0;
          }
          if (ok) {
            const int c0 = sp * CPS;
            const int nch = min(CPS, chunks - c0);
            uint8_t* dst = c.ring + (size_t)slot * kStageBytes;
            mbar_expect_tx(&c.full_bar[slot], (uint32_t)(nch * (CB + 64)));
            const size_t chunk_index = (size_t)tile * chunks + c0;
            bulk_g2s(dst, codes + chunk_index * CB, (uint32_t)(nch * CB), &c.full_bar[slot]);
            bulk_g2s(dst + CPS * CB, scales + chunk_index * 64, (uint32_t)(nch * 64), &c.full_bar[slot]);
          }
          }
          ok = __all_sync((1u << PL) - 1u, ok);      // lock step: every lane of the pass is done (or has failed)
        }
        it0 += nst;
        start = (start + ngroups % grid) % grid;
      }
      if (c.prof != nullptr && lane == 0) c.prof[5] += stall;
    }
    return;
  }

  // ---------------- consumers ----------------
  for (int i = tid; i < kNB * 256; i += kCThreads) c.red[i] = 0.f;
  if (tid < 2 * kNB) c.red_cnt[tid] = 0;
  TpState tp;
  tp.epoch_base = a.tp_world > 1 ? *(volatile int*)a.tp_epoch : 0;
  tp.rp_ops = 0;
  unsigned int epoch = 0;
  int it0 = 0, g0 = 0, start = 0;
  bool ok = true;

  // ---- embedding rows -> h0 (each CTA copies a slice) ----
  {
    const int vecs = a.H / 8;
    for (int i = blockIdx.x * kCThreads + tid; i < a.B * vecs; i += grid * kCThreads) {
      const int b = i / vecs, v = i % vecs;
      const long long tok = a.tokens[b];
      const uint4 val = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.embed) + (size_t)tok * a.H + v * 8);
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.h0) + (size_t)b * a.H + v * 8) = val;
    }
  }
  ok = grid_barrier(a, c, epoch);

  for (int q = 0; q <= 4 * L && ok; q++) {
    const OpInfo op = get_op(a, q);
    const void* next_nw = nullptr;
    int next_nk = 0;
    if (q < 4 * L) {
      const OpInfo nx = get_op(a, q + 1);
      next_nw = nx.norm_w;
      next_nk = nx.K;
    }
    ok = consume_op<T, WFK>(a, op, c, start, it0, g0, tp, next_nw, next_nk);
    if (!ok) break;
    {
      const int Np = (int)ceil_to_i64(op.N, 16);
      const int ngroups = (Np / 16) / op.RT;
      start = (start + ngroups % grid) % grid;
    }
    ok = grid_barrier(a, c, epoch);
    if (!ok) break;
    if (q < 4 * L && (q & 3) == 0) {
      const long long ta0 = (c.prof != nullptr && tid == 0) ? clock64() : 0;
      ok = attention_phase<T, FP8KV, D, HI>(a, a.layers[q >> 2], c);
      if (c.prof != nullptr && tid == 0) c.prof[4] += clock64() - ta0;
      if (!ok) break;
      ok = grid_barrier(a, c, epoch);
    }
  }

  // ---- arg-max -> tokens, lengths + 1 (CTA 0); leave the counters zero for the next launch ----
  if (ok && blockIdx.x == 0) {
    if (a.tp_world > 1) {
      // vocabulary-parallel lm_head: every rank publishes its best key per sequence to every peer
      const int kepoch = tp.epoch_base + tp.rp_ops + 1;
      if (tid < a.B) {
        const unsigned long long k = atomicAdd(a.amax + tid, 0ull);
        for (int rk = 0; rk < a.tp_world; rk++) a.tp_keys[rk][(size_t)a.tp_rank * kMaxM + tid] = k;
      }
      consumer_sync();
      if (tid < a.tp_world) {
        __threadfence_system();
        st_release_sys_s32(a.tp_kflags[tid] + a.tp_rank, kepoch);
      }
      if (tid < a.tp_world) {
        const int* f = a.tp_kflags[a.tp_rank] + tid;
        bool got = false;
        for (int i = 0; i < kSpinGlobal; i++) {
          if (ld_acquire_sys_s32(f) >= kepoch) { got = true; break; }
          if (i > 8) __nanosleep(20);
        }
        if (!got) { atomicCAS(a.err, 0, 36); *c.abort_s = 1; }
      }
      consumer_sync();
      if (tid < a.B && !*c.abort_s) {
        unsigned long long best = 0ull;
        for (int rk = 0; rk < a.tp_world; rk++) {
          const unsigned long long k = ld_relaxed_sys_u64(a.tp_keys[a.tp_rank] + (size_t)rk * kMaxM + tid);
          best = k > best ? k : best;
        }
        a.tokens[tid] = (long long)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
        a.amax[tid] = 0ull;
        a.past_len[tid] += 1;
      }
      if (tid == 0) *a.tp_epoch = kepoch;
    } else if (tid < a.B) {
      const unsigned long long best = atomicAdd(a.amax + tid, 0ull);
      a.tokens[tid] = (long long)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
      a.amax[tid] = 0ull;
      a.past_len[tid] += 1;
    }
  }
  consumer_sync();
  if (tid == 0) {
    if (c.prof != nullptr) c.prof[7] += clock64() - t_start;
    __threadfence();
    const unsigned int prev = atomicAdd(a.barrier + 1, 1u);
    if (prev == gridDim.x - 1) {
      a.barrier[0] = 0u;
      a.barrier[1] = 0u;
      *(volatile int*)a.abort_word = 0;
      __threadfence();
    }
  }
}

size_t phase_bytes(int wfk, int M, int kp_max, int D, int nsplit) {
  size_t x = wfk == WFK_I8 ? (size_t)2 * M * (kp_max + kPad) + (size_t)(kp_max / 64) * kMaxM * 8
                           : (size_t)2 * M * (kp_max + kPad);
  size_t at = (size_t)16 * (D + 8) * 2 + (size_t)16 * D * 4 + (size_t)kCW * 32 * 4 + 32 * 4 + (size_t)16 * nsplit * 4;
  size_t p = x > at ? x : at;
  return (p + 127) & ~(size_t)127;
}

size_t fixed_bytes() { return (size_t)kNB * 256 * 4 + 2 * kNB * 4 + 64 * 4 + 8 * 4 + 8 * 4 + 16 + 128; }

size_t mega_smem(int stages, size_t phase) {
  return (size_t)stages * kStageBytes + (size_t)2 * stages * 8 + fixed_bytes() + phase;
}

template <typename T, int WFK, bool FP8KV, int D>
cudaError_t launch_hi(const MegaArgs& a, size_t smem, int grid, cudaStream_t s, bool coop) {
  const int G = a.Hq / a.Hkv;
  void* params[1] = {(void*)&a};
  const void* fn = G > 8 ? (const void*)decode_mega_kernel<T, WFK, FP8KV, D, true>
                         : (const void*)decode_mega_kernel<T, WFK, FP8KV, D, false>;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  if (coop) return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), params, smem, s);
  return cudaLaunchKernel(fn, dim3(grid), dim3(kThreads), params, smem, s);
}

template <typename T, int WFK>
cudaError_t launch_kv(const MegaArgs& a, size_t smem, int grid, cudaStream_t s, bool coop) {
  if (a.D == 128) {
    return a.kv_fp8 ? launch_hi<T, WFK, true, 128>(a, smem, grid, s, coop)
                    : launch_hi<T, WFK, false, 128>(a, smem, grid, s, coop);
  }
  if (a.D == 64) {
    return a.kv_fp8 ? launch_hi<T, WFK, true, 64>(a, smem, grid, s, coop)
                    : launch_hi<T, WFK, false, 64>(a, smem, grid, s, coop);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

// Host-visible mirror of MegaArgs (same field order and types); see decode_mega.h-style comments in
// engine/mega.py, which fills it through ctypes.
IPEX_API int ipex_decode_mega_args_bytes(void) { return (int)sizeof(MegaArgs); }
IPEX_API int ipex_decode_mega_layer_bytes(void) { return (int)sizeof(MegaLayer); }
IPEX_API int ipex_decode_mega_max_batch(void) { return kMaxM; }

// Shared-memory plan: returns the ring depth (>= 4) that fits, or 0 when the shape does not fit at all.
IPEX_API int ipex_decode_mega_stages(int wf, int M, int kmax, int D, int nsplit) {
  const int wfk = wf == WF_SYM_INT4 ? WFK_I8 : WFK_FP8;
  const int kp = (int)ceil_to_i64(kmax, 128);
  const size_t phase = phase_bytes(wfk, M, kp, D, nsplit);
  int stages = 192 / kCPS4;
  while (stages >= 4 && mega_smem(stages, phase) > 227 * 1024) stages--;
  return stages >= 4 ? stages : 0;
}

// One decode step.  `args` points to a host copy of MegaArgs; wf is WF_SYM_INT4 or WF_FP8_E4M3; dtype DT_F16 / DT_BF16.
// `coop` != 0 launches cooperatively (all CTAs guaranteed co-resident, which the grid barriers need).
// Returns a cudaError_t.
IPEX_API int ipex_decode_mega(const void* args, int wf, int dtype, int kmax, int grid, int coop, void* stream) {
  if (args == nullptr) return (int)cudaErrorInvalidValue;
  MegaArgs a = *reinterpret_cast<const MegaArgs*>(args);
  if (a.B < 1 || a.B > kMaxM || a.Hq % a.Hkv != 0 || a.Hq / a.Hkv > 16 || (a.H % 64) != 0 || (a.I % 64) != 0 ||
      (a.Nqkv % 16) != 0 || (a.V % 16) != 0 || (a.I % 16) != 0 || a.nsplit < 1 || a.nsplit > 64 || a.err == nullptr)
    return (int)cudaErrorInvalidValue;
  if (wf != WF_SYM_INT4 && wf != WF_FP8_E4M3) return (int)cudaErrorInvalidValue;
  const int wfk = wf == WF_SYM_INT4 ? WFK_I8 : WFK_FP8;
  if (wfk == WFK_FP8 && ((a.H % 128) != 0 || (a.I % 128) != 0 || ((a.Hq * a.D) % 128) != 0))
    return (int)cudaErrorInvalidValue;
  const int kp = (int)ceil_to_i64(kmax, 128);
  const size_t phase = phase_bytes(wfk, a.B, kp, a.D, a.nsplit);
  if (a.stages < 4 || mega_smem(a.stages, phase) > 227 * 1024) return (int)cudaErrorInvalidValue;
  const size_t smem = mega_smem(a.stages, phase);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) {
    return wfk == WFK_I8 ? (int)launch_kv<__half, WFK_I8>(a, smem, grid, s, coop != 0)
                         : (int)launch_kv<__half, WFK_FP8>(a, smem, grid, s, coop != 0);
  }
  if (dtype == DT_BF16) {
    return wfk == WFK_I8 ? (int)launch_kv<__nv_bfloat16, WFK_I8>(a, smem, grid, s, coop != 0)
                         : (int)launch_kv<__nv_bfloat16, WFK_FP8>(a, smem, grid, s, coop != 0);
  }
  return (int)cudaErrorInvalidValue;
}
