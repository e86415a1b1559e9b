// Low-bit GEMV / skinny GEMM for decode (M <= 8), bulk-async (TMA) pipelined version, sm_100a.
//
// Same contract as gemv_lowbit.cu (y = epilogue(prologue(x) * dequant(W)^T), tile layout of
// native/host/quant_core.cpp), different data movement.  Decode GEMVs of a 7B model stream 8-45 MB each and
// last only microseconds, so a kernel that starts loading when its warps are ready to compute spends most of
// its life waiting for the first bytes.  Here
//   * a producer warp streams the CTA's weight tiles with cp.async.bulk (global -> shared, completion on an
//     mbarrier) through a ring of stages; a row tile's K chunks are contiguous in the tile layout, so one
//     bulk copy moves up to 16 chunks (16 KB of 4-bit codes) plus one copy for their scales;
//   * the producer never waits for the previous kernel (weights do not depend on it): with programmatic
//     dependent launch the ring is already full when griddepcontrol.wait returns and the consumers have
//     finished staging / normalising x;
//   * sixteen consumer warps split the chunks of a stage, run the fragment-order mma pipeline straight out of
//     shared memory (4-bit codes become fp16 operands with ONE logic op per pair: the constant offsets are
//     removed from the fp32 accumulator once per 64-group), and release the stage through an "empty" mbarrier;
//   * CTAs are persistent over row-tile groups, so x is staged (and RMS-normalised) once per CTA.
// Every mbarrier wait is bounded; on expiry the kernel records an error code in *err and leaves.
#include "common/utils.cuh"
#include <cuda_fp8.h>

namespace {

constexpr int kCW = 16;                      // consumer warps
constexpr int kCThreads = kCW * 32;          // 512
constexpr int kThreadsTma = kCThreads + 32;  // + producer warp
constexpr int kSpinLimit = 1 << 22;
constexpr int kNB = 4;                        // reduction buffers in flight

struct TmaArgs {
  const uint8_t* w;
  const void* x;
  void* y;
  const void* norm_w;
  const void* bias;
  const void* residual;
  const float* lut;
  int* err;
  int M, N, K;
  int ldx, ldy, ldr;
  float eps, norm_offset;
  int act;
  int stages;  // ring depth
  int cps;     // chunks (of 128 k) per stage
  // tensor-parallel row-parallel layers: fused all-reduce over NVLink peer memory (tp_world > 1)
  int tp_rank, tp_world, tp_npad;
  float* const* tp_bufs;   // [tp_world] device pointers: rank r's partial buffer [tp_world][8][tp_npad] fp32
  int* const* tp_flags;    // [tp_world] device pointers: rank r's per-tile arrival counters
  // mixture-of-experts mode (moe_ranges != null): ONE launch walks every expert that received tokens.  The
  // (token, choice) slots are sorted by expert: moe_ranges[e] = (first position, count) in moe_order.  For each
  // expert (and each group of at most M of its tokens) the CTA stages those rows of x again and streams its share
  // of the expert's row tiles; the weight ring keeps flowing across experts.  x row = moe_order[pos] / moe_xdiv
  // (moe_gather) or pos; y row = moe_order[pos] (moe_scatter) or pos.
  const uint8_t* const* moe_w = nullptr;
  const int* moe_ranges = nullptr;
  const int* moe_order = nullptr;
  int moe_experts = 0, moe_slots = 0, moe_gather = 0, moe_scatter = 0, moe_xdiv = 1;
};

// Barrier of the kCW consumer warps with a bounded wait: sync[0] counts arrivals (monotonic, `target` = warps x
// passes so far), sync[1] != 0 means a warp gave up.  Returns false if the others did not arrive.
__device__ __forceinline__ bool pass_barrier(int* sync, int target) {
  __syncwarp();
  int good = 1;
  if ((threadIdx.x & 31) == 0) {
    __threadfence_block();
    atomicAdd(sync, 1);
    good = 0;
    for (int i = 0; i < (1 << 22); i++) {
      if (*(volatile int*)(sync + 1) != 0) break;
      if (*(volatile int*)sync >= target) { good = 1; break; }
      __nanosleep(32);
    }
    __threadfence_block();
  }
  good = __shfl_sync(0xffffffffu, good, 0);
  return good != 0;
}

// Enumerates the passes of a launch: one for a plain GEMV; in mixture-of-experts mode one per (expert that received
// tokens, group of at most `mcap` of them).  Producer and consumers walk the same sequence.
struct PassWalk {
  int e = -1, base = 0, cnt = 0, first = 0;
  __device__ bool next(const TmaArgs& a, int mcap) {
    if (a.moe_ranges == nullptr) {
      if (e >= 0) return false;
      e = 0;
      return true;
    }
    if (e >= 0) {
      base += mcap;
      if (base < cnt) return true;
    }
    for (++e; e < a.moe_experts; ++e) {
      cnt = a.moe_ranges[2 * e + 1];
      cnt = cnt < a.moe_slots ? cnt : a.moe_slots;
      if (cnt > 0) {
        first = a.moe_ranges[2 * e];
        base = 0;
        return true;
      }
    }
    return false;
  }
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

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
// bounded wait for the phase with the given parity; false on expiry
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  uint32_t done = 0;
  for (int i = 0; i < kSpinLimit; i++) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    // back off: a waiting warp must not eat the issue slots of the warps that have data
    if (i >= 2) __nanosleep(i < 32 ? 32 : 128);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCThreads) : "memory"); }

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// word = 8 nibbles in magic order -> four fp16x2 operands WITHOUT removing the offsets:
//   p[0], p[2] = 1024 + q      (weights 0,1 and 4,5 of the octet)
//   p[1], p[3] = 1024 + 16 q   (weights 2,3 and 6,7)
// The activations paired with p[1]/p[3] are stored pre-divided by 16, and the constant parts
// (1024 + zero point) * x are removed once per 64-group from the fp32 accumulator (see xcorr), so the
// dequantization costs one logic op per pair instead of a logic op and a floating point op.
struct Int4Raw {
  uint32_t p[4];
  __device__ __forceinline__ explicit Int4Raw(uint32_t u) {
    constexpr uint32_t kMagic = 0x64006400u;
    const uint32_t u2 = u >> 8;
    p[0] = (u & 0x000F000Fu) | kMagic;
    p[1] = (u & 0x00F000F0u) | kMagic;
    p[2] = (u2 & 0x000F000Fu) | kMagic;
    p[3] = (u2 & 0x00F000F0u) | kMagic;
  }
};

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == 1) return g / (1.0f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.0f + tanhf(k0 * (g + k1 * g * g * g)));
}

// x -> fp16 rows in shared memory (optionally RMS-normalised), zero padded to Kp; consumer threads only
template <typename T, bool PRESCALE>
__device__ void stage_x(const TmaArgs& a, __half* xs, int xs_stride, int Kp, float* scratch,
                        const int* xrow = nullptr) {
  const int tid = threadIdx.x;
  const T* x = reinterpret_cast<const T*>(a.x);
  const T* nw = reinterpret_cast<const T*>(a.norm_w);
  const int nvec = a.K / 8;  // K % 64 == 0
  for (int m = 0; m < a.M; m++) {
    const T* xr = x + (size_t)(xrow != nullptr ? xrow[m] : m) * a.ldx;
    float rstd = 1.0f;
    if (nw != nullptr) {
      float ss = 0.f;
      for (int v = tid; v < nvec; v += kCThreads) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; j++) { const float f = DT<T>::to_f(e[j]); ss += f * f; }
      }
      ss = warp_sum(ss);
      if ((tid & 31) == 0) scratch[tid >> 5] = ss;
      consumer_sync();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kCW; w++) tot += scratch[w];
      rstd = rsqrtf(tot / (float)a.K + a.eps);
      consumer_sync();
    }
    for (int v = tid; v < Kp / 8; v += kCThreads) {
      __align__(16) __half o[8];
      if (v < nvec) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
        const T* e = reinterpret_cast<const T*>(&raw);
        uint4 wraw = make_uint4(0, 0, 0, 0);
        if (nw != nullptr) wraw = *reinterpret_cast<const uint4*>(nw + v * 8);
        const T* we = reinterpret_cast<const T*>(&wraw);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float f = DT<T>::to_f(e[j]);
          if (nw != nullptr) f = f * rstd * (DT<T>::to_f(we[j]) + a.norm_offset);
          f = fminf(fmaxf(f, -65504.f), 65504.f);
          if (PRESCALE && (j & 2)) f *= 0.0625f;   // partners of the "1024 + 16 q" operands
          o[j] = __float2half_rn(f);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] = __float2half_rn(0.f);
      }
      *reinterpret_cast<uint4*>(xs + m * xs_stride + v * 8) = *reinterpret_cast<const uint4*>(o);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Integer path for symmetric int4 (internal family code WF_I8): the activations of a token become 15-bit integers
// xi = hi * 128 + lo (hi, lo int8, one fp32 scale per token), the 4-bit codes become int8 operands with one logic
// op per FOUR weights, and the products run on the s8 tensor-core instruction (m16n8k32).  Exact integer
// accumulation per 64-group, then one int->float conversion and one FMA with the group's weight scale per output.
// The "- 8" of the codes is applied by starting the accumulators at -8 * sum(x) of the group (precomputed when x is
// staged), so it costs nothing in the loop.  Operand order: a word of 8 codes masks into bytes (k0,k4,k1,k5) and
// (k2,k6,k3,k7); x is stored in the same order, so no byte shuffles are needed on either side.
// ------------------------------------------------------------------------------------------------------------------
constexpr int WF_I8 = 100;
constexpr int kI8Pad = 64;  // extra bytes per staged token row: 8 rows x 4 lanes x 16 B hit 32 distinct 16-byte banks

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// x -> (hi, lo) int8 rows in the octet order above, per-token scale, per-(group, token) accumulator seeds.
//   xh / xl : [M][Kp + kI8Pad] bytes      dxs : [8] floats      seeds : [Kp/64][8 tokens] int2 = (-8 sum hi, -8 sum lo)
template <typename T>
__device__ void stage_x_i8(const TmaArgs& a, int8_t* xh, int8_t* xl, int stride, int Kp, float* dxs, int2* seeds,
                           float* scratch, const int* xrow = nullptr) {
  const int tid = threadIdx.x;
  const T* x = reinterpret_cast<const T*>(a.x);
  const T* nw = reinterpret_cast<const T*>(a.norm_w);
  const int nvec = a.K / 8;  // K % 64 == 0
  const int groups = Kp / 64;
  for (int i = tid; i < groups * 8; i += kCThreads)
    if ((i & 7) >= a.M) seeds[i] = make_int2(0, 0);
  if (tid < 8) dxs[tid] = 0.f;
  for (int m = 0; m < a.M; m++) {
    const T* xr = x + (size_t)(xrow != nullptr ? xrow[m] : m) * a.ldx;
    float ss = 0.f, mx = 0.f;
    for (int v = tid; v < nvec; v += kCThreads) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
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
    if ((tid & 31) == 0) { scratch[tid >> 5] = ss; scratch[kCW + (tid >> 5)] = mx; }
    consumer_sync();
    float tot = 0.f, amax = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; w++) { tot += scratch[w]; amax = fmaxf(amax, scratch[kCW + w]); }
    const float rstd = nw != nullptr ? rsqrtf(tot / (float)a.K + a.eps) : 1.0f;
    amax *= rstd;
    const float dx = amax > 0.f ? amax / 16383.f : 1.0f;
    const float inv = rstd / dx;   // value * weight * inv = integer
    if (tid == 0) dxs[m] = dx;
    consumer_sync();
    for (int v0 = 0; v0 < Kp / 8; v0 += kCThreads) {
      const int v = v0 + tid;
      int sh = 0, sl = 0;
      if (v < Kp / 8) {
        uint32_t ph[2] = {0, 0}, pl[2] = {0, 0};
        if (v < nvec) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
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
            // element j of the octet -> byte position in (k0,k4,k1,k5 | k2,k6,k3,k7)
            const int pos = ((j & 2) ? 4 : 0) + ((j & 1) ? 2 : 0) + ((j & 4) ? 1 : 0);
            ph[pos >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (pos & 3));
            pl[pos >> 2] |= (uint32_t)lo << (8 * (pos & 3));
          }
        }
        *reinterpret_cast<uint2*>(xh + (size_t)m * stride + v * 8) = make_uint2(ph[0], ph[1]);
        *reinterpret_cast<uint2*>(xl + (size_t)m * stride + v * 8) = make_uint2(pl[0], pl[1]);
      }
      // 8 consecutive octets (= 8 consecutive lanes) form a 64-group
      sh += __shfl_xor_sync(0xffffffffu, sh, 1); sl += __shfl_xor_sync(0xffffffffu, sl, 1);
      sh += __shfl_xor_sync(0xffffffffu, sh, 2); sl += __shfl_xor_sync(0xffffffffu, sl, 2);
      sh += __shfl_xor_sync(0xffffffffu, sh, 4); sl += __shfl_xor_sync(0xffffffffu, sl, 4);
      if ((tid & 7) == 0 && v < Kp / 8) seeds[(v >> 3) * 8 + m] = make_int2(-8 * sh, -8 * sl);
    }
  }
}

template <int WF, typename T, int RT>
#ifndef IPEX_GEMV_MIN_BLOCKS
#define IPEX_GEMV_MIN_BLOCKS 1
#endif
__global__ void __launch_bounds__(kThreadsTma, IPEX_GEMV_MIN_BLOCKS) gemv_tma_kernel(TmaArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr bool kI8 = WF == WF_I8;
  constexpr bool k4bit = WF == WF_SYM_INT4 || WF == WF_ASYM_INT4 || WF == WF_LUT4 || kI8;
  constexpr int CB = k4bit ? 1024 : 2048;                 // code bytes per 128-k chunk of a row tile
  constexpr int SB = 64;                                  // scale bytes per chunk
  constexpr int MB = WF == WF_ASYM_INT4 ? 64 : 0;         // min bytes per chunk
  const int Kp = (int)ceil_to_i64(a.K, 128);
  const int Np = (int)ceil_to_i64(a.N, 16);
  const int chunks = Kp / 128;
  const int xs_stride = kI8 ? Kp + kI8Pad : Kp + 8;   // elements of xs (fp16) / bytes of each int8 plane
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int STAGES = a.stages, CPS = a.cps;
  const int Mcap = a.M;                  // rows the shared-memory layout holds; a.M becomes the rows of the pass
  const bool moe = a.moe_ranges != nullptr;
  const int stage_bytes = CPS * (CB + SB + MB);
  const int stages_per_tile = (chunks + CPS - 1) / CPS;
  const int ntiles = Np / 16;
  const int ngroups = (ntiles + RT - 1) / RT;

  // shared memory carve-up (the ring first: bulk copies need 16-byte alignment, it gets 128)
  uint8_t* ring = smem_raw;
  size_t off = (size_t)STAGES * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + off);
  uint64_t* empty_bar = full_bar + STAGES;
  off += (size_t)2 * STAGES * sizeof(uint64_t);
  off = (off + 15) & ~(size_t)15;
  __half* xs = reinterpret_cast<__half*>(smem_raw + off);
  off += ((size_t)Mcap * xs_stride * sizeof(__half) + 15) & ~(size_t)15;
  float* red = reinterpret_cast<float*>(smem_raw + off);      // [kNB][RT][16][8], zero between uses
  off += (size_t)kNB * RT * 128 * sizeof(float);
  int* red_cnt = reinterpret_cast<int*>(smem_raw + off);      // [kNB] tickets
  int* red_gen = red_cnt + kNB;                                // [kNB] generations
  off += 2 * kNB * sizeof(int);
  float* scratch = reinterpret_cast<float*>(smem_raw + off);
  off += 128;
  int* xrow = reinterpret_cast<int*>(smem_raw + off);          // expert mode: rows of x / y of the pass [2][8]
  int* yrow = xrow + 8;
  int* pass_sync = yrow + 8;                                   // [0] arrivals at the pass barrier, [1] abort flag
  off += 96;
  float* dxs = reinterpret_cast<float*>(smem_raw + off);       // integer path: per-token activation scale
  off += 32;
  int2* seeds = reinterpret_cast<int2*>(smem_raw + off);       // integer path: [Kp/64][8] accumulator seeds
  if (kI8) off += (size_t)(Kp / 64) * 8 * sizeof(int2);
  float* xcorr = reinterpret_cast<float*>(smem_raw + off);     // int4: [M][Kp/64]
  if (WF == WF_SYM_INT4 || WF == WF_ASYM_INT4) off += (size_t)Mcap * (Kp / 64) * sizeof(float);
  float* xsum = reinterpret_cast<float*>(smem_raw + off);      // asym: [M][Kp/64]
  if (WF == WF_ASYM_INT4) off += (size_t)Mcap * (Kp / 64) * sizeof(float);
  uint32_t* lut256 = reinterpret_cast<uint32_t*>(smem_raw + off);

  const size_t code_bytes = k4bit ? (size_t)Np * Kp / 2 : (size_t)Np * Kp;

  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kCW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kCW) {
    // ---------------- producer: independent of the previous kernel, starts immediately ----------------
    if (lane == 0) {
      int it = 0, goff = 0;
      bool ok = true;
      PassWalk walk;
      if (moe) pdl_wait();               // the expert ranges come from the kernel before this one
      while (ok && walk.next(a, Mcap)) {
        const uint8_t* codes = moe ? a.moe_w[walk.e] : a.w;
        const uint8_t* scales = codes + code_bytes;
        const uint8_t* mins = scales + (size_t)Np * (Kp / 64) * 2;
        // row-tile groups are dealt round-robin over the CTAs, continuing where the previous pass stopped
        for (int grp = (blockIdx.x + gridDim.x - goff) % gridDim.x; grp < ngroups && ok; grp += gridDim.x) {
          for (int r = 0; r < RT && ok; r++) {
            const int tile = grp * RT + r;
            if (tile >= ntiles) break;
            for (int sp = 0; sp < stages_per_tile; sp++, it++) {
              const int slot = it % STAGES;
              if (it >= STAGES) {
                if (!mbar_wait(&empty_bar[slot], ((it / STAGES) - 1) & 1)) {
                  atomicExch(a.err, 1);
                  ok = false;
                  break;
                }
              }
              const int c0 = sp * CPS;
              const int nch = min(CPS, chunks - c0);
              uint8_t* dst = ring + (size_t)slot * stage_bytes;
              mbar_expect_tx(&full_bar[slot], (uint32_t)(nch * (CB + SB + MB)));
              const size_t chunk_index = (size_t)tile * chunks + c0;
              bulk_g2s(dst, codes + chunk_index * CB, (uint32_t)(nch * CB), &full_bar[slot]);
              bulk_g2s(dst + CPS * CB, scales + chunk_index * SB, (uint32_t)(nch * SB), &full_bar[slot]);
              if (MB)
                bulk_g2s(dst + CPS * (CB + SB), mins + chunk_index * MB, (uint32_t)(nch * MB), &full_bar[slot]);
            }
          }
        }
        goff = (goff + ngroups) % gridDim.x;
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  pdl_wait();
  constexpr bool kInt4 = WF == WF_SYM_INT4 || WF == WF_ASYM_INT4;
  for (int i = tid; i < kNB * RT * 128; i += kCThreads) red[i] = 0.f;
  if (tid < 2 * kNB) red_cnt[tid] = 0;
  if (WF == WF_LUT4 && tid < 256) {
    __half2 v = __floats2half2_rn(a.lut[tid & 15], a.lut[tid >> 4]);
    lut256[tid] = *reinterpret_cast<uint32_t*>(&v);
  }
  int8_t* xh = reinterpret_cast<int8_t*>(xs);
  int8_t* xl = xh + (size_t)Mcap * xs_stride;
  T* y = reinterpret_cast<T*>(a.y);
  int it = 0, giter = 0, goff = 0, npass = 0;
  bool ok = true;
  PassWalk walk;
  if (moe) {
    if (tid == 0) { pass_sync[0] = 0; pass_sync[1] = 0; }
    consumer_sync();
  }
  while (ok && walk.next(a, Mcap)) {
    if (moe) {
      // Every warp must be done with the previous pass's rows before they are replaced.  A warp that gave up on a
      // bounded wait never arrives, so this barrier is bounded too (and watches the abort flag).
      if (!pass_barrier(pass_sync, ++npass * kCW)) {
        if (lane == 0) atomicExch(a.err, 5);
        break;
      }
      a.M = walk.cnt - walk.base < Mcap ? walk.cnt - walk.base : Mcap;
      if (tid < a.M) {
        const int pos = walk.first + walk.base + tid;
        int slot = a.moe_order[pos];
        slot = slot < 0 ? 0 : (slot >= a.moe_slots ? a.moe_slots - 1 : slot);
        xrow[tid] = a.moe_gather ? slot / a.moe_xdiv : pos;
        yrow[tid] = a.moe_scatter ? slot : pos;
      }
      consumer_sync();
    }
    if constexpr (kI8) stage_x_i8<T>(a, xh, xl, xs_stride, Kp, dxs, seeds, scratch, moe ? xrow : nullptr);
    else stage_x<T, kInt4>(a, xs, xs_stride, Kp, scratch, moe ? xrow : nullptr);
    consumer_sync();
    if (kInt4) {
      // per (row of x, 64-group): the constant part of sum_k A_k x'_k to take out of the accumulator, and for the
      // asymmetric format the plain sum of x (for the "+ min" term)
      const int groups = Kp / 64;
      const float zlo = WF == WF_SYM_INT4 ? 1032.f : 1024.f;
      const float zhi = WF == WF_SYM_INT4 ? 1152.f : 1024.f;
      for (int i = tid; i < a.M * groups; i += kCThreads) {
        const int m = i / groups, gi = i % groups;
        float slo = 0.f, shi = 0.f;
        for (int k = 0; k < 64; k++) {
          const float v = __half2float(xs[m * xs_stride + gi * 64 + k]);
          if (k & 2) shi += v; else slo += v;
        }
        xcorr[i] = zlo * slo + zhi * shi;
        if (WF == WF_ASYM_INT4) xsum[i] = slo + 16.f * shi;
      }
      consumer_sync();
    }

    const bool has_x = g < a.M;
    // row-tile groups are dealt round-robin over the CTAs, continuing where the previous pass stopped
    for (int grp = (blockIdx.x + gridDim.x - goff) % gridDim.x; grp < ngroups && ok; grp += gridDim.x, giter++) {
      float acc[RT][4];
#pragma unroll
      for (int r = 0; r < RT; r++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[r][i] = 0.f;
#pragma unroll
      for (int r = 0; r < RT; r++) {
        const int tile = grp * RT + r;
        if (tile >= ntiles) break;
        for (int sp = 0; sp < stages_per_tile; sp++, it++) {
          const int slot = it % STAGES;
          if (!mbar_wait(&full_bar[slot], (it / STAGES) & 1)) {
            atomicExch(a.err, 2);
            ok = false;
            break;
          }
          const int c0 = sp * CPS;
          const int nch = min(CPS, chunks - c0);
          const uint8_t* st = ring + (size_t)slot * stage_bytes;
          const uint8_t* st_scales = st + CPS * CB;
          const uint8_t* st_mins = st + CPS * (CB + SB);
          for (int c = warp; c < nch; c += kCW) {
            const int cg = c0 + c;
            if constexpr (kI8) {
              const uint8_t* tp = st + c * CB;
              const uint4 qa = *reinterpret_cast<const uint4*>(tp + g * 64 + t * 16);
              const uint4 qb = *reinterpret_cast<const uint4*>(tp + (g + 8) * 64 + t * 16);
              const uint32_t s0 = *reinterpret_cast<const uint32_t*>(st_scales + c * SB + (0 * 16 + 2 * g) * 2);
              const uint32_t s1 = *reinterpret_cast<const uint32_t*>(st_scales + c * SB + (1 * 16 + 2 * g) * 2);
              uint4 h0 = make_uint4(0, 0, 0, 0), h1 = h0, l0 = h0, l1 = h0;
              if (has_x) {
                const int8_t* ph = xh + (size_t)g * xs_stride + cg * 128 + 16 * t;
                const int8_t* pl = xl + (size_t)g * xs_stride + cg * 128 + 16 * t;
                h0 = *reinterpret_cast<const uint4*>(ph);
                h1 = *reinterpret_cast<const uint4*>(ph + 64);
                l0 = *reinterpret_cast<const uint4*>(pl);
                l1 = *reinterpret_cast<const uint4*>(pl + 64);
              }
              const int4 sd0 = *reinterpret_cast<const int4*>(seeds + (2 * cg) * 8 + 2 * t);
              const int4 sd1 = *reinterpret_cast<const int4*>(seeds + (2 * cg + 1) * 8 + 2 * t);
              constexpr uint32_t kM = 0x0F0F0F0Fu;
              // group 0 (words x, y), group 1 (words z, w)
              int ah0[4] = {sd0.x, sd0.z, sd0.x, sd0.z}, al0[4] = {sd0.y, sd0.w, sd0.y, sd0.w};
              int ah1[4] = {sd1.x, sd1.z, sd1.x, sd1.z}, al1[4] = {sd1.y, sd1.w, sd1.y, sd1.w};
              {
                const uint32_t a0 = qa.x & kM, a1 = qb.x & kM, a2 = (qa.x >> 4) & kM, a3 = (qb.x >> 4) & kM;
                mma_s8(ah0, a0, a1, a2, a3, h0.x, h0.y);
                mma_s8(al0, a0, a1, a2, a3, l0.x, l0.y);
              }
              {
                const uint32_t a0 = qa.z & kM, a1 = qb.z & kM, a2 = (qa.z >> 4) & kM, a3 = (qb.z >> 4) & kM;
                mma_s8(ah1, a0, a1, a2, a3, h1.x, h1.y);
                mma_s8(al1, a0, a1, a2, a3, l1.x, l1.y);
              }
              {
                const uint32_t a0 = qa.y & kM, a1 = qb.y & kM, a2 = (qa.y >> 4) & kM, a3 = (qb.y >> 4) & kM;
                mma_s8(ah0, a0, a1, a2, a3, h0.z, h0.w);
                mma_s8(al0, a0, a1, a2, a3, l0.z, l0.w);
              }
              {
                const uint32_t a0 = qa.w & kM, a1 = qb.w & kM, a2 = (qa.w >> 4) & kM, a3 = (qb.w >> 4) & kM;
                mma_s8(ah1, a0, a1, a2, a3, h1.z, h1.w);
                mma_s8(al1, a0, a1, a2, a3, l1.z, l1.w);
              }
              const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
              const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));
              acc[r][0] += d0.x * (float)(ah0[0] * 128 + al0[0]) + d1.x * (float)(ah1[0] * 128 + al1[0]);
              acc[r][1] += d0.x * (float)(ah0[1] * 128 + al0[1]) + d1.x * (float)(ah1[1] * 128 + al1[1]);
              acc[r][2] += d0.y * (float)(ah0[2] * 128 + al0[2]) + d1.y * (float)(ah1[2] * 128 + al1[2]);
              acc[r][3] += d0.y * (float)(ah0[3] * 128 + al0[3]) + d1.y * (float)(ah1[3] * 128 + al1[3]);
              continue;
            }
            uint4 xa0 = make_uint4(0, 0, 0, 0), xa1 = xa0, xb0 = xa0, xb1 = xa0;
            if (has_x) {
              const __half* xp = xs + g * xs_stride + cg * 128 + 16 * t;
              xa0 = *reinterpret_cast<const uint4*>(xp);
              xa1 = *reinterpret_cast<const uint4*>(xp + 8);
              xb0 = *reinterpret_cast<const uint4*>(xp + 64);
              xb1 = *reinterpret_cast<const uint4*>(xp + 72);
            }
            if constexpr (k4bit) {
              const uint8_t* tp = st + c * CB;
              const uint4 qa = *reinterpret_cast<const uint4*>(tp + g * 64 + t * 16);
              const uint4 qb = *reinterpret_cast<const uint4*>(tp + (g + 8) * 64 + t * 16);
              const uint32_t s0 = *reinterpret_cast<const uint32_t*>(st_scales + c * SB + (0 * 16 + 2 * g) * 2);
              const uint32_t s1 = *reinterpret_cast<const uint32_t*>(st_scales + c * SB + (1 * 16 + 2 * g) * 2);
              const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
              const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));
              float c0v[4] = {0.f, 0.f, 0.f, 0.f}, c1v[4] = {0.f, 0.f, 0.f, 0.f};
              if constexpr (WF == WF_LUT4) {
                auto lp = [&](uint32_t word, int byte) { return lut256[(word >> (8 * byte)) & 0xFF]; };
                mma_f16(c0v, lp(qa.x, 0), lp(qb.x, 0), lp(qa.x, 1), lp(qb.x, 1), xa0.x, xa0.y);
                mma_f16(c0v, lp(qa.x, 2), lp(qb.x, 2), lp(qa.x, 3), lp(qb.x, 3), xa0.z, xa0.w);
                mma_f16(c0v, lp(qa.y, 0), lp(qb.y, 0), lp(qa.y, 1), lp(qb.y, 1), xa1.x, xa1.y);
                mma_f16(c0v, lp(qa.y, 2), lp(qb.y, 2), lp(qa.y, 3), lp(qb.y, 3), xa1.z, xa1.w);
                mma_f16(c1v, lp(qa.z, 0), lp(qb.z, 0), lp(qa.z, 1), lp(qb.z, 1), xb0.x, xb0.y);
                mma_f16(c1v, lp(qa.z, 2), lp(qb.z, 2), lp(qa.z, 3), lp(qb.z, 3), xb0.z, xb0.w);
                mma_f16(c1v, lp(qa.w, 0), lp(qb.w, 0), lp(qa.w, 1), lp(qb.w, 1), xb1.x, xb1.y);
                mma_f16(c1v, lp(qa.w, 2), lp(qb.w, 2), lp(qa.w, 3), lp(qb.w, 3), xb1.z, xb1.w);
              } else {
                // two independent accumulation chains per 64-group keep the tensor pipe busy
                float c0w[4] = {0.f, 0.f, 0.f, 0.f}, c1w[4] = {0.f, 0.f, 0.f, 0.f};
                {
                  Int4Raw A(qa.x), B(qb.x);
                  mma_f16(c0v, A.p[0], B.p[0], A.p[1], B.p[1], xa0.x, xa0.y);
                  mma_f16(c0w, A.p[2], B.p[2], A.p[3], B.p[3], xa0.z, xa0.w);
                }
                {
                  Int4Raw A(qa.z), B(qb.z);
                  mma_f16(c1v, A.p[0], B.p[0], A.p[1], B.p[1], xb0.x, xb0.y);
                  mma_f16(c1w, A.p[2], B.p[2], A.p[3], B.p[3], xb0.z, xb0.w);
                }
                {
                  Int4Raw A(qa.y), B(qb.y);
                  mma_f16(c0v, A.p[0], B.p[0], A.p[1], B.p[1], xa1.x, xa1.y);
                  mma_f16(c0w, A.p[2], B.p[2], A.p[3], B.p[3], xa1.z, xa1.w);
                }
                {
                  Int4Raw A(qa.w), B(qb.w);
                  mma_f16(c1v, A.p[0], B.p[0], A.p[1], B.p[1], xb1.x, xb1.y);
                  mma_f16(c1w, A.p[2], B.p[2], A.p[3], B.p[3], xb1.z, xb1.w);
                }
                const int groups = Kp / 64;
                const int n0 = 2 * t, n1 = 2 * t + 1;
                const float k00 = n0 < a.M ? xcorr[n0 * groups + 2 * cg] : 0.f;
                const float k01 = n0 < a.M ? xcorr[n0 * groups + 2 * cg + 1] : 0.f;
                const float k10 = n1 < a.M ? xcorr[n1 * groups + 2 * cg] : 0.f;
                const float k11 = n1 < a.M ? xcorr[n1 * groups + 2 * cg + 1] : 0.f;
                c0v[0] += c0w[0] - k00; c0v[1] += c0w[1] - k10; c0v[2] += c0w[2] - k00; c0v[3] += c0w[3] - k10;
                c1v[0] += c1w[0] - k01; c1v[1] += c1w[1] - k11; c1v[2] += c1w[2] - k01; c1v[3] += c1w[3] - k11;
              }
              acc[r][0] += d0.x * c0v[0] + d1.x * c1v[0];
              acc[r][1] += d0.x * c0v[1] + d1.x * c1v[1];
              acc[r][2] += d0.y * c0v[2] + d1.y * c1v[2];
              acc[r][3] += d0.y * c0v[3] + d1.y * c1v[3];
              if constexpr (WF == WF_ASYM_INT4) {
                const uint32_t m0 = *reinterpret_cast<const uint32_t*>(st_mins + c * MB + (0 * 16 + 2 * g) * 2);
                const uint32_t m1 = *reinterpret_cast<const uint32_t*>(st_mins + c * MB + (1 * 16 + 2 * g) * 2);
                const float2 mn0 = __half22float2(*reinterpret_cast<const __half2*>(&m0));
                const float2 mn1 = __half22float2(*reinterpret_cast<const __half2*>(&m1));
                const int groups = Kp / 64;
                const int n0 = 2 * t, n1 = 2 * t + 1;
                const float xs00 = n0 < a.M ? xsum[n0 * groups + 2 * cg] : 0.f;
                const float xs01 = n0 < a.M ? xsum[n0 * groups + 2 * cg + 1] : 0.f;
                const float xs10 = n1 < a.M ? xsum[n1 * groups + 2 * cg] : 0.f;
                const float xs11 = n1 < a.M ? xsum[n1 * groups + 2 * cg + 1] : 0.f;
                acc[r][0] += mn0.x * xs00 + mn1.x * xs01;
                acc[r][1] += mn0.x * xs10 + mn1.x * xs11;
                acc[r][2] += mn0.y * xs00 + mn1.y * xs01;
                acc[r][3] += mn0.y * xs10 + mn1.y * xs11;
              }
            } else {
              // 8-bit families: a 128-k chunk = two [16 rows][64 k] tiles of 1024 bytes
              float cc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
              const uint4 xv[4] = {xa0, xa1, xb0, xb1};
#pragma unroll
              for (int h = 0; h < 2; h++) {
                const uint8_t* tp = st + c * CB + h * 1024;
                const uint4 qa = *reinterpret_cast<const uint4*>(tp + g * 64 + t * 16);
                const uint4 qb = *reinterpret_cast<const uint4*>(tp + (g + 8) * 64 + t * 16);
                const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
                const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
                const uint32_t xw[8] = {xv[2 * h].x, xv[2 * h].y, xv[2 * h].z, xv[2 * h].w,
                                        xv[2 * h + 1].x, xv[2 * h + 1].y, xv[2 * h + 1].z, xv[2 * h + 1].w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  uint32_t a0, a1, a2, a3;
                  if constexpr (WF == WF_INT8) {
                    const uint32_t ua = wa[j] ^ 0x80808080u, ub = wb[j] ^ 0x80808080u;
                    constexpr uint32_t k1152 = 0x64806480u;
                    a0 = h2_sub(__byte_perm(ua, 0x64646464u, 0x4140), k1152);
                    a2 = h2_sub(__byte_perm(ua, 0x64646464u, 0x4342), k1152);
                    a1 = h2_sub(__byte_perm(ub, 0x64646464u, 0x4140), k1152);
                    a3 = h2_sub(__byte_perm(ub, 0x64646464u, 0x4342), k1152);
                  } else {
                    constexpr __nv_fp8_interpretation_t kind = WF == WF_FP8_E4M3 ? __NV_E4M3 : __NV_E5M2;
                    __half2_raw r0 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wa[j] & 0xFFFF), kind);
                    __half2_raw r2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wa[j] >> 16), kind);
                    __half2_raw r1 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wb[j] & 0xFFFF), kind);
                    __half2_raw r3 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wb[j] >> 16), kind);
                    a0 = (uint32_t)r0.x | ((uint32_t)r0.y << 16);
                    a2 = (uint32_t)r2.x | ((uint32_t)r2.y << 16);
                    a1 = (uint32_t)r1.x | ((uint32_t)r1.y << 16);
                    a3 = (uint32_t)r3.x | ((uint32_t)r3.y << 16);
                  }
                  mma_f16(cc[h], a0, a1, a2, a3, xw[2 * j], xw[2 * j + 1]);
                }
              }
              if constexpr (WF == WF_INT8) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                  const uint32_t s = *reinterpret_cast<const uint32_t*>(st_scales + c * SB + h * 32 + 2 * g * 2);
                  const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&s));
                  acc[r][0] += d.x * cc[h][0];
                  acc[r][1] += d.x * cc[h][1];
                  acc[r][2] += d.y * cc[h][2];
                  acc[r][3] += d.y * cc[h][3];
                }
              } else {
                const float2 d = *reinterpret_cast<const float2*>(st_scales + c * SB + 2 * g * 4);
                acc[r][0] += d.x * (cc[0][0] + cc[1][0]);
                acc[r][1] += d.x * (cc[0][1] + cc[1][1]);
                acc[r][2] += d.y * (cc[0][2] + cc[1][2]);
                acc[r][3] += d.y * (cc[0][3] + cc[1][3]);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty_bar[slot]);
        }
        if (!ok) break;
      }
      if (!ok) break;
      if constexpr (kI8) {
        const float dxa = dxs[2 * t], dxb = dxs[2 * t + 1];
#pragma unroll
        for (int r = 0; r < RT; r++) {
          acc[r][0] *= dxa; acc[r][1] *= dxb; acc[r][2] *= dxa; acc[r][3] *= dxb;
        }
      }

      // ---- cross-warp reduction without a CTA-wide barrier ----
      // Every warp adds its partial tile into one of kNB zero-initialised shared accumulators (shared-memory
      // float atomics) and then takes a ticket; the warp that draws the last ticket finalises the tile (reads
      // and re-zeroes the accumulator with atomicExch, applies the epilogue, stores) and publishes the buffer
      // for reuse by bumping its generation.  Fast warps run ahead into the next groups' buffers meanwhile.
      const int b = giter % kNB;
      {
        volatile int* genp = red_gen + b;
        bool ready = false;
        for (int i = 0; i < kSpinLimit; i++) {
          if (*genp == giter / kNB) { ready = true; break; }
          __nanosleep(64);
        }
        if (!ready) {
          atomicExch(a.err, 3);
          ok = false;
          break;
        }
      }
      float* rbuf = red + (size_t)b * RT * 128;
#pragma unroll
      for (int r = 0; r < RT; r++) {
        float* rp = rbuf + (size_t)r * 128;
        atomicAdd(&rp[g * 8 + 2 * t], acc[r][0]);
        atomicAdd(&rp[g * 8 + 2 * t + 1], acc[r][1]);
        atomicAdd(&rp[(g + 8) * 8 + 2 * t], acc[r][2]);
        atomicAdd(&rp[(g + 8) * 8 + 2 * t + 1], acc[r][3]);
      }
      __threadfence_block();
      __syncwarp();
      int ticket = 0;
      if (lane == 0) ticket = atomicAdd(red_cnt + b, 1);
      ticket = __shfl_sync(0xffffffffu, ticket, 0);
      if (ticket == kCW - 1) {
        __threadfence_block();
        if (a.tp_world > 1 && a.act == 0 && RT == 1) {
          // ---- fused all-reduce of this 16-row tile over peer memory ----
          // 1. push this rank's partial tile into slot [tp_rank] of EVERY rank's buffer (plain stores to the
          //    peers' mapped memory), 2. release-increment the tile's arrival counter on every rank,
          // 3. wait (bounded) until all tp_world partials of the tile have arrived here, 4. sum them locally.
          // Other warps of the CTA keep streaming the next tiles meanwhile.
          float pv[4];
          int pn[4], pc[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int i = lane + 32 * j;
            pc[j] = i % 8;
            pn[j] = grp * 16 + i / 8;
            pv[j] = atomicExch(&rbuf[i], 0.f);
          }
          for (int rk = 0; rk < a.tp_world; rk++) {
            float* dst = a.tp_bufs[rk] + (size_t)a.tp_rank * 8 * a.tp_npad;
#pragma unroll
            for (int j = 0; j < 4; j++)
              if (pn[j] < a.N && pc[j] < a.M) dst[(size_t)pc[j] * a.tp_npad + pn[j]] = pv[j];
          }
          __threadfence_system();
          __syncwarp();
          if (lane < a.tp_world) red_release_sys_add(a.tp_flags[lane] + grp, 1);
          int* my_flag = a.tp_flags[a.tp_rank] + grp;
          bool arrived = false;
          if (lane == 0) {
            for (int i = 0; i < kSpinLimit; i++) {
              if (ld_acquire_sys(my_flag) >= a.tp_world) { arrived = true; break; }
              __nanosleep(64);
            }
            if (arrived) *my_flag = 0;   // self-cleaning: the next user of this counter is two launches away
            else atomicExch(a.err, 4);
          }
          arrived = __shfl_sync(0xffffffffu, (int)arrived, 0) != 0;
          if (arrived) {
            const float* src = a.tp_bufs[a.tp_rank];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              if (pn[j] < a.N && pc[j] < a.M) {
                float sv = 0.f;
                for (int rk = 0; rk < a.tp_world; rk++)
                  sv += ld_relaxed_sys_f32(src + ((size_t)rk * 8 + pc[j]) * a.tp_npad + pn[j]);
                if (a.bias != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[pn[j]]);
                if (a.residual != nullptr)
                  sv += DT<T>::to_f(reinterpret_cast<const T*>(a.residual)[(size_t)pc[j] * a.ldr + pn[j]]);
                y[(size_t)pc[j] * a.ldy + pn[j]] = DT<T>::from_f(sv);
              }
            }
          }
        } else if (a.act == 0) {
#pragma unroll
          for (int j = 0; j < RT * 4; j++) {
            const int i = lane + 32 * j;            // index into [RT][16 rows][8 cols]
            const int r = i / 128, row = (i % 128) / 8, col = i % 8;
            float sv = atomicExch(&rbuf[i], 0.f);
            const int n = (grp * RT + r) * 16 + row;
            if (n < a.N && col < a.M) {
              if (a.bias != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[n]);
              if (a.residual != nullptr)
                sv += DT<T>::to_f(reinterpret_cast<const T*>(a.residual)[(size_t)col * a.ldr + n]);
              y[(size_t)(moe ? yrow[col] : col) * a.ldy + n] = DT<T>::from_f(sv);
            }
          }
        } else if (RT == 2) {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int i = lane + 32 * j;
            const int row = i / 8, col = i % 8;
            float gsum = atomicExch(&rbuf[i], 0.f), usum = atomicExch(&rbuf[128 + i], 0.f);
            const int n = grp * 16 + row;
            if (n < a.N / 2 && col < a.M) {
              if (a.bias != nullptr) {
                gsum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)grp * 32 + row]);
                usum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)grp * 32 + 16 + row]);
              }
              y[(size_t)(moe ? yrow[col] : col) * a.ldy + n] = DT<T>::from_f(act_apply(gsum, a.act) * usum);
            }
          }
        }
        __threadfence_block();
        __syncwarp();
        if (lane == 0) {
          red_cnt[b] = 0;
          __threadfence_block();
          *(volatile int*)(red_gen + b) = giter / kNB + 1;
        }
      }
    }
    goff = (goff + ngroups) % gridDim.x;
    if (moe && !ok && lane == 0) *(volatile int*)(pass_sync + 1) = 1;   // tell the warps waiting at the pass barrier
  }  // passes
}

struct LaunchPlan {
  int stages, cps, grid;
  size_t smem;
};

// Tuning knobs (set once per process through ipex_gemv_tma_tune): CTAs per SM the grid is sized for, and the
// shared-memory budget of one CTA.  The default leaves half of every SM free so that, under programmatic
// dependent launch, the next kernel's CTAs can become resident and fill their rings while this one computes.
int g_ctas_per_sm = 1;
int g_budget_kb = 140;
int g_cps4 = 32;
int g_int_path = 1;   // symmetric int4: integer tensor-core path (0 = fp16 operands)

template <int WF, int RT>
LaunchPlan plan(const TmaArgs& a) {
  constexpr bool k4bit = WF == WF_SYM_INT4 || WF == WF_ASYM_INT4 || WF == WF_LUT4 || WF == WF_I8;
  const int CB = k4bit ? 1024 : 2048;
  const int MB = WF == WF_ASYM_INT4 ? 64 : 0;
  const int Kp = (int)ceil_to_i64(a.K, 128), Np = (int)ceil_to_i64(a.N, 16);
  const int chunks = Kp / 128;
  LaunchPlan p;
  p.cps = k4bit ? g_cps4 : g_cps4 / 2;
  if (p.cps < 1) p.cps = 1;
  if (p.cps > chunks) p.cps = chunks;
  const size_t stage_bytes = (size_t)p.cps * (CB + 64 + MB);
  const size_t xrow = WF == WF_I8 ? (size_t)(Kp + kI8Pad) : (size_t)(Kp + 8);   // x 2 bytes (fp16, or two int8 planes)
  size_t fixed = (((size_t)a.M * xrow * 2 + 15) & ~(size_t)15) + (size_t)kNB * RT * 128 * 4 + 2 * kNB * 4 + 128 +
                 96 + 32 + 256;
  if (WF == WF_I8) fixed += (size_t)(Kp / 64) * 8 * 8;
  if (WF == WF_ASYM_INT4) fixed += (size_t)a.M * (Kp / 64) * 4;
  if (WF == WF_SYM_INT4 || WF == WF_ASYM_INT4) fixed += (size_t)a.M * (Kp / 64) * 4;
  if (WF == WF_LUT4) fixed += 1024;
  size_t budget = (size_t)g_budget_kb * 1024;
  if (budget < fixed + 3 * (stage_bytes + 16)) budget = fixed + 3 * (stage_bytes + 16);
  int stages = (int)((budget - fixed) / (stage_bytes + 16));
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  p.stages = stages;
  p.smem = (size_t)stages * stage_bytes + 2 * stages * 8 + 16 + fixed;
  const int ngroups = (Np / 16 + RT - 1) / RT;
  int per_sm = g_ctas_per_sm;
  while (per_sm > 1 && p.smem * per_sm > 220 * 1024) per_sm--;
  p.grid = ngroups < 148 * per_sm ? ngroups : 148 * per_sm;
  return p;
}

template <int WF, typename T, int RT>
cudaError_t launch_tma(TmaArgs a, cudaStream_t stream, bool pdl) {
  LaunchPlan p = plan<WF, RT>(a);
  // expert mode: a.M is only the number of an expert's tokens multiplied per pass; shrink it until the rows fit
  while (a.moe_ranges != nullptr && p.smem > 227 * 1024 && a.M > 1) {
    a.M--;
    p = plan<WF, RT>(a);
  }
  if (p.smem > 227 * 1024) return cudaErrorInvalidValue;
  a.stages = p.stages;
  a.cps = p.cps;
  auto kern = gemv_tma_kernel<WF, T, RT>;
  if (p.smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
    if (e != cudaSuccess) return e;
  }
  return launch_kernel(kern, dim3(p.grid), dim3(kThreadsTma), p.smem, stream, pdl, a);
}

template <int WF, typename T>
cudaError_t dispatch_rt(const TmaArgs& a, cudaStream_t s, bool pdl) {
  if (a.act != 0) return launch_tma<WF, T, 2>(a, s, pdl);
  return launch_tma<WF, T, 1>(a, s, pdl);
}

template <typename T>
cudaError_t dispatch_wf(int wf, const TmaArgs& a, cudaStream_t s, bool pdl) {
  switch (wf) {
    case WF_SYM_INT4:
      return g_int_path ? dispatch_rt<WF_I8, T>(a, s, pdl) : dispatch_rt<WF_SYM_INT4, T>(a, s, pdl);
    case WF_ASYM_INT4: return dispatch_rt<WF_ASYM_INT4, T>(a, s, pdl);
    case WF_LUT4: return dispatch_rt<WF_LUT4, T>(a, s, pdl);
    case WF_FP8_E4M3: return dispatch_rt<WF_FP8_E4M3, T>(a, s, pdl);
    case WF_FP8_E5M2: return dispatch_rt<WF_FP8_E5M2, T>(a, s, pdl);
    case WF_INT8: return dispatch_rt<WF_INT8, T>(a, s, pdl);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// Symmetric int4: 1 = integer (s8 tensor core) path, 0 = fp16-operand path.
IPEX_API void ipex_gemv_tma_int_path(int on) { g_int_path = on != 0; }

// Process-wide tuning of the pipelined GEMV (values <= 0 keep the current setting).
IPEX_API void ipex_gemv_tma_tune(int ctas_per_sm, int budget_kb, int chunks_per_stage_4bit) {
  if (ctas_per_sm > 0) g_ctas_per_sm = ctas_per_sm > 4 ? 4 : ctas_per_sm;
  if (budget_kb > 0) g_budget_kb = budget_kb > 220 ? 220 : budget_kb;
  if (chunks_per_stage_4bit > 0) g_cps4 = chunks_per_stage_4bit > 32 ? 32 : chunks_per_stage_4bit;
}

// Same arguments as ipex_gemv_lowbit plus `err`: a device int the kernel sets non-zero if one of its bounded
// mbarrier waits expires (1 = producer waiting for a free stage, 2 = consumer waiting for data).
// Returns cudaErrorInvalidValue when x does not fit shared memory (the caller then splits M or uses the
// non-pipelined kernel).
static int gemv_tma_entry(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx, int ldy,
                          const void* norm_w, float eps, float norm_offset, const void* bias, const void* residual,
                          int ldr, int act, const float* lut, int dtype, int pdl, int* err, void* stream, int tp_rank,
                          int tp_world, int tp_npad, const void* tp_bufs, const void* tp_flags) {
  if (M < 1 || M > 8 || (K % 64) != 0 || err == nullptr) return (int)cudaErrorInvalidValue;
  if ((ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return (int)cudaErrorInvalidValue;
  if (tp_world > 1 && (act != 0 || tp_bufs == nullptr || tp_flags == nullptr || tp_npad < N || tp_world > 8))
    return (int)cudaErrorInvalidValue;
  TmaArgs a;
  a.w = (const uint8_t*)w; a.x = x; a.y = y; a.norm_w = norm_w; a.bias = bias; a.residual = residual; a.lut = lut;
  a.err = err;
  a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = ldr; a.eps = eps; a.norm_offset = norm_offset;
  a.act = act; a.stages = 0; a.cps = 0;
  a.tp_rank = tp_rank; a.tp_world = tp_world; a.tp_npad = tp_npad;
  a.tp_bufs = reinterpret_cast<float* const*>(tp_bufs);
  a.tp_flags = reinterpret_cast<int* const*>(tp_flags);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) return (int)dispatch_wf<__half>(wf, a, s, pdl != 0);
  if (dtype == DT_BF16) return (int)dispatch_wf<__nv_bfloat16>(wf, a, s, pdl != 0);
  return (int)cudaErrorInvalidValue;
}

IPEX_API int ipex_gemv_lowbit_tma(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx, int ldy,
                                  const void* norm_w, float eps, float norm_offset, const void* bias,
                                  const void* residual, int ldr, int act, const float* lut, int dtype, int pdl,
                                  int* err, void* stream) {
  return gemv_tma_entry(w, wf, x, y, M, N, K, ldx, ldy, norm_w, eps, norm_offset, bias, residual, ldr, act, lut, dtype,
                        pdl, err, stream, 0, 1, 0, nullptr, nullptr);
}

// Mixture-of-experts GEMV for small batches, ONE launch for all experts: the (token, choice) slots were sorted by
// expert on the device (ipex_moe_sort_slots: `order` [slots], `ranges` [experts][2] = first position, count); the
// persistent CTAs walk the experts that received tokens, stage those tokens' rows of x and stream the expert's
// weights once for up to eight of them (`max_rows` = most tokens one expert can get, at most the token count).
// gather: x row = order[pos] / x_div, else pos; scatter: y row = order[pos], else pos.  act != 0: gate/up
// interleaved row tiles, N / 2 output columns.
IPEX_API int ipex_moe_gemv_tma(const void* w_list, int wf, const void* ranges, const void* order, int experts,
                               int slots, int max_rows, const void* x, int x_div, int gather, int scatter, void* y,
                               int N, int K, int ldx, int ldy, int act, const float* lut, int dtype, int* err,
                               void* stream) {
  if (experts < 1 || slots < 1 || max_rows < 1 || x_div < 1 || (K % 64) != 0 || err == nullptr ||
      w_list == nullptr || ranges == nullptr || order == nullptr || wf == WF_F16 || wf == WF_BF16)
    return (int)cudaErrorInvalidValue;
  if ((ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return (int)cudaErrorInvalidValue;
  TmaArgs a;
  a.w = nullptr; a.x = x; a.y = y; a.norm_w = nullptr; a.bias = nullptr; a.residual = nullptr; a.lut = lut;
  a.err = err;
  a.M = max_rows < 8 ? max_rows : 8;
  a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = 0; a.eps = 0.f; a.norm_offset = 0.f;
  a.act = act; a.stages = 0; a.cps = 0;
  a.tp_rank = 0; a.tp_world = 1; a.tp_npad = 0; a.tp_bufs = nullptr; a.tp_flags = nullptr;
  a.moe_w = reinterpret_cast<const uint8_t* const*>(w_list);
  a.moe_ranges = reinterpret_cast<const int*>(ranges);
  a.moe_order = reinterpret_cast<const int*>(order);
  a.moe_experts = experts; a.moe_slots = slots; a.moe_gather = gather; a.moe_scatter = scatter; a.moe_xdiv = x_div;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) return (int)dispatch_wf<__half>(wf, a, s, false);
  if (dtype == DT_BF16) return (int)dispatch_wf<__nv_bfloat16>(wf, a, s, false);
  return (int)cudaErrorInvalidValue;
}

// Row-parallel GEMV fused with its all-reduce (tensor parallelism): every rank runs the same launch on its K-slice
// of the weight; the kernel exchanges the 16-row partial tiles through peer memory and every rank ends with the
// full sum (+ bias, + residual) in y.  tp_bufs / tp_flags are device arrays of tp_world pointers into the ranks'
// symmetric buffers for the call's parity (two parities alternate between consecutive calls); the arrival
// counters must be zero before the first call and are left zero.  Bounded waits: *err = 4 if a peer never arrives.
IPEX_API int ipex_gemv_lowbit_tma_ar(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx,
                                     int ldy, const void* norm_w, float eps, float norm_offset, const void* bias,
                                     const void* residual, int ldr, const float* lut, int dtype, int pdl, int* err,
                                     void* stream, int tp_rank, int tp_world, int tp_npad, const void* tp_bufs,
                                     const void* tp_flags) {
  return gemv_tma_entry(w, wf, x, y, M, N, K, ldx, ldy, norm_w, eps, norm_offset, bias, residual, ldr, 0, lut, dtype,
                        pdl, err, stream, tp_rank, tp_world, tp_npad, tp_bufs, tp_flags);
}
