// Low-bit GEMV / skinny GEMM for decode (M <= 8), warp-private streaming version, sm_100a.
//
//   y[M, N] = epilogue( prologue(x)[M, K] * dequant(W)[N, K]^T )      W: symmetric int4 or fp8 e4m3 device tiles
//
// Same contract and tile layout as gemv_tma.cu.  That kernel splits every 16-row tile over sixteen warps, so at
// K = 4096 a warp multiplies two 1 KB chunks and then takes part in a sixteen-way reduction through shared-memory
// atomics and tickets: ~220 warp instructions per chunk, of which fewer than half are the contraction, and a marginal
// streaming rate of ~2.75 TB/s.  Here the bookkeeping is taken out of the K loop:
//   * every warp owns a ring of stages and its own mbarriers; lane 0 refills a stage right after the warp has read
//     it (cp.async.bulk, global -> shared), so the K loop has no cross-warp synchronisation at all and the first
//     stages are requested before griddepcontrol.wait (weights never depend on the previous kernel);
//   * a tile is shared by `wpt` warps (1, 2, 4, 8 or 16, chosen on the host so that all warps of the GPU have work):
//     each takes a contiguous range of the tile's K chunks, accumulates it in registers, and the partial tiles meet
//     once per tile in a double-buffered shared buffer behind a named barrier of just those warps;
//   * activations are staged once per CTA as 15-bit integers (int8 hi / lo rows) or e4m3 hi / lo rows, and hi / lo of
//     a token are two B columns of the same tensor-core instruction (mma.sync m16n8k32 s8 / e4m3), so one MMA per 512
//     weights serves up to four tokens; five to eight tokens use a second MMA on the same weight operands.
// Every mbarrier wait is bounded; on expiry the warp records an error code in *err, stops multiplying and keeps
// attending the barriers of its group so that nobody waits for it.
#include "common/utils.cuh"
#include <cuda_fp8.h>

namespace {

#ifndef IPEX_GEMV_STREAM_WARPS
#define IPEX_GEMV_STREAM_WARPS 16
#endif
// Warps per CTA (all of them stream and multiply).  Sixteen, one CTA per SM.  Eight-warp CTAs, two per SM (so that
// under programmatic dependent launch the next kernel's CTAs can become resident while this one drains) measured
// slower on every shape: fused qkv of a 7B model 12.0 us against 10.4 us, 7B decode 2.22 ms per token against 1.95.
constexpr int kW = IPEX_GEMV_STREAM_WARPS;
constexpr int kCtasPerSM = 16 / kW;
constexpr int kThreads = kW * 32;
constexpr int kSpin = 1 << 22;
constexpr int kPad = 64;            // extra bytes per staged activation row (bank spread)
constexpr int WFK_I8 = 0, WFK_FP8 = 1;

struct StreamArgs {
  const uint8_t* w;
  const void* x;
  void* y;
  const void* norm_w;
  const void* bias;
  const void* residual;
  int* err;
  int M, N, K;
  int ldx, ldy, ldr;
  float eps, norm_offset;
  int act;      // 0 none, 1 silu(gate)*up, 2 gelu_tanh(gate)*up  (row tiles interleaved gate, up)
  int stages;   // ring depth of a warp
  int cpw;      // 128-k chunks per stage
  int wpt;      // warps per tile
  // row-parallel layers of a tensor-parallel model: all-reduce fused over NVLink peer memory (tp_world > 1)
  int tp_rank, tp_world, tp_npad;
  float* const* tp_bufs;   // [tp_world] device pointers: rank r's partial buffer [tp_world][8][tp_npad] fp32
  int* const* tp_flags;    // [tp_world] device pointers: rank r's per-tile arrival counters
  // mixture-of-experts mode (moe_ranges != null): ONE launch walks every expert that received tokens.  The (token,
  // choice) slots are sorted by expert: moe_ranges[e] = (first position, count) in moe_order.  A pass = one expert
  // and up to M of its tokens: the CTA stages those rows of x and every warp group streams its share of the
  // expert's row tiles; the rings run ahead across passes.  x row = moe_order[pos] / moe_xdiv (moe_gather) or pos;
  // y row = moe_order[pos] (moe_scatter) or pos.
  const uint8_t* const* moe_w;
  const int* moe_ranges;
  const int* moe_order;
  int moe_experts, moe_slots, moe_gather, moe_scatter, moe_xdiv;
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
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
    if (i >= 8) __nanosleep(i < 64 ? 20 : 100);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void group_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D = A * B + {c0, c1, c0, c1}: a token's accumulator seeds (hi, lo) start rows g and g + 8 alike
__device__ __forceinline__ void mma_s8_seed(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1, int c0, int c1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == 1) return g / (1.0f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.0f + tanhf(k0 * (g + k1 * g * g * g)));
}

// ------------------------------------------------------------------------------------------------------------------
// Activation staging, all 512 threads.  Token m becomes two byte rows of xq (2m: hi, 2m + 1: lo), a scale dxs[m], and
// (int8 path) per-(64-group, token) accumulator seeds (-8 sum hi, -8 sum lo) that apply the "- 8" of the codes.
//   int8 : xi = round(x / dx) in [-16383, 16383], hi = xi >> 7, lo = xi & 127, bytes in the octet order
//          (k0,k4,k1,k5 | k2,k6,k3,k7) of the masked weight words;
//   fp8  : hi = e4m3(x / dx), lo = e4m3(x / dx - hi), natural k order.
// RMS norm fused (norm_w != null); rows zero padded to Kp.  scratch: [M][2][kW] floats.  xrow (expert mode): the rows
// of x to stage; M rows (a.M is only the capacity there).
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int WFK>
__device__ void stage_x(const StreamArgs& a, int M, const int* xrow, uint8_t* xq, int2* seeds, int NT, float* dxs,
                        float* scratch, int Kp) {
  const int tid = threadIdx.x;
  const T* x = reinterpret_cast<const T*>(a.x);
  const T* nw = reinterpret_cast<const T*>(a.norm_w);
  const int nvec = a.K / 8;   // K % 64 == 0
  const int stride = Kp + kPad;
  const int groups = Kp / 64;
  if (WFK == WFK_I8)
    for (int i = tid; i < groups * NT; i += kThreads)
      if ((i % NT) >= M) seeds[i] = make_int2(0, 0);
  // The sixteen warps split into one team per row (sixteen, eight, four or two warps each), so the rows are
  // staged side by side: every global load of a row is in flight at once instead of row after row.
  const int warp = tid >> 5;
  const int mp2 = M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
  const int wpr = kW / mp2 > 0 ? kW / mp2 : 1;                     // warps per row
  const int m = warp / wpr;                                         // this thread's first row (>= M: none)
  const int tr = (warp % wpr) * 32 + (tid & 31), team = wpr * 32;
  const T* xr = x + (size_t)(m < M ? (xrow != nullptr ? xrow[m] : m) : 0) * a.ldx;
  // pass 1: sum of squares and largest |x * w| of the row
  if (m < M) {
    float ss = 0.f, mx = 0.f;
    for (int v = tr; v < nvec; v += team) {
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
    if ((tid & 31) == 0) {
      scratch[(m * 2) * kW + (warp % wpr)] = ss;
      scratch[(m * 2 + 1) * kW + (warp % wpr)] = mx;
    }
  }
  __syncthreads();
  // pass 2: quantize
  if (m < M) {
    float tot = 0.f, amax = 0.f;
    for (int w = 0; w < wpr; w++) {
      tot += scratch[(m * 2) * kW + w];
      amax = fmaxf(amax, scratch[(m * 2 + 1) * kW + w]);
    }
    const float rstd = nw != nullptr ? rsqrtf(tot / (float)a.K + a.eps) : 1.0f;
    amax *= rstd;
    const float top = WFK == WFK_I8 ? 16383.f : 448.f;
    const float dx = amax > 0.f ? amax / top : 1.0f;
    const float inv = rstd / dx;
    if (tr == 0) dxs[m] = dx;
    uint8_t* xh = xq + (size_t)(2 * m) * stride;
    uint8_t* xl = xq + (size_t)(2 * m + 1) * stride;
    for (int v0 = 0; v0 < Kp / 8; v0 += team) {
      const int v = v0 + tr;
      int sh = 0, sl = 0;
      if (v < Kp / 8) {
        uint32_t ph[2] = {0, 0}, pl[2] = {0, 0};
        if (v < nvec) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
          const T* e = reinterpret_cast<const T*>(&raw);
          uint4 wraw = make_uint4(0, 0, 0, 0);
          if (nw != nullptr) wraw = *reinterpret_cast<const uint4*>(nw + v * 8);
          const T* we = reinterpret_cast<const T*>(&wraw);
          if constexpr (WFK == WFK_I8) {
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
          } else {
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
              const float r0 = f0 - __half2float(__ushort_as_half(hr.x));
              const float r1 = f1 - __half2float(__ushort_as_half(hr.y));
              const __nv_fp8x2_storage_t l = __nv_cvt_float2_to_fp8x2(make_float2(r0, r1), __NV_SATFINITE, __NV_E4M3);
              ph[j >> 2] |= (uint32_t)h << (16 * ((j >> 1) & 1));
              pl[j >> 2] |= (uint32_t)l << (16 * ((j >> 1) & 1));
            }
          }
        }
        *reinterpret_cast<uint2*>(xh + v * 8) = make_uint2(ph[0], ph[1]);
        *reinterpret_cast<uint2*>(xl + v * 8) = make_uint2(pl[0], pl[1]);
      }
      if constexpr (WFK == WFK_I8) {
        // 8 consecutive octets (= 8 consecutive lanes) form a 64-group
        sh += __shfl_xor_sync(0xffffffffu, sh, 1); sl += __shfl_xor_sync(0xffffffffu, sl, 1);
        sh += __shfl_xor_sync(0xffffffffu, sh, 2); sl += __shfl_xor_sync(0xffffffffu, sl, 2);
        sh += __shfl_xor_sync(0xffffffffu, sh, 4); sl += __shfl_xor_sync(0xffffffffu, sl, 4);
        if ((tid & 7) == 0 && v < Kp / 8) seeds[(v >> 3) * NT + m] = make_int2(-8 * sh, -8 * sl);
      }
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------------------------
// One stage (nch chunks of one 16-row tile, starting at chunk c0 of the row) by one warp.
// acc[h][0] += row g, acc[h][1] += row g + 8 of token t + 4h (unscaled by the token's dx).
// ------------------------------------------------------------------------------------------------------------------
template <int MH>
__device__ __forceinline__ void stage_mma_i8(const uint8_t* st, int cpw, int nch, int c0, const uint8_t* xq,
                                             const int2* seeds, int M, int stride, float (&acc)[MH][2]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr uint32_t kM = 0x0F0F0F0Fu;
  constexpr int NT = 4 * MH;
  const uint8_t* sc = st + cpw * 1024;
  const bool has_x0 = g < 2 * (M < 4 ? M : 4);
  const bool has_x1 = MH > 1 && g < 2 * (M - 4);
  const uint8_t* xrow0 = xq + (size_t)g * stride + 16 * t;
  const uint8_t* xrow1 = xq + (size_t)(g + 8) * stride + 16 * t;
#pragma unroll 2
  for (int ch = 0; ch < nch; ch++) {
    const int cg = c0 + ch;
    const uint8_t* tp = st + ch * 1024;
    const uint4 qa = *reinterpret_cast<const uint4*>(tp + g * 64 + t * 16);
    const uint4 qb = *reinterpret_cast<const uint4*>(tp + (g + 8) * 64 + t * 16);
    const uint32_t s0 = *reinterpret_cast<const uint32_t*>(sc + ch * 64 + (0 * 16 + 2 * g) * 2);
    const uint32_t s1 = *reinterpret_cast<const uint32_t*>(sc + ch * 64 + (1 * 16 + 2 * g) * 2);
    const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
    const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));
    const uint32_t a00 = qa.x & kM, a01 = qb.x & kM, a02 = (qa.x >> 4) & kM, a03 = (qb.x >> 4) & kM;
    const uint32_t a10 = qa.z & kM, a11 = qb.z & kM, a12 = (qa.z >> 4) & kM, a13 = (qb.z >> 4) & kM;
    const uint32_t a20 = qa.y & kM, a21 = qb.y & kM, a22 = (qa.y >> 4) & kM, a23 = (qb.y >> 4) & kM;
    const uint32_t a30 = qa.w & kM, a31 = qb.w & kM, a32 = (qa.w >> 4) & kM, a33 = (qb.w >> 4) & kM;
#pragma unroll
    for (int h = 0; h < MH; h++) {
      uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
      if (h == 0 ? has_x0 : has_x1) {
        const uint8_t* xr = h == 0 ? xrow0 : xrow1;
        xa = *reinterpret_cast<const uint4*>(xr + cg * 128);
        xb = *reinterpret_cast<const uint4*>(xr + cg * 128 + 64);
      }
      const int2 sd0 = seeds[(2 * cg) * NT + 4 * h + t];
      const int2 sd1 = seeds[(2 * cg + 1) * NT + 4 * h + t];
      int c0v[4], c1v[4];
      mma_s8_seed(c0v, a00, a01, a02, a03, xa.x, xa.y, sd0.x, sd0.y);
      mma_s8_seed(c1v, a10, a11, a12, a13, xb.x, xb.y, sd1.x, sd1.y);
      mma_s8(c0v, a20, a21, a22, a23, xa.z, xa.w);
      mma_s8(c1v, a30, a31, a32, a33, xb.z, xb.w);
      acc[h][0] += d0.x * (float)(c0v[0] * 128 + c0v[1]) + d1.x * (float)(c1v[0] * 128 + c1v[1]);
      acc[h][1] += d0.y * (float)(c0v[2] * 128 + c0v[3]) + d1.y * (float)(c1v[2] * 128 + c1v[3]);
    }
  }
}

// fp8 e4m3 weights against the e4m3 (hi, lo) activation rows: no conversion of the codes at all.  A 128-k chunk is
// two [16 rows][64 B] tiles in natural k order; a lane's 16 bytes of a weight row and the same 16 bytes of an
// activation row are the operands of two m16n8k32 MMAs (the contraction order of the instruction is permuted the
// same way on both sides, which leaves the sum unchanged).  One fp32 scale per (row, 128 k).
template <int MH>
__device__ __forceinline__ void stage_mma_fp8(const uint8_t* st, int cpw, int nch, int c0, const uint8_t* xq, int M,
                                              int stride, float (&acc)[MH][2]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint8_t* sc = st + cpw * 2048;
  const bool has_x0 = g < 2 * (M < 4 ? M : 4);
  const bool has_x1 = MH > 1 && g < 2 * (M - 4);
  const uint8_t* xrow0 = xq + (size_t)g * stride + 16 * t;
  const uint8_t* xrow1 = xq + (size_t)(g + 8) * stride + 16 * t;
#pragma unroll 2
  for (int ch = 0; ch < nch; ch++) {
    const int cg = c0 + ch;
    const uint8_t* tp = st + ch * 2048 + g * 64 + t * 16;
    const uint4 qa0 = *reinterpret_cast<const uint4*>(tp);
    const uint4 qb0 = *reinterpret_cast<const uint4*>(tp + 512);
    const uint4 qa1 = *reinterpret_cast<const uint4*>(tp + 1024);
    const uint4 qb1 = *reinterpret_cast<const uint4*>(tp + 1536);
    const float2 d = *reinterpret_cast<const float2*>(sc + ch * 64 + 2 * g * 4);
#pragma unroll
    for (int h = 0; h < MH; h++) {
      uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
      if (h == 0 ? has_x0 : has_x1) {
        const uint8_t* xr = h == 0 ? xrow0 : xrow1;
        x0 = *reinterpret_cast<const uint4*>(xr + cg * 128);
        x1 = *reinterpret_cast<const uint4*>(xr + cg * 128 + 64);
      }
      float c0v[4] = {0.f, 0.f, 0.f, 0.f}, c1v[4] = {0.f, 0.f, 0.f, 0.f};
      mma_e4m3(c0v, qa0.x, qb0.x, qa0.y, qb0.y, x0.x, x0.y);
      mma_e4m3(c1v, qa1.x, qb1.x, qa1.y, qb1.y, x1.x, x1.y);
      mma_e4m3(c0v, qa0.z, qb0.z, qa0.w, qb0.w, x0.z, x0.w);
      mma_e4m3(c1v, qa1.z, qb1.z, qa1.w, qb1.w, x1.z, x1.w);
      acc[h][0] += d.x * ((c0v[0] + c0v[1]) + (c1v[0] + c1v[1]));
      acc[h][1] += d.y * ((c0v[2] + c0v[3]) + (c1v[2] + c1v[3]));
    }
  }
}

// Position of a warp in its sequence of stages: unit (RT consecutive row tiles), tile of the unit, stage of the tile.
struct Walk {
  int unit, r, sp;
  // expert mode: the pass (expert e, its tokens [base, base + M) of cnt, first position `first` in the sorted
  // order, pidx = passes so far); a plain GEMV is one pass
  int e, base, cnt, first, pidx;
  const uint8_t* w;   // weight matrix of the pass (looked up once per pass, not per stage)
};

template <typename T, int WFK, int RT, int MH, bool MOE /* expert walk compiled in */>
__global__ void __launch_bounds__(kThreads, kCtasPerSM) gemv_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int CB = WFK == WFK_I8 ? 1024 : 2048;   // code bytes per 128-k chunk of a row tile
  constexpr int SB = 64;                            // scale bytes per chunk
  constexpr int NT = 4 * MH;
  const int Kp = (int)ceil_to_i64(a.K, 128);
  const int Np = (int)ceil_to_i64(a.N, 16);
  const int chunks = Kp / 128;
  const int stride = Kp + kPad;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int S = a.stages, CPW = a.cpw, wpt = a.wpt;
  const int stage_bytes = CPW * (CB + SB);
  const int ntiles = Np / 16;
  const int nunits = (ntiles + RT - 1) / RT;
  const int G = kW / wpt, grp = warp / wpt, wi = warp % wpt;
  // this warp's chunks of every tile, and how many stages they make
  const int cper = (chunks + wpt - 1) / wpt;
  const int cbeg = wi * cper < chunks ? wi * cper : chunks;
  const int cend = cbeg + cper < chunks ? cbeg + cper : chunks;
  const int spt = (cend - cbeg + CPW - 1) / CPW;
  const int ustep = gridDim.x * G;

  // shared memory: rings | barriers | xq | seeds | dxs | scratch | reduction buffers
  uint8_t* ring = smem_raw + (size_t)warp * S * stage_bytes;
  size_t off = (size_t)kW * S * stage_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + off) + warp * S;
  off += (size_t)kW * S * sizeof(uint64_t);
  off = (off + 15) & ~(size_t)15;
  uint8_t* xq = smem_raw + off;
  off += ((size_t)2 * a.M * stride + 15) & ~(size_t)15;
  int2* seeds = reinterpret_cast<int2*>(smem_raw + off);
  if (WFK == WFK_I8) off += (size_t)(Kp / 64) * NT * sizeof(int2);
  float* dxs = reinterpret_cast<float*>(smem_raw + off);
  off += 32;
  float* scratch = reinterpret_cast<float*>(smem_raw + off);
  off += (size_t)8 * 2 * kW * sizeof(float);
  int* xrow = reinterpret_cast<int*>(smem_raw + off);      // expert mode: rows of x / y of the pass, [2][8]
  int* yrow = xrow + 8;
  off += 64;
  float* red = reinterpret_cast<float*>(smem_raw + off);   // [G][2][wpt][RT * MH * 2][32] when wpt > 1

  const bool moe = MOE;
  const int Mcap = a.M;
  const size_t code_bytes = (size_t)Np * chunks * CB / 16;

  // lane 0 requests stage `w` of this warp into ring slot `slot`
  auto issue = [&](const Walk& w, int slot) {
    const uint8_t* codes = w.w;
    const uint8_t* scales = codes + code_bytes;
    const int tile = w.unit * RT + w.r;
    const int c0 = cbeg + w.sp * CPW;
    const int nch = cend - c0 < CPW ? cend - c0 : CPW;
    uint8_t* dst = ring + (size_t)slot * stage_bytes;
    mbar_expect_tx(&full[slot], (uint32_t)(nch * (CB + SB)));
    const size_t chunk_index = (size_t)tile * chunks + c0;
    bulk_g2s(dst, codes + chunk_index * CB, (uint32_t)(nch * CB), &full[slot]);
    bulk_g2s(dst + CPW * CB, scales + chunk_index * SB, (uint32_t)(nch * SB), &full[slot]);
  };
  // next pass of the launch (false when there is none); sets the first unit of this warp's group in it.  Units are
  // dealt round-robin over the CTAs, continuing where the previous pass stopped.
  auto next_pass = [&](Walk& w) {
    if (!moe) {
      if (w.pidx >= 0) return false;
      w.w = a.w;
    } else {
      bool found = false;
      if (w.pidx >= 0) {
        w.base += Mcap;
        found = w.base < w.cnt;
      }
      if (!found) {
        for (++w.e; w.e < a.moe_experts; ++w.e) {
          int cnt = a.moe_ranges[2 * w.e + 1];
          cnt = cnt < a.moe_slots ? cnt : a.moe_slots;
          if (cnt > 0) {
            w.cnt = cnt;
            w.first = a.moe_ranges[2 * w.e];
            w.base = 0;
            w.w = a.moe_w[w.e];
            found = true;
            break;
          }
        }
      }
      if (!found) return false;
    }
    w.pidx++;
    const int goff = moe ? (int)(((long long)w.pidx * nunits) % gridDim.x) : 0;
    w.unit = (int)((blockIdx.x + gridDim.x - goff) % gridDim.x) + gridDim.x * grp;
    w.r = 0;
    w.sp = 0;
    return true;
  };
  // first / next stage of the warp's sequence; false when the sequence has ended
  auto first_stage = [&](Walk& w) {
    if (spt <= 0) return false;
    while (next_pass(w))
      if (w.unit < nunits) return true;
    return false;
  };
  auto advance = [&](Walk& w) {
    if (++w.sp < spt) return true;
    w.sp = 0;
    if (++w.r < RT && w.unit * RT + w.r < ntiles) return true;
    w.r = 0;
    w.unit += ustep;
    if (w.unit < nunits) return true;
    while (next_pass(w))
      if (w.unit < nunits) return true;
    return false;
  };

  Walk iw = {0, 0, 0, -1, 0, 0, 0, -1, nullptr};
  bool more = false;   // stages left to request (lane 0)
  if (moe) pdl_wait();   // the expert ranges come from the kernel before this one
  if (lane == 0) {
    for (int s = 0; s < S; s++) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // fill the ring before waiting for the previous kernel: the weights do not depend on it
    more = first_stage(iw);
    for (int s = 0; s < S && more; s++) {
      issue(iw, s);
      more = advance(iw);
    }
  }
  __syncwarp();
  pdl_launch_dependents();
  pdl_wait();
  if (!moe) stage_x<T, WFK>(a, a.M, nullptr, xq, seeds, NT, dxs, scratch, Kp);

  T* y = reinterpret_cast<T*>(a.y);
  bool ok = true;
  int slot = 0;
  uint32_t phase = 0;
  int nu = 0;   // units done (parity of the reduction buffer)

  // ---- fused all-reduce (row-parallel layers, RT == 1): the finishing warp of a tile pushes its partial sums into
  // slot [tp_rank] of EVERY rank's buffer (plain stores to the peers' mapped memory) and release-increments the
  // tile's arrival counter on every rank.  It collects the tile one unit later (tp_collect), after it has streamed
  // the next tile, so the NVLink round trip and the skew between the ranks hide behind its own work.
  int tp_pending = -1;
  auto tp_collect = [&](int unit) {
    int* my_flag = a.tp_flags[a.tp_rank] + unit;
    int arrived = 0;
    if (lane == 0) {
      for (int i = 0; i < kSpin; i++) {
        if (ld_acquire_sys(my_flag) >= a.tp_world) { arrived = 1; break; }
        __nanosleep(64);
      }
      if (arrived) *my_flag = 0;   // self-cleaning: the next user of this counter is two launches away
      else atomicExch(a.err, 4);
    }
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (!arrived) return;
    const float* src = a.tp_bufs[a.tp_rank];
#pragma unroll
    for (int h = 0; h < MH; h++) {
      const int m = t + 4 * h;
      if (m >= a.M) continue;
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int n = unit * 16 + g + 8 * half;
        if (n >= a.N) continue;
        float sv = 0.f;
        for (int rk = 0; rk < a.tp_world; rk++) sv += ld_relaxed_sys_f32(src + ((size_t)rk * 8 + m) * a.tp_npad + n);
        if (a.bias != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[n]);
        if (a.residual != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(a.residual)[(size_t)m * a.ldr + n]);
        y[(size_t)m * a.ldy + n] = DT<T>::from_f(sv);
      }
    }
  };

  Walk cw = {0, 0, 0, -1, 0, 0, 0, -1, nullptr};
  int M = a.M;          // rows of the current pass
  while (next_pass(cw)) {
    if (moe) {
      __syncthreads();    // every warp is done with the previous pass's rows
      M = cw.cnt - cw.base < Mcap ? cw.cnt - cw.base : Mcap;
      if (tid < M) {
        const int pos = cw.first + cw.base + tid;
        int slot = a.moe_order[pos];
        slot = slot < 0 ? 0 : (slot >= a.moe_slots ? a.moe_slots - 1 : slot);
        xrow[tid] = a.moe_gather ? slot / a.moe_xdiv : pos;
        yrow[tid] = a.moe_scatter ? slot : pos;
      }
      __syncthreads();
      stage_x<T, WFK>(a, M, xrow, xq, seeds, NT, dxs, scratch, Kp);
    }
    for (int unit = cw.unit; unit < nunits; unit += ustep, nu++) {
      float acc[RT][MH][2];
#pragma unroll
      for (int r = 0; r < RT; r++)
#pragma unroll
        for (int h = 0; h < MH; h++) acc[r][h][0] = acc[r][h][1] = 0.f;
#pragma unroll
      for (int r = 0; r < RT; r++) {
        if (unit * RT + r >= ntiles) break;
        for (int sp = 0; sp < spt; sp++) {
          if (ok && !mbar_wait(&full[slot], phase)) {
            if (lane == 0) atomicExch(a.err, 2);
            ok = false;
          }
          if (ok) {
            const int c0 = cbeg + sp * CPW;
            const int nch = cend - c0 < CPW ? cend - c0 : CPW;
            const uint8_t* st = ring + (size_t)slot * stage_bytes;
            if constexpr (WFK == WFK_I8) stage_mma_i8<MH>(st, CPW, nch, c0, xq, seeds, M, stride, acc[r]);
            else stage_mma_fp8<MH>(st, CPW, nch, c0, xq, M, stride, acc[r]);
          }
          __syncwarp();
          if (lane == 0 && ok && more) {
            // the warp's reads of this slot (generic proxy) are ordered before the refill (async proxy)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(iw, slot);
            more = advance(iw);
          }
          if (++slot == S) { slot = 0; phase ^= 1; }
        }
      }
      // ---- the wpt partial tiles meet in shared memory; warp 0 of the group finishes the unit ----
      if (wpt > 1) {
        float* buf = red + ((size_t)(grp * 2 + (nu & 1)) * wpt) * (RT * MH * 2 * 32);
        if (wi != 0) {
#pragma unroll
          for (int r = 0; r < RT; r++)
#pragma unroll
            for (int h = 0; h < MH; h++) {
              buf[((size_t)wi * RT * MH * 2 + (r * MH + h) * 2 + 0) * 32 + lane] = acc[r][h][0];
              buf[((size_t)wi * RT * MH * 2 + (r * MH + h) * 2 + 1) * 32 + lane] = acc[r][h][1];
            }
        }
        group_sync(1 + grp, wpt * 32);
        if (wi != 0) continue;
        for (int w = 1; w < wpt; w++) {
#pragma unroll
          for (int r = 0; r < RT; r++)
#pragma unroll
            for (int h = 0; h < MH; h++) {
              acc[r][h][0] += buf[((size_t)w * RT * MH * 2 + (r * MH + h) * 2 + 0) * 32 + lane];
              acc[r][h][1] += buf[((size_t)w * RT * MH * 2 + (r * MH + h) * 2 + 1) * 32 + lane];
            }
        }
      }
      if (RT == 1 && a.tp_world > 1) {
        if (tp_pending >= 0) tp_collect(tp_pending);
        tp_pending = -1;
        if (!ok) continue;
        for (int rk = 0; rk < a.tp_world; rk++) {
          float* dst = a.tp_bufs[rk] + (size_t)a.tp_rank * 8 * a.tp_npad;
#pragma unroll
          for (int h = 0; h < MH; h++) {
            const int m = t + 4 * h;
            if (m >= a.M) continue;
            const float dx = dxs[m];
#pragma unroll
            for (int half = 0; half < 2; half++) {
              const int n = unit * 16 + g + 8 * half;
              if (n < a.N) dst[(size_t)m * a.tp_npad + n] = acc[0][h][half] * dx;
            }
          }
        }
        __threadfence_system();
        __syncwarp();
        if (lane < a.tp_world) red_release_sys_add(a.tp_flags[lane] + unit, 1);
        tp_pending = unit;
        continue;
      }
      if (!ok) continue;
      // ---- epilogue: lane (g, t) holds rows g and g + 8 of the unit's tiles for tokens t and t + 4 ----
#pragma unroll
      for (int h = 0; h < MH; h++) {
        const int m = t + 4 * h;
        if (m >= M) continue;
        const float dx = dxs[m];
        const size_t ym = moe ? (size_t)yrow[m] : (size_t)m;   // output row of token m
        if (RT == 2 && a.act != 0) {
#pragma unroll
          for (int half = 0; half < 2; half++) {
            const int row = g + 8 * half;
            const int n = unit * 16 + row;
            if (n >= a.N / 2) continue;
            float gsum = acc[0][h][half] * dx, usum = acc[RT - 1][h][half] * dx;
            if (a.bias != nullptr) {
              gsum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)unit * 32 + row]);
              usum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)unit * 32 + 16 + row]);
            }
            y[ym * a.ldy + n] = DT<T>::from_f(act_apply(gsum, a.act) * usum);
          }
        } else {
#pragma unroll
          for (int r = 0; r < RT; r++)
#pragma unroll
            for (int half = 0; half < 2; half++) {
              const int n = (unit * RT + r) * 16 + g + 8 * half;
              if (n >= a.N) continue;
              float sv = acc[r][h][half] * dx;
              if (a.bias != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[n]);
              if (a.residual != nullptr)
                sv += DT<T>::to_f(reinterpret_cast<const T*>(a.residual)[(size_t)m * a.ldr + n]);
              y[ym * a.ldy + n] = DT<T>::from_f(sv);
            }
        }
      }
    }
  }  // passes
  if (tp_pending >= 0) tp_collect(tp_pending);
}

struct Plan {
  int stages, cpw, wpt, grid;
  size_t smem;
};

int g_ring_kb = 168 / kCtasPerSM;   // shared memory of one CTA given to its warps' rings (ipex_gemv_stream_tune)
int g_cpw = 0;         // chunks per stage, 0 = automatic
int g_wpt = 0;         // warps per tile, 0 = automatic

template <int WFK, int RT, int MH>
bool make_plan(const StreamArgs& a, Plan& p) {
  constexpr int CB = WFK == WFK_I8 ? 1024 : 2048;
  const int Kp = (int)ceil_to_i64(a.K, 128), Np = (int)ceil_to_i64(a.N, 16);
  const int chunks = Kp / 128;
  const int nunits = (Np / 16 + RT - 1) / RT;
  const int sms = 148 * kCtasPerSM;
  p.grid = nunits < sms ? nunits : sms;
  // warps per tile: as few as keep every warp of the GPU busy (a warp needs at least two chunks of the tile).
  // Wider splits balance the groups of an SM better on paper but did not measure faster (more reductions, shorter
  // uninterrupted runs per warp).
  int wpt = g_wpt;
  if (wpt <= 0) {
    wpt = 1;
    while (wpt < kW && (int64_t)nunits * wpt < (int64_t)p.grid * kW && 2 * wpt <= chunks) wpt *= 2;
  }
  while (wpt > 1 && 2 * wpt > chunks) wpt /= 2;
  p.wpt = wpt;
  const int cper = (chunks + wpt - 1) / wpt;
  size_t fixed = (size_t)kW * 16 * 8 + 16 + (((size_t)2 * a.M * (Kp + kPad) + 15) & ~(size_t)15) + 32 +
                 (size_t)8 * 2 * kW * 4 + 64 + 128;
  if (WFK == WFK_I8) fixed += (size_t)(Kp / 64) * 4 * MH * 8;
  if (wpt > 1) fixed += (size_t)kW * 2 * RT * MH * 2 * 32 * 4;
  const size_t cap = 227 * 1024;
  if (fixed + (size_t)kW * 2 * (CB + 64) > cap) return false;
  size_t ring = (size_t)g_ring_kb * 1024;
  if (fixed + ring > cap) ring = cap - fixed;
  const size_t per_warp = ring / kW;
  // stage size: at most the warp's share of a tile, about a third of its ring, at least one chunk
  int cpw = g_cpw > 0 ? g_cpw : (int)(per_warp / 3 / (CB + 64));
  if (cpw > cper) cpw = cper;
  if (cpw > 8) cpw = 8;
  if (cpw < 1) cpw = 1;
  int stages = (int)(per_warp / ((size_t)cpw * (CB + 64)));
  if (stages > 16) stages = 16;
  if (stages < 2) return false;
  p.cpw = cpw;
  p.stages = stages;
  p.smem = fixed + (size_t)kW * stages * cpw * (CB + 64);
  return p.smem <= cap;
}

template <typename T, int WFK, int RT, int MH>
cudaError_t launch_stream(StreamArgs a, cudaStream_t stream, bool pdl) {
  Plan p;
  if (!make_plan<WFK, RT, MH>(a, p)) return cudaErrorInvalidValue;
  a.stages = p.stages;
  a.cpw = p.cpw;
  a.wpt = p.wpt;
  auto kern = a.moe_ranges != nullptr ? gemv_stream_kernel<T, WFK, RT, 1, true> : gemv_stream_kernel<T, WFK, RT, MH, false>;
  if (p.smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
    if (e != cudaSuccess) return e;
  }
  return launch_kernel(kern, dim3(p.grid), dim3(kThreads), p.smem, stream, pdl, a);
}

template <typename T, int WFK>
cudaError_t dispatch(const StreamArgs& a, cudaStream_t s, bool pdl) {
  if (a.act != 0) {
    return a.M <= 4 ? launch_stream<T, WFK, 2, 1>(a, s, pdl) : launch_stream<T, WFK, 2, 2>(a, s, pdl);
  }
  return a.M <= 4 ? launch_stream<T, WFK, 1, 1>(a, s, pdl) : launch_stream<T, WFK, 1, 2>(a, s, pdl);
}

}  // namespace

// Process-wide tuning: shared memory given to the rings (<= 0 keeps it), chunks per stage and warps per tile
// (0 = automatic, negative keeps the setting).
IPEX_API void ipex_gemv_stream_tune(int ring_kb, int chunks_per_stage, int warps_per_tile) {
  if (ring_kb > 0) g_ring_kb = ring_kb > 200 ? 200 : ring_kb;
  if (chunks_per_stage >= 0) g_cpw = chunks_per_stage > 8 ? 8 : chunks_per_stage;
  if (warps_per_tile >= 0 && (warps_per_tile & (warps_per_tile - 1)) == 0 && warps_per_tile <= kW)
    g_wpt = warps_per_tile;
}

// Same arguments as ipex_gemv_lowbit_tma (+ the tensor-parallel ones of ipex_gemv_lowbit_tma_ar); weight families:
// symmetric int4 and fp8 e4m3.  Returns cudaErrorInvalidValue for anything else or when the staged activations
// leave no room for the rings (the caller then uses the other GEMV kernels).
// *err: 2 = a bounded wait for weight data expired, 4 = a peer's partial tile never arrived.
static int stream_entry(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx, int ldy,
                        const void* norm_w, float eps, float norm_offset, const void* bias, const void* residual,
                        int ldr, int act, int dtype, int pdl, int* err, void* stream, int tp_rank, int tp_world,
                        int tp_npad, const void* tp_bufs, const void* tp_flags) {
  if (M < 1 || M > 8 || N < 1 || (K % 64) != 0 || err == nullptr) return (int)cudaErrorInvalidValue;
  if ((ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return (int)cudaErrorInvalidValue;
  if (wf != WF_SYM_INT4 && wf != WF_FP8_E4M3) return (int)cudaErrorInvalidValue;
  if (wf == WF_FP8_E4M3 && (K % 128) != 0) return (int)cudaErrorInvalidValue;
  if (act != 0 && (N % 32) != 0) return (int)cudaErrorInvalidValue;
  if (tp_world > 1 && (act != 0 || tp_bufs == nullptr || tp_flags == nullptr || tp_npad < N || tp_world > 8))
    return (int)cudaErrorInvalidValue;
  StreamArgs a;
  a.w = (const uint8_t*)w; a.x = x; a.y = y; a.norm_w = norm_w; a.bias = bias; a.residual = residual;
  a.err = err;
  a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = ldr; a.eps = eps; a.norm_offset = norm_offset;
  a.act = act; a.stages = 0; a.cpw = 0; a.wpt = 1;
  a.tp_rank = tp_rank; a.tp_world = tp_world; a.tp_npad = tp_npad;
  a.tp_bufs = reinterpret_cast<float* const*>(tp_bufs);
  a.tp_flags = reinterpret_cast<int* const*>(tp_flags);
  a.moe_w = nullptr; a.moe_ranges = nullptr; a.moe_order = nullptr;
  a.moe_experts = 0; a.moe_slots = 0; a.moe_gather = 0; a.moe_scatter = 0; a.moe_xdiv = 1;
  cudaStream_t s = (cudaStream_t)stream;
  auto run = [&](const StreamArgs& b, bool dep) -> int {
    if (dtype == DT_F16) {
      return wf == WF_SYM_INT4 ? (int)dispatch<__half, WFK_I8>(b, s, dep) : (int)dispatch<__half, WFK_FP8>(b, s, dep);
    }
    if (dtype == DT_BF16) {
      return wf == WF_SYM_INT4 ? (int)dispatch<__nv_bfloat16, WFK_I8>(b, s, dep)
                               : (int)dispatch<__nv_bfloat16, WFK_FP8>(b, s, dep);
    }
    return (int)cudaErrorInvalidValue;
  };
  int rc = run(a, pdl != 0);
  if (rc != (int)cudaErrorInvalidValue || M <= 4 || tp_world > 1) return rc;
  // five to eight rows of a long contraction do not fit beside the rings: two launches of up to four rows each
  // (the weights are streamed twice, still far cheaper than leaving the pipelined kernels).  Not under tensor
  // parallelism: the arrival counters of a call serve one launch.
  const size_t es = 2;   // fp16 / bf16
  StreamArgs lo = a, hi = a;
  lo.M = 4;
  hi.M = M - 4;
  hi.x = reinterpret_cast<const uint8_t*>(x) + (size_t)4 * ldx * es;
  hi.y = reinterpret_cast<uint8_t*>(y) + (size_t)4 * ldy * es;
  if (residual != nullptr) hi.residual = reinterpret_cast<const uint8_t*>(residual) + (size_t)4 * ldr * es;
  rc = run(lo, pdl != 0);
  if (rc != 0) return rc;
  return run(hi, pdl != 0);
}

IPEX_API int ipex_gemv_lowbit_stream(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx,
                                     int ldy, const void* norm_w, float eps, float norm_offset, const void* bias,
                                     const void* residual, int ldr, int act, const float* lut, int dtype, int pdl,
                                     int* err, void* stream) {
  (void)lut;
  return stream_entry(w, wf, x, y, M, N, K, ldx, ldy, norm_w, eps, norm_offset, bias, residual, ldr, act, dtype, pdl,
                      err, stream, 0, 1, 0, nullptr, nullptr);
}

// Row-parallel GEMV fused with its all-reduce (tensor parallelism), same contract as ipex_gemv_lowbit_tma_ar: every
// rank runs the same launch on its K-slice of the weight; the finishing warp of a 16-row tile stores its partial
// sums into every rank's symmetric buffer over NVLink, bumps the tile's arrival counter on every rank, and collects
// the full sum (+ bias, + residual) one tile later.  tp_bufs / tp_flags are device arrays of tp_world pointers for
// the call's parity; the counters must be zero before the first call and are left zero.
IPEX_API int ipex_gemv_lowbit_stream_ar(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx,
                                        int ldy, const void* norm_w, float eps, float norm_offset, const void* bias,
                                        const void* residual, int ldr, const float* lut, int dtype, int pdl, int* err,
                                        void* stream, int tp_rank, int tp_world, int tp_npad, const void* tp_bufs,
                                        const void* tp_flags) {
  (void)lut;
  return stream_entry(w, wf, x, y, M, N, K, ldx, ldy, norm_w, eps, norm_offset, bias, residual, ldr, 0, dtype, pdl,
                      err, stream, tp_rank, tp_world, tp_npad, tp_bufs, tp_flags);
}

// Mixture-of-experts GEMV for small batches, ONE launch for all experts (same contract as ipex_moe_gemv_tma): the
// (token, choice) slots were sorted by expert on the device (ipex_moe_sort_slots: `order` [slots], `ranges`
// [experts][2] = first position, count); the CTAs walk the experts that received tokens, stage up to four of an
// expert's rows of x at a time and stream its weights through the warp-private rings, which keep running ahead
// across experts.  gather: x row = order[pos] / x_div, else pos; scatter: y row = order[pos], else pos.
// Weight families: symmetric int4 and fp8 e4m3; anything else returns cudaErrorInvalidValue (use the other kernel).
// norm_w != null: every staged row is RMS-normalised with that weight first (the layer's post-attention norm).
IPEX_API int ipex_moe_gemv_stream_norm(const void* w_list, int wf, const void* ranges, const void* order,
                                       int experts, int slots, int max_rows, const void* x, int x_div, int gather,
                                       int scatter, void* y, int N, int K, int ldx, int ldy, int act, int dtype,
                                       int* err, void* stream, const void* norm_w, float eps, float norm_offset) {
  if (experts < 1 || slots < 1 || max_rows < 1 || x_div < 1 || (K % 64) != 0 || err == nullptr ||
      w_list == nullptr || ranges == nullptr || order == nullptr)
    return (int)cudaErrorInvalidValue;
  if (wf != WF_SYM_INT4 && wf != WF_FP8_E4M3) return (int)cudaErrorInvalidValue;
  if (wf == WF_FP8_E4M3 && (K % 128) != 0) return (int)cudaErrorInvalidValue;
  if ((ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return (int)cudaErrorInvalidValue;
  if (act != 0 && (N % 32) != 0) return (int)cudaErrorInvalidValue;
  StreamArgs a;
  a.w = nullptr; a.x = x; a.y = y; a.norm_w = norm_w; a.bias = nullptr; a.residual = nullptr;
  a.err = err;
  a.M = max_rows < 4 ? max_rows : 4;      // rows of one pass (one MMA per 512 weights serves four tokens)
  a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = 0; a.eps = eps; a.norm_offset = norm_offset;
  a.act = act; a.stages = 0; a.cpw = 0; a.wpt = 1;
  a.tp_rank = 0; a.tp_world = 1; a.tp_npad = 0; a.tp_bufs = nullptr; a.tp_flags = nullptr;
  a.moe_w = reinterpret_cast<const uint8_t* const*>(w_list);
  a.moe_ranges = reinterpret_cast<const int*>(ranges);
  a.moe_order = reinterpret_cast<const int*>(order);
  a.moe_experts = experts; a.moe_slots = slots; a.moe_gather = gather; a.moe_scatter = scatter; a.moe_xdiv = x_div;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) {
    return wf == WF_SYM_INT4 ? (int)dispatch<__half, WFK_I8>(a, s, false) : (int)dispatch<__half, WFK_FP8>(a, s, false);
  }
  if (dtype == DT_BF16) {
    return wf == WF_SYM_INT4 ? (int)dispatch<__nv_bfloat16, WFK_I8>(a, s, false)
                             : (int)dispatch<__nv_bfloat16, WFK_FP8>(a, s, false);
  }
  return (int)cudaErrorInvalidValue;
}

// Without a fused norm (the rows of x are used as they are).
IPEX_API int ipex_moe_gemv_stream(const void* w_list, int wf, const void* ranges, const void* order, int experts,
                                  int slots, int max_rows, const void* x, int x_div, int gather, int scatter, void* y,
                                  int N, int K, int ldx, int ldy, int act, const float* lut, int dtype, int* err,
                                  void* stream) {
  (void)lut;
  return ipex_moe_gemv_stream_norm(w_list, wf, ranges, order, experts, slots, max_rows, x, x_div, gather, scatter, y, N,
                                   K, ldx, ldy, act, dtype, err, stream, nullptr, 0.f, 0.f);
}
