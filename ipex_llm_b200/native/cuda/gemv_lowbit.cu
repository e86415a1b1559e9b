// Low-bit GEMV / skinny GEMM for decode (M <= 8 activation rows), sm_100a.
//
//   y[M, N] = epilogue( prologue(x)[M, K] * dequant(W)[N, K]^T )
//
// Replaces the reference's closed `xe_linear.forward_new` (M = 1), `xe_batch.batch_forward` (small M) and
// `xe_linear.mlp_forward_xpu` (fused gate/up + SiLU*mul) kernels
// (python/llm/src/ipex_llm/transformers/low_bit_linear.py:506-538, 657-668; models/common.py:145-160).
//
// Design (bandwidth bound: every weight byte is read exactly once, at 16 bytes per lane):
//  * W is stored in the tile layout of native/host/quant_core.cpp: a warp-wide 16-byte load fetches a
//    [16 rows x 128 k] tile slice that is already in mma.m16n8k16 A-fragment order, so no shuffles and no
//    shared-memory staging of weights are needed.  4-bit codes become fp16 with the lop3 magic-number trick
//    (exact small integers), the per-group scale is applied to the fp32 accumulator of each 64-group.
//  * The M <= 8 activation rows are the 8 columns of the mma B operand: batch 1..8 costs the same.
//  * Each CTA owns RT row tiles and all of K; its 8 warps split K, then reduce through shared memory.
//  * Optional fused prologue: RMSNorm of x (each CTA re-derives the row statistics; x is tiny).
//    Optional fused epilogues: + bias, + residual, SiLU/GELU(gate) * up on interleaved gate/up row tiles.
//  * Programmatic dependent launch: the weight slice of the CTA is prefetched into L2 before
//    griddepcontrol.wait, so the DRAM stream of kernel i+1 overlaps the tail of kernel i.
#include "common/utils.cuh"
#include <cuda_fp8.h>
#include <type_traits>

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct GemvArgs {
  const uint8_t* w;
  const void* x;
  void* y;
  const void* norm_w;
  const void* bias;
  const void* residual;
  const float* lut;
  int M, N, K;
  int ldx, ldy, ldr;
  float eps, norm_offset;
  int act;  // 0 none, 1 silu(gate)*up, 2 gelu_tanh(gate)*up  (row tiles interleaved gate, up)
  // mixture-of-experts mode (w_list != null): blockIdx.y is a (token, choice) slot; the slot's expert id selects the
  // weight matrix on the device, x row = slot / x_div, y row = slot, one token per slot (M = 1)
  const uint8_t* const* w_list;
  const int64_t* expert_ids;
  int x_div;
  int x_div_slots;  // number of slots (grid.y)
  // expert-grouped mode (moe_ranges != null): blockIdx.y is an EXPERT, blockIdx.z a group of eight of its slots.
  // moe_ranges[e] = (first position, count) in the expert-sorted slot list moe_order; the expert's weights are read
  // once for up to eight tokens.  x row = moe_order[pos] / x_div (moe_gather) or pos; y row = moe_order[pos]
  // (moe_scatter) or pos.
  const int* moe_ranges = nullptr;
  const int* moe_order = nullptr;
  int moe_gather = 0, moe_scatter = 0, moe_experts = 0, moe_zchunks = 1, moe_rows = 8;
};

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

// word = 8 nibbles in magic order; pair index p (0..3) -> fp16x2 of weights (2p, 2p+1), zero point removed.
template <int ZP /* 8 for symmetric, 0 for asymmetric */>
struct Int4Pairs {
  uint32_t p[4];
  __device__ __forceinline__ explicit Int4Pairs(uint32_t u) {
    constexpr uint32_t kMagic = 0x64006400u;                       // 1024.0 | 1024.0
    constexpr uint32_t kSubLo = ZP == 8 ? 0x64086408u : 0x64006400u;  // 1032 or 1024
    constexpr uint32_t kSixteenth = 0x2C002C00u;                   // 1/16
    constexpr uint32_t kSubHi = ZP == 8 ? 0xD480D480u : 0xD400D400u;  // -72 or -64
    uint32_t lo = (u & 0x000F000Fu) | kMagic;
    uint32_t hi = (u & 0x00F000F0u) | kMagic;
    uint32_t u2 = u >> 8;
    uint32_t lo2 = (u2 & 0x000F000Fu) | kMagic;
    uint32_t hi2 = (u2 & 0x00F000F0u) | kMagic;
    p[0] = h2_sub(lo, kSubLo);
    p[1] = h2_fma(hi, kSixteenth, kSubHi);
    p[2] = h2_sub(lo2, kSubLo);
    p[3] = h2_fma(hi2, kSixteenth, kSubHi);
  }
};

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == 1) return g / (1.0f + __expf(-g));
  // tanh-approximated GELU
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * g * (1.0f + t);
}

template <typename T>
__device__ __forceinline__ float load_as_float(const void* p, size_t i) {
  return DT<T>::to_f(reinterpret_cast<const T*>(p)[i]);
}

// Stage x (optionally RMS-normalised) into shared memory as fp16 rows of stride xs_stride, zero padded to Kp.
template <typename T>
__device__ void stage_x(const GemvArgs& a, __half* xs, int xs_stride, int Kp, float* scratch,
                        const int* xrow = nullptr) {
  const int tid = threadIdx.x;
  const T* x0 = reinterpret_cast<const T*>(a.x);
  for (int m = 0; m < a.M; m++) {
    // rows of x are consecutive, or picked through xrow (expert-grouped mode); x[m * ldx + k] below is row m's k
    const T* x = xrow != nullptr ? x0 + ((ptrdiff_t)xrow[m] - (ptrdiff_t)m) * (ptrdiff_t)a.ldx : x0;
    float rstd = 1.0f;
    if (a.norm_w != nullptr) {
      float ss = 0.f;
      for (int k = tid; k < a.K; k += kThreads) {
        float v = DT<T>::to_f(x[(size_t)m * a.ldx + k]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      if ((tid & 31) == 0) scratch[tid >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; w++) tot += scratch[w];
      rstd = rsqrtf(tot / (float)a.K + a.eps);
      __syncthreads();
    }
    const T* nw = reinterpret_cast<const T*>(a.norm_w);
    for (int k = tid; k < Kp; k += kThreads) {
      float v = 0.f;
      if (k < a.K) {
        v = DT<T>::to_f(x[(size_t)m * a.ldx + k]);
        if (nw != nullptr) v = v * rstd * (DT<T>::to_f(nw[k]) + a.norm_offset);
        v = fminf(fmaxf(v, -65504.f), 65504.f);
      }
      xs[m * xs_stride + k] = __float2half_rn(v);
    }
  }
}

template <int WF, typename T, int RT>
__global__ void __launch_bounds__(kThreads) gemv_tiled_kernel(GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr bool k4bit = WF == WF_SYM_INT4 || WF == WF_ASYM_INT4 || WF == WF_LUT4;
  const int Kp = (int)ceil_to_i64(a.K, 128);
  const int Np = (int)ceil_to_i64(a.N, 16);
  const int chunks = Kp / 128;
  const int xs_stride = Kp + 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tile_row0 = blockIdx.x * RT;
  __shared__ int s_xrow[8], s_yrow[8];
  const bool grouped = a.moe_ranges != nullptr;
  if (grouped) {
    pdl_wait();                      // the ranges and the order come from the kernel before this one
    const int e = blockIdx.y, first = a.moe_ranges[2 * e], cnt = a.moe_ranges[2 * e + 1];
    const int base = blockIdx.z * a.moe_rows;
    if (base >= cnt) return;
    a.M = cnt - base < a.moe_rows ? cnt - base : a.moe_rows;
    a.w = a.w_list[e];
    if (tid < a.M) {
      const int pos = first + base + tid, slot = a.moe_order[pos];
      s_xrow[tid] = a.moe_gather ? slot / a.x_div : pos;
      s_yrow[tid] = a.moe_scatter ? slot : pos;
    }
    __syncthreads();
  } else if (a.w_list != nullptr) {
    const int slot = blockIdx.y;
    a.w = a.w_list[a.expert_ids[slot]];
    a.x = reinterpret_cast<const T*>(a.x) + (size_t)(slot / a.x_div) * a.ldx;
    a.y = reinterpret_cast<T*>(a.y) + (size_t)slot * a.ldy;
  }

  __half* xs = reinterpret_cast<__half*>(smem_raw);
  size_t off = ((size_t)a.M * xs_stride * sizeof(__half) + 15) & ~(size_t)15;
  float* red = reinterpret_cast<float*>(smem_raw + off);            // [kWarps][RT][16][8]
  off += (size_t)kWarps * RT * 128 * sizeof(float);
  float* scratch = reinterpret_cast<float*>(smem_raw + off);        // [kWarps]
  off += 64;
  float* xsum = reinterpret_cast<float*>(smem_raw + off);           // asym: [M][Kp/64]
  if (WF == WF_ASYM_INT4) off += (size_t)a.M * (Kp / 64) * sizeof(float);
  uint32_t* lut256 = reinterpret_cast<uint32_t*>(smem_raw + off);   // lut4: 256 x half2

  // plane addresses
  const uint8_t* codes = a.w;
  const size_t code_bytes = k4bit ? (size_t)Np * Kp / 2 : (size_t)Np * Kp;
  const uint8_t* scales = a.w + code_bytes;
  const size_t tile_bytes_per_row = k4bit ? (size_t)chunks * 1024 : (size_t)chunks * 2048;

  // ---- independent of the predecessor kernel: pull this CTA's weight slice towards L2 ----
  if (tid == 0) {
    const uint8_t* p = codes + (size_t)tile_row0 * tile_bytes_per_row;
    size_t total = (size_t)RT * tile_bytes_per_row;
    size_t avail = code_bytes - (size_t)tile_row0 * tile_bytes_per_row;
    if (total > avail) total = avail;
    for (size_t o = 0; o < total; o += 32768) {
      uint32_t n = (uint32_t)((total - o) < 32768 ? (total - o) : 32768);
      prefetch_l2_bulk(p + o, n);
    }
  }
  pdl_launch_dependents();
  pdl_wait();

  if (WF == WF_LUT4) {
    // byte -> (lut[lo nibble], lut[hi nibble]) as half2
    __half2 v = __floats2half2_rn(a.lut[tid & 15], a.lut[tid >> 4]);
    lut256[tid] = *reinterpret_cast<uint32_t*>(&v);
  }
  stage_x<T>(a, xs, xs_stride, Kp, scratch, grouped ? s_xrow : nullptr);
  __syncthreads();
  if (WF == WF_ASYM_INT4) {
    const int groups = Kp / 64;
    for (int i = tid; i < a.M * groups; i += kThreads) {
      int m = i / groups, gi = i % groups;
      float s = 0.f;
      for (int k = 0; k < 64; k++) s += __half2float(xs[m * xs_stride + gi * 64 + k]);
      xsum[i] = s;
    }
    __syncthreads();
  }

  float acc[RT][4];
#pragma unroll
  for (int r = 0; r < RT; r++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[r][i] = 0.f;

  const bool has_x = g < a.M;

  if constexpr (k4bit) {
    const uint8_t* mins = scales + (size_t)Np * (Kp / 64) * 2;
    for (int c = warp; c < chunks; c += kWarps) {
      uint4 xa0 = make_uint4(0, 0, 0, 0), xa1 = xa0, xb0 = xa0, xb1 = xa0;
      if (has_x) {
        const __half* xp = xs + g * xs_stride + c * 128 + 16 * t;
        xa0 = *reinterpret_cast<const uint4*>(xp);
        xa1 = *reinterpret_cast<const uint4*>(xp + 8);
        xb0 = *reinterpret_cast<const uint4*>(xp + 64);
        xb1 = *reinterpret_cast<const uint4*>(xp + 72);
      }
#pragma unroll
      for (int r = 0; r < RT; r++) {
        const size_t tile = (size_t)(tile_row0 + r) * chunks + c;
        if ((tile_row0 + r) * 16 >= Np) continue;
        const uint8_t* tp = codes + tile * 1024;
        const uint4 qa = ldg_nc_v4(tp + g * 64 + t * 16);
        const uint4 qb = ldg_nc_v4(tp + (g + 8) * 64 + t * 16);
        const uint32_t s0 = ldg_nc_u32(scales + ((tile * 2 + 0) * 16 + 2 * g) * 2);
        const uint32_t s1 = ldg_nc_u32(scales + ((tile * 2 + 1) * 16 + 2 * g) * 2);
        const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
        const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));

        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (WF == WF_LUT4) {
          auto lut_pair = [&](uint32_t word, int byte) { return lut256[(word >> (8 * byte)) & 0xFF]; };
          // natural order: byte b of a word = weights (2b, 2b+1)
          mma_f16(c0, lut_pair(qa.x, 0), lut_pair(qb.x, 0), lut_pair(qa.x, 1), lut_pair(qb.x, 1), xa0.x, xa0.y);
          mma_f16(c0, lut_pair(qa.x, 2), lut_pair(qb.x, 2), lut_pair(qa.x, 3), lut_pair(qb.x, 3), xa0.z, xa0.w);
          mma_f16(c0, lut_pair(qa.y, 0), lut_pair(qb.y, 0), lut_pair(qa.y, 1), lut_pair(qb.y, 1), xa1.x, xa1.y);
          mma_f16(c0, lut_pair(qa.y, 2), lut_pair(qb.y, 2), lut_pair(qa.y, 3), lut_pair(qb.y, 3), xa1.z, xa1.w);
          mma_f16(c1, lut_pair(qa.z, 0), lut_pair(qb.z, 0), lut_pair(qa.z, 1), lut_pair(qb.z, 1), xb0.x, xb0.y);
          mma_f16(c1, lut_pair(qa.z, 2), lut_pair(qb.z, 2), lut_pair(qa.z, 3), lut_pair(qb.z, 3), xb0.z, xb0.w);
          mma_f16(c1, lut_pair(qa.w, 0), lut_pair(qb.w, 0), lut_pair(qa.w, 1), lut_pair(qb.w, 1), xb1.x, xb1.y);
          mma_f16(c1, lut_pair(qa.w, 2), lut_pair(qb.w, 2), lut_pair(qa.w, 3), lut_pair(qb.w, 3), xb1.z, xb1.w);
        } else {
          constexpr int ZP = WF == WF_SYM_INT4 ? 8 : 0;
          {
            Int4Pairs<ZP> A(qa.x), B(qb.x);
            mma_f16(c0, A.p[0], B.p[0], A.p[1], B.p[1], xa0.x, xa0.y);
            mma_f16(c0, A.p[2], B.p[2], A.p[3], B.p[3], xa0.z, xa0.w);
          }
          {
            Int4Pairs<ZP> A(qa.y), B(qb.y);
            mma_f16(c0, A.p[0], B.p[0], A.p[1], B.p[1], xa1.x, xa1.y);
            mma_f16(c0, A.p[2], B.p[2], A.p[3], B.p[3], xa1.z, xa1.w);
          }
          {
            Int4Pairs<ZP> A(qa.z), B(qb.z);
            mma_f16(c1, A.p[0], B.p[0], A.p[1], B.p[1], xb0.x, xb0.y);
            mma_f16(c1, A.p[2], B.p[2], A.p[3], B.p[3], xb0.z, xb0.w);
          }
          {
            Int4Pairs<ZP> A(qa.w), B(qb.w);
            mma_f16(c1, A.p[0], B.p[0], A.p[1], B.p[1], xb1.x, xb1.y);
            mma_f16(c1, A.p[2], B.p[2], A.p[3], B.p[3], xb1.z, xb1.w);
          }
        }
        acc[r][0] += d0.x * c0[0] + d1.x * c1[0];
        acc[r][1] += d0.x * c0[1] + d1.x * c1[1];
        acc[r][2] += d0.y * c0[2] + d1.y * c1[2];
        acc[r][3] += d0.y * c0[3] + d1.y * c1[3];
        if constexpr (WF == WF_ASYM_INT4) {
          const uint32_t m0 = ldg_nc_u32(mins + ((tile * 2 + 0) * 16 + 2 * g) * 2);
          const uint32_t m1 = ldg_nc_u32(mins + ((tile * 2 + 1) * 16 + 2 * g) * 2);
          const float2 mn0 = __half22float2(*reinterpret_cast<const __half2*>(&m0));
          const float2 mn1 = __half22float2(*reinterpret_cast<const __half2*>(&m1));
          const int groups = Kp / 64;
          // the min term is added once per 64-group: only the lanes with t == 0..3 own distinct columns,
          // every lane adds it for its own two columns, and only from the k-quarter t == 0 of the group
          const int n0 = 2 * t, n1 = 2 * t + 1;
          const float xs00 = n0 < a.M ? xsum[n0 * groups + 2 * c] : 0.f;
          const float xs01 = n0 < a.M ? xsum[n0 * groups + 2 * c + 1] : 0.f;
          const float xs10 = n1 < a.M ? xsum[n1 * groups + 2 * c] : 0.f;
          const float xs11 = n1 < a.M ? xsum[n1 * groups + 2 * c + 1] : 0.f;
          acc[r][0] += mn0.x * xs00 + mn1.x * xs01;
          acc[r][1] += mn0.x * xs10 + mn1.x * xs11;
          acc[r][2] += mn0.y * xs00 + mn1.y * xs01;
          acc[r][3] += mn0.y * xs10 + mn1.y * xs11;
        }
      }
    }
  } else {
    // 8-bit families: tiles of [16 rows][64 k]; one loop step = 128 k = two tiles
    const int tiles_per_row = Kp / 64;
    for (int c = warp; c < chunks; c += kWarps) {
      uint4 xv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) xv[i] = make_uint4(0, 0, 0, 0);
      if (has_x) {
        const __half* xp = xs + g * xs_stride + c * 128 + 16 * t;
        xv[0] = *reinterpret_cast<const uint4*>(xp);
        xv[1] = *reinterpret_cast<const uint4*>(xp + 8);
        xv[2] = *reinterpret_cast<const uint4*>(xp + 64);
        xv[3] = *reinterpret_cast<const uint4*>(xp + 72);
      }
#pragma unroll
      for (int r = 0; r < RT; r++) {
        if ((tile_row0 + r) * 16 >= Np) continue;
        float cc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const size_t tile = (size_t)(tile_row0 + r) * tiles_per_row + 2 * c + h;
          const uint8_t* tp = codes + tile * 1024;
          const uint4 qa = ldg_nc_v4(tp + g * 64 + t * 16);
          const uint4 qb = ldg_nc_v4(tp + (g + 8) * 64 + t * 16);
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
          const uint8_t* sp = scales;
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const size_t tile = (size_t)(tile_row0 + r) * tiles_per_row + 2 * c + h;
            const uint32_t s = ldg_nc_u32(sp + (tile * 16 + 2 * g) * 2);
            const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&s));
            acc[r][0] += d.x * cc[h][0];
            acc[r][1] += d.x * cc[h][1];
            acc[r][2] += d.y * cc[h][2];
            acc[r][3] += d.y * cc[h][3];
          }
        } else {
          const float* sp = reinterpret_cast<const float*>(scales);
          const size_t blk = (size_t)(tile_row0 + r) * chunks + c;
          const float2 d = *reinterpret_cast<const float2*>(sp + blk * 16 + 2 * g);
          acc[r][0] += d.x * (cc[0][0] + cc[1][0]);
          acc[r][1] += d.x * (cc[0][1] + cc[1][1]);
          acc[r][2] += d.y * (cc[0][2] + cc[1][2]);
          acc[r][3] += d.y * (cc[0][3] + cc[1][3]);
        }
      }
    }
  }

  // ---- cross-warp reduction and epilogue ----
#pragma unroll
  for (int r = 0; r < RT; r++) {
    float* rp = red + ((size_t)(warp * RT + r) * 16) * 8;
    rp[g * 8 + 2 * t] = acc[r][0];
    rp[g * 8 + 2 * t + 1] = acc[r][1];
    rp[(g + 8) * 8 + 2 * t] = acc[r][2];
    rp[(g + 8) * 8 + 2 * t + 1] = acc[r][3];
  }
  __syncthreads();
  T* y = reinterpret_cast<T*>(a.y);
  if (a.act == 0) {
    for (int i = tid; i < RT * 128; i += kThreads) {
      const int r = i / 128, col = (i % 128) / 16, row = i % 16;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; w++) s += red[((size_t)(w * RT + r) * 16 + row) * 8 + col];
      const int n = (tile_row0 + r) * 16 + row;
      if (n < a.N && col < a.M) {
        if (a.bias != nullptr) s += load_as_float<T>(a.bias, n);
        if (a.residual != nullptr) s += load_as_float<T>(a.residual, (size_t)col * a.ldr + n);
        y[(size_t)(grouped ? s_yrow[col] : col) * a.ldy + n] = DT<T>::from_f(s);
      }
    }
  } else if (RT == 2) {
    // row tile 0 = gate rows, row tile 1 = up rows of the same 16 output features
    if (tid < 128) {
      const int col = tid / 16, row = tid % 16;
      float gsum = 0.f, usum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; w++) {
        gsum += red[((size_t)(w * RT + 0) * 16 + row) * 8 + col];
        usum += red[((size_t)(w * RT + 1) * 16 + row) * 8 + col];
      }
      const int n = blockIdx.x * 16 + row;
      if (n < a.N / 2 && col < a.M) {
        if (a.bias != nullptr) {
          gsum += load_as_float<T>(a.bias, (size_t)blockIdx.x * 32 + row);
          usum += load_as_float<T>(a.bias, (size_t)blockIdx.x * 32 + 16 + row);
        }
        y[(size_t)(grouped ? s_yrow[col] : col) * a.ldy + n] = DT<T>::from_f(act_apply(gsum, a.act) * usum);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// dense half-precision weights, row-major [N, K]  (fp16 / bf16 "low_bit" modes, unquantized lm_head,
// the fp16 target model of self-speculative decoding)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T, int RT>
__global__ void __launch_bounds__(kThreads) gemv_dense_kernel(GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int Kp = (int)ceil_to_i64(a.K, 64);
  const int xs_stride = Kp + 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * RT * 16;
  T* xs = reinterpret_cast<T*>(smem_raw);
  size_t off = ((size_t)a.M * xs_stride * sizeof(T) + 15) & ~(size_t)15;
  float* red = reinterpret_cast<float*>(smem_raw + off);
  off += (size_t)kWarps * RT * 128 * sizeof(float);
  float* scratch = reinterpret_cast<float*>(smem_raw + off);
  const T* W = reinterpret_cast<const T*>(a.w);

  pdl_launch_dependents();
  pdl_wait();

  // stage x (optionally normalised) in its own dtype
  {
    const T* x = reinterpret_cast<const T*>(a.x);
    const T* nw = reinterpret_cast<const T*>(a.norm_w);
    // K is a multiple of 16, so 8-element vectors never straddle the end of a row
    const bool vec = (a.ldx & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                     (nw == nullptr || (reinterpret_cast<uintptr_t>(nw) & 15) == 0);
    if (vec) {
      // all rows at once: one pass for the sums of squares with ONE block reduction (through `red`, free until
      // the epilogue), one pass that normalises and stores 16 bytes per row and thread
      float rstd[8];
#pragma unroll
      for (int m = 0; m < 8; m++) rstd[m] = 1.f;
      if (nw != nullptr) {
        float ss[8];
#pragma unroll
        for (int m = 0; m < 8; m++) ss[m] = 0.f;
        for (int k = tid * 8; k < a.K; k += kThreads * 8) {
#pragma unroll
          for (int m = 0; m < 8; m++) {
            if (m < a.M) {
              const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + k);
              const T* pv = reinterpret_cast<const T*>(&v);
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float f = DT<T>::to_f(pv[j]);
                ss[m] += f * f;
              }
            }
          }
        }
#pragma unroll
        for (int m = 0; m < 8; m++) {
          ss[m] = warp_sum(ss[m]);
          if (lane == 0) red[warp * 8 + m] = ss[m];
        }
        __syncthreads();
#pragma unroll
        for (int m = 0; m < 8; m++) {
          float tot = 0.f;
          for (int w = 0; w < kWarps; w++) tot += red[w * 8 + m];
          rstd[m] = rsqrtf(tot / (float)a.K + a.eps);
        }
      }
      for (int k = tid * 8; k < Kp; k += kThreads * 8) {
        uint4 nv = make_uint4(0, 0, 0, 0);
        if (nw != nullptr && k < a.K) nv = *reinterpret_cast<const uint4*>(nw + k);
        const T* pn = reinterpret_cast<const T*>(&nv);
#pragma unroll
        for (int m = 0; m < 8; m++) {
          if (m < a.M) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (k < a.K) {
              v = *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + k);
              if (nw != nullptr) {
                T* pv = reinterpret_cast<T*>(&v);
#pragma unroll
                for (int j = 0; j < 8; j++)
                  pv[j] = DT<T>::from_f(DT<T>::to_f(pv[j]) * rstd[m] * (DT<T>::to_f(pn[j]) + a.norm_offset));
              }
            }
            *reinterpret_cast<uint4*>(xs + m * xs_stride + k) = v;
          }
        }
      }
    } else {
      for (int m = 0; m < a.M; m++) {
        float rstd = 1.f;
        if (nw != nullptr) {
          float ss = 0.f;
          for (int k = tid; k < a.K; k += kThreads) {
            float v = DT<T>::to_f(x[(size_t)m * a.ldx + k]);
            ss += v * v;
          }
          ss = warp_sum(ss);
          if (lane == 0) scratch[warp] = ss;
          __syncthreads();
          float tot = 0.f;
          for (int w = 0; w < kWarps; w++) tot += scratch[w];
          rstd = rsqrtf(tot / (float)a.K + a.eps);
          __syncthreads();
        }
        for (int k = tid; k < Kp; k += kThreads) {
          float v = 0.f;
          if (k < a.K) {
            v = DT<T>::to_f(x[(size_t)m * a.ldx + k]);
            if (nw != nullptr) v = v * rstd * (DT<T>::to_f(nw[k]) + a.norm_offset);
          }
          xs[m * xs_stride + k] = DT<T>::from_f(v);
        }
      }
    }
  }
  __syncthreads();

  float acc[RT][4];
#pragma unroll
  for (int r = 0; r < RT; r++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[r][i] = 0.f;
  const bool has_x = g < a.M;
  const int chunks = Kp / 64;
  for (int c = warp; c < chunks; c += kWarps) {
    const int k0 = c * 64 + 16 * t;
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
    if (has_x) {
      x0 = *reinterpret_cast<const uint4*>(xs + g * xs_stride + k0);
      x1 = *reinterpret_cast<const uint4*>(xs + g * xs_stride + k0 + 8);
    }
#pragma unroll
    for (int r = 0; r < RT; r++) {
      const int ra = row0 + r * 16 + g, rb = ra + 8;
      uint4 wa0 = make_uint4(0, 0, 0, 0), wa1 = wa0, wb0 = wa0, wb1 = wa0;
      if (k0 < a.K) {
        if (ra < a.N) {
          wa0 = ldg_nc_v4(W + (size_t)ra * a.K + k0);
          wa1 = ldg_nc_v4(W + (size_t)ra * a.K + k0 + 8);
        }
        if (rb < a.N) {
          wb0 = ldg_nc_v4(W + (size_t)rb * a.K + k0);
          wb1 = ldg_nc_v4(W + (size_t)rb * a.K + k0 + 8);
        }
      }
      if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) {
        mma_f16(acc[r], wa0.x, wb0.x, wa0.y, wb0.y, x0.x, x0.y);
        mma_f16(acc[r], wa0.z, wb0.z, wa0.w, wb0.w, x0.z, x0.w);
        mma_f16(acc[r], wa1.x, wb1.x, wa1.y, wb1.y, x1.x, x1.y);
        mma_f16(acc[r], wa1.z, wb1.z, wa1.w, wb1.w, x1.z, x1.w);
      } else {
        mma_bf16(acc[r], wa0.x, wb0.x, wa0.y, wb0.y, x0.x, x0.y);
        mma_bf16(acc[r], wa0.z, wb0.z, wa0.w, wb0.w, x0.z, x0.w);
        mma_bf16(acc[r], wa1.x, wb1.x, wa1.y, wb1.y, x1.x, x1.y);
        mma_bf16(acc[r], wa1.z, wb1.z, wa1.w, wb1.w, x1.z, x1.w);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RT; r++) {
    float* rp = red + ((size_t)(warp * RT + r) * 16) * 8;
    rp[g * 8 + 2 * t] = acc[r][0];
    rp[g * 8 + 2 * t + 1] = acc[r][1];
    rp[(g + 8) * 8 + 2 * t] = acc[r][2];
    rp[(g + 8) * 8 + 2 * t + 1] = acc[r][3];
  }
  __syncthreads();
  T* y = reinterpret_cast<T*>(a.y);
  if (RT == 2 && a.act != 0) {
    // rows [row0, row0+16) hold a gate tile, the next 16 its up tile (16-row interleaved weight)
    for (int i = tid; i < 128; i += kThreads) {
      const int col = i / 16, row = i % 16;
      float gsum = 0.f, usum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; w++) {
        gsum += red[((size_t)(w * RT) * 16 + row) * 8 + col];
        usum += red[((size_t)(w * RT + 1) * 16 + row) * 8 + col];
      }
      const int n = blockIdx.x * 16 + row;
      if (n < a.N / 2 && col < a.M) {
        if (a.bias != nullptr) {
          gsum += load_as_float<T>(a.bias, (size_t)row0 + row);
          usum += load_as_float<T>(a.bias, (size_t)row0 + 16 + row);
        }
        y[(size_t)col * a.ldy + n] = DT<T>::from_f(act_apply(gsum, a.act) * usum);
      }
    }
    return;
  }
  for (int i = tid; i < RT * 128; i += kThreads) {
    const int r = i / 128, col = (i % 128) / 16, row = i % 16;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; w++) s += red[((size_t)(w * RT + r) * 16 + row) * 8 + col];
    const int n = row0 + r * 16 + row;
    if (n < a.N && col < a.M) {
      if (a.bias != nullptr) s += load_as_float<T>(a.bias, n);
      if (a.residual != nullptr) s += load_as_float<T>(a.residual, (size_t)col * a.ldr + n);
      y[(size_t)col * a.ldy + n] = DT<T>::from_f(s);
    }
  }
}

template <int WF, typename T, int RT>
cudaError_t launch_tiled(const GemvArgs& a, cudaStream_t stream, bool pdl) {
  const int Kp = (int)ceil_to_i64(a.K, 128);
  const int Np = (int)ceil_to_i64(a.N, 16);
  size_t smem = (((size_t)a.M * (Kp + 8) * 2 + 15) & ~(size_t)15) + (size_t)kWarps * RT * 128 * 4 + 64;
  if (WF == WF_ASYM_INT4) smem += (size_t)a.M * (Kp / 64) * 4;
  if (WF == WF_LUT4) smem += 1024;
  auto kern = gemv_tiled_kernel<WF, T, RT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  dim3 grid((Np / 16 + RT - 1) / RT, a.w_list != nullptr ? a.x_div_slots : 1);
  if (a.moe_ranges != nullptr) grid = dim3(grid.x, a.moe_experts, a.moe_zchunks);
  return launch_kernel(kern, grid, dim3(kThreads), smem, stream, pdl, a);
}

template <int WF, typename T>
cudaError_t dispatch_rt(const GemvArgs& a, cudaStream_t s, bool pdl) {
  if (a.act != 0) return launch_tiled<WF, T, 2>(a, s, pdl);
  return launch_tiled<WF, T, 1>(a, s, pdl);
}

template <typename T>
cudaError_t dispatch_wf(int wf, const GemvArgs& a, cudaStream_t s, bool pdl) {
  switch (wf) {
    case WF_SYM_INT4: return dispatch_rt<WF_SYM_INT4, T>(a, s, pdl);
    case WF_ASYM_INT4: return dispatch_rt<WF_ASYM_INT4, T>(a, s, pdl);
    case WF_LUT4: return dispatch_rt<WF_LUT4, T>(a, s, pdl);
    case WF_FP8_E4M3: return dispatch_rt<WF_FP8_E4M3, T>(a, s, pdl);
    case WF_FP8_E5M2: return dispatch_rt<WF_FP8_E5M2, T>(a, s, pdl);
    case WF_INT8: return dispatch_rt<WF_INT8, T>(a, s, pdl);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// y[M,N] = epi(pro(x) W^T).  wf: weight family (WF_*), dtype: activation dtype (DT_F16 / DT_BF16).
// norm_w != NULL fuses RMSNorm(x) * (norm_w + norm_offset); act != 0 expects gate/up interleaved row tiles and
// writes N/2 columns.  Returns a cudaError_t.
IPEX_API int ipex_gemv_lowbit(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx, int ldy,
                              const void* norm_w, float eps, float norm_offset, const void* bias, const void* residual,
                              int ldr, int act, const float* lut, int dtype, int pdl, void* stream) {
  const bool dense = wf == WF_F16 || wf == WF_BF16;
  if (M < 1 || M > 8 || (K % (dense ? 16 : 64)) != 0) return (int)cudaErrorInvalidValue;
  GemvArgs a;
  a.w = (const uint8_t*)w; a.x = x; a.y = y; a.norm_w = norm_w; a.bias = bias; a.residual = residual; a.lut = lut;
  a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = ldr; a.eps = eps; a.norm_offset = norm_offset;
  a.act = act;
  a.w_list = nullptr; a.expert_ids = nullptr; a.x_div = 1; a.x_div_slots = 1;
  cudaStream_t s = (cudaStream_t)stream;
  if (wf == WF_F16 || wf == WF_BF16) {
    const int Kp = (int)ceil_to_i64(K, 64);
    if (act != 0) {
      // gate/up interleaved in 16-row tiles: one CTA per (gate tile, up tile) pair, N/2 output columns
      if ((N % 32) != 0) return (int)cudaErrorInvalidValue;
      size_t smem2 = (((size_t)M * (Kp + 8) * 2 + 15) & ~(size_t)15) + (size_t)kWarps * 2 * 128 * 4 + 64;
      dim3 grid2(N / 32);
      if (wf == WF_F16 && dtype == DT_F16) {
        auto kern = gemv_dense_kernel<__half, 2>;
        if (smem2 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        return (int)launch_kernel(kern, grid2, dim3(kThreads), smem2, s, pdl != 0, a);
      }
      if (wf == WF_BF16 && dtype == DT_BF16) {
        auto kern = gemv_dense_kernel<__nv_bfloat16, 2>;
        if (smem2 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        return (int)launch_kernel(kern, grid2, dim3(kThreads), smem2, s, pdl != 0, a);
      }
      return (int)cudaErrorInvalidValue;
    }
    size_t smem = (((size_t)M * (Kp + 8) * 2 + 15) & ~(size_t)15) + (size_t)kWarps * 128 * 4 + 64;
    dim3 grid((N + 15) / 16);
    if (wf == WF_F16) {
      if (dtype != DT_F16) return (int)cudaErrorInvalidValue;
      auto kern = gemv_dense_kernel<__half, 1>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      return (int)launch_kernel(kern, grid, dim3(kThreads), smem, s, pdl != 0, a);
    } else {
      if (dtype != DT_BF16) return (int)cudaErrorInvalidValue;
      auto kern = gemv_dense_kernel<__nv_bfloat16, 1>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      return (int)launch_kernel(kern, grid, dim3(kThreads), smem, s, pdl != 0, a);
    }
  }
  if (dtype == DT_F16) return (int)dispatch_wf<__half>(wf, a, s, pdl != 0);
  if (dtype == DT_BF16) return (int)dispatch_wf<__nv_bfloat16>(wf, a, s, pdl != 0);
  return (int)cudaErrorInvalidValue;
}

// Mixture-of-experts GEMV for decode: `nslots` = tokens x experts-per-token independent GEMVs in one launch.
// Slot s uses the weight matrix w_list[expert_ids[s]] (all of family `wf`, shape [N, K], device tile layout), reads
// x row s / x_div and writes y row s.  The expert choice never leaves the device.  act != 0: gate/up interleaved
// row tiles, N/2 output columns.
IPEX_API int ipex_moe_gemv(const void* w_list, int wf, const void* expert_ids, int nslots, const void* x, int x_div,
                           void* y, int N, int K, int ldx, int ldy, int act, const float* lut, int dtype, int pdl,
                           void* stream) {
  if (nslots < 1 || nslots > 65535 || x_div < 1 || (K % 64) != 0 || wf == WF_F16 || wf == WF_BF16)
    return (int)cudaErrorInvalidValue;
  GemvArgs a;
  a.w = nullptr; a.x = x; a.y = y; a.norm_w = nullptr; a.bias = nullptr; a.residual = nullptr; a.lut = lut;
  a.M = 1; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = 0; a.eps = 0.f; a.norm_offset = 0.f;
  a.act = act;
  a.w_list = reinterpret_cast<const uint8_t* const*>(w_list);
  a.expert_ids = reinterpret_cast<const int64_t*>(expert_ids);
  a.x_div = x_div; a.x_div_slots = nslots;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) return (int)dispatch_wf<__half>(wf, a, s, pdl != 0);
  if (dtype == DT_BF16) return (int)dispatch_wf<__nv_bfloat16>(wf, a, s, pdl != 0);
  return (int)cudaErrorInvalidValue;
}

// Tokens of one expert that one CTA of ipex_moe_gemv_grouped multiplies at a time: eight when their staged rows
// leave room for three CTAs per SM, else as many as keep two CTAs per SM (long contractions).
IPEX_API int ipex_moe_gemv_group_rows(int K) {
  const size_t row = ((size_t)ceil_to_i64(K, 128) + 8) * 2;
  if (8 * row <= 68 * 1024) return 8;
  int r = (int)((104 * 1024) / row);
  return r < 1 ? 1 : (r > 8 ? 8 : r);
}

// Expert-grouped form for small batches: the slots are sorted by expert (ipex_moe_sort_slots) and CTA (tile, e, z)
// multiplies up to R = ipex_moe_gemv_group_rows(K) of expert e's tokens with one read of its weights.  gather: x row =
// order[pos] / x_div, else pos; scatter: y row = order[pos], else pos.  zchunks >= ceil(max tokens of one expert / R).
IPEX_API int ipex_moe_gemv_grouped(const void* w_list, int wf, const void* ranges, const void* order, int experts,
                                   int zchunks, const void* x, int x_div, int gather, int scatter, void* y, int N,
                                   int K, int ldx, int ldy, int act, const float* lut, int dtype, void* stream) {
  if (experts < 1 || experts > 65535 || zchunks < 1 || zchunks > 65535 || x_div < 1 || (K % 64) != 0 ||
      wf == WF_F16 || wf == WF_BF16 || ranges == nullptr || order == nullptr)
    return (int)cudaErrorInvalidValue;
  GemvArgs a;
  a.w = nullptr; a.x = x; a.y = y; a.norm_w = nullptr; a.bias = nullptr; a.residual = nullptr; a.lut = lut;
  a.moe_rows = ipex_moe_gemv_group_rows(K);
  a.M = a.moe_rows; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = 0; a.eps = 0.f; a.norm_offset = 0.f;
  a.act = act;
  a.w_list = reinterpret_cast<const uint8_t* const*>(w_list);
  a.expert_ids = nullptr;
  a.x_div = x_div; a.x_div_slots = 1;
  a.moe_ranges = reinterpret_cast<const int*>(ranges);
  a.moe_order = reinterpret_cast<const int*>(order);
  a.moe_gather = gather; a.moe_scatter = scatter; a.moe_experts = experts; a.moe_zchunks = zchunks;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) return (int)dispatch_wf<__half>(wf, a, s, false);
  if (dtype == DT_BF16) return (int)dispatch_wf<__nv_bfloat16>(wf, a, s, false);
  return (int)cudaErrorInvalidValue;
}
