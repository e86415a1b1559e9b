// Prefill / batch GEMM on the 5th-generation tensor cores:
//     out[M, N] = x[M, K] . W[N, K]^T  (+ bias) (+ residual)   or   act(gate) * up  for interleaved gate/up rows
// with W either dense fp16/bf16 or packed low-bit tiles that are dequantized inside the kernel.
//
// The weight rows sit on the MMA's M side (128 rows per tile) and the tokens on its N side (32..256 per tile), so a
// short prompt still fills the instruction: D[TMEM lane = weight row][TMEM column = token].  Both operands are
// K-major in shared memory in the 128-byte swizzle that TMA writes and tcgen05.mma reads directly.
//
// One persistent CTA per SM; roles by warp:
//   warp 0       one lane issues the TMA loads into a ring of stages (tokens always; weights when they are dense);
//   warp 1       allocates TMEM; one lane issues tcgen05.mma (4 per 64-wide k block) and commits: a commit releases
//                the stage, the last commit of a tile hands the accumulator to the epilogue;
//   warps 2..5   epilogue: tcgen05.ld the accumulator (each warp owns one 32-lane quarter), bias / residual /
//                activation, convert, store.  Two accumulators alternate in TMEM, so the epilogue of tile i
//                overlaps the main loop of tile i+1;
//   warps 6..13  (packed weights only) dequantizers: each thread owns half a weight row of the tile, reads the packed
//                bytes straight from global memory (next unit prefetched into registers, later units into L2),
//                expands them to the activation dtype and writes the swizzled operand tile the MMA expects.
// Every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, records a code in the global
// error flag (8 loader, 9 MMA issuer, 10 epilogue, 11 dequantizer) and every role leaves its loop; TMEM is
// released on all paths.
//
// Reference counterpart: the XMX GEMM branch of xe_linear.forward_new (python/llm/src/ipex_llm/transformers/
// low_bit_linear.py:640-668 picks it for prompts) and xe_batch.batch_forward for batches.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/utils.cuh"
#include "tcgen05_common.cuh"

namespace {

using namespace tc5;

constexpr int kBM = 128;  // weight rows per tile (MMA M)
constexpr int kBK = 64;   // k per stage: 64 x 2 B = one 128-byte swizzle row
constexpr int kBaseThreads = 192;
constexpr int kDequantThreads = 256;
constexpr int kPrefetchUnits = 6;  // how far ahead (in 32-byte units per thread) packed weights are pulled into L2

struct GemmArgs {
  const uint8_t* w;  // packed weights (unused for dense)
  const float* lut;  // 16 code values for the table families
  void* out;
  const void* bias;      // [N] or null
  const void* residual;  // [M, ldr] or null
  int64_t ldo, ldr;
  int64_t Np, Kp;  // padded extents of the packed layout
  int M, N, K;
  int m_tiles, n_tiles;
  int act;  // 0: none; 1 silu, 2 gelu(tanh): rows come as 16-row tiles gate, up, gate, up ... and out has N/2 columns
  int* err;
  // tensor parallel (tp_world > 1): the output is the sum of every rank's product.  tp_stage[r] / tp_flags[r] point
  // at rank r's staging buffer [tp_world][tiles][128][BT] of T and its per-(tile, lane quarter) arrival counters.
  int tp_rank, tp_world;
  void* const* tp_stage;
  int* const* tp_flags;
  // all-gather in front of the GEMM (ag_flags != null): x is this rank's copy of the gathered activation, rows
  // [r * ag_rows, (r + 1) * ag_rows) are pushed into it by rank r, which then sets ag_flags[r] to ag_epoch.  The
  // loader waits for the ranks a token tile covers before it issues the tile's first load.
  const int* ag_flags;
  int ag_rows, ag_epoch;
  // ... and the push of this rank's own rows, done by the epilogue warps of every CTA before their first tile:
  // ag_src [rows of this rank, K] (row stride ag_ld_src) goes to rows tp_rank * ag_rows .. of ag_dst[p] for every
  // rank p (ag_dst[p] = rank p's gathered buffer, row stride K); the CTA that draws the last ticket of ag_ticket
  // publishes ag_epoch in slot tp_rank of every rank's flag array ag_peer_flags[p].
  const void* ag_src;
  int64_t ag_ld_src;
  void* const* ag_dst;
  int* const* ag_peer_flags;
  int* ag_ticket;
  int ag_world;
  // grouped use (mixture-of-experts prompts): the launch covers rows [m_range[0], m_range[0] + m_range[1]) of x and
  // out, read from DEVICE memory when the kernel starts, so the host never learns how many tokens an expert got.
  // M / m_tiles given at launch are the upper bound that sized the grid.
  const int* m_range;
};

__device__ __forceinline__ int pair_row(int r) { return (r & 7) * 2 + (r >> 3); }

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == 1) return g / (1.0f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.0f + tanhf(k0 * (g + k1 * g * g * g)));
}

// ------------------------------------------------------------------------------------------------------------------
// two-lane arithmetic in the activation dtype
// ------------------------------------------------------------------------------------------------------------------
template <typename T> struct V2;
template <> struct V2<__half> {
  using type = __half2;
  static __device__ __forceinline__ type bits(uint32_t u) { return *reinterpret_cast<type*>(&u); }
  static __device__ __forceinline__ uint32_t raw(type v) { return *reinterpret_cast<uint32_t*>(&v); }
  static __device__ __forceinline__ type splat(float f) { return __float2half2_rn(f); }
  static constexpr uint32_t kMagic = 0x64006400u;  // 1024 + q
  static constexpr float kMagicBase = 1024.f;
};
template <> struct V2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ type bits(uint32_t u) { return *reinterpret_cast<type*>(&u); }
  static __device__ __forceinline__ uint32_t raw(type v) { return *reinterpret_cast<uint32_t*>(&v); }
  static __device__ __forceinline__ type splat(float f) { return __float2bfloat162_rn(f); }
  static constexpr uint32_t kMagic = 0x43004300u;  // 128 + q
  static constexpr float kMagicBase = 128.f;
};

// Per-(row, scale group) constants of the dequantizer, already in the two-lane type.
template <typename T>
struct Scale {
  typename V2<T>::type d, m;
};

// 8 codes of one 32-bit word (4-bit families) -> 8 values in k order, packed as 4 x two-lane.
// int4 words hold element k in nibble {0,4,1,5,2,6,3,7}[k]: (w >> 4i) & 0x000F000F is the pair (2i, 2i+1).
template <typename T, int WF>
__device__ __forceinline__ uint4 expand4(uint32_t w, const Scale<T>& sc, const uint32_t* lut2) {
  using V = V2<T>;
  uint32_t r[4];
  if constexpr (WF == WF_LUT4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t pair = lut2[(w >> (8 * i)) & 0xFFu];  // (lut[lo nibble], lut[hi nibble]) in T
      r[i] = V::raw(__hmul2(V::bits(pair), sc.d));
    }
  } else {
    const typename V::type off = V::splat(V::kMagicBase + (WF == WF_SYM_INT4 ? 8.f : 0.f));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t t = ((w >> (4 * i)) & 0x000F000Fu) | V::kMagic;
      const typename V::type q = __hsub2(V::bits(t), off);  // exact: small integers
      r[i] = V::raw(WF == WF_SYM_INT4 ? __hmul2(q, sc.d) : __hfma2(q, sc.d, sc.m));
    }
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}

// Exponent re-bias for fp8 -> 16-bit float by bit placement: the fp8 byte goes to the top of the 16-bit lane, the
// 7 magnitude bits are shifted down into the wider exponent field, and the missing 2^delta is folded into the
// scale.  Works for denormals too (both formats are linear there).
template <typename T, int WF> struct Fp8Place;
// `pre` (a power of two, applied to the placed value first) keeps the scale out of fp16's denormal range: e5m2
// codes reach 57344, so their scales are ~1e-6; codes below 2^-12 of full range may flush, which is far under
// the format's own resolution.
template <> struct Fp8Place<__half, WF_FP8_E4M3> {
  static constexpr int sh = 1; static constexpr float mul = 256.f; static constexpr float pre = 1.f;
};
template <> struct Fp8Place<__half, WF_FP8_E5M2> {
  static constexpr int sh = 0; static constexpr float mul = 4096.f; static constexpr float pre = 1.f / 4096.f;
};
template <> struct Fp8Place<__nv_bfloat16, WF_FP8_E4M3> {
  static constexpr int sh = 4; static constexpr float mul = 1.329227995784916e36f /* 2^120 */;
  static constexpr float pre = 1.f;
};
template <> struct Fp8Place<__nv_bfloat16, WF_FP8_E5M2> {
  static constexpr int sh = 3; static constexpr float mul = 5.192296858534828e33f /* 2^112 */;
  static constexpr float pre = 1.f;
};

// 8 bytes (two words) of an 8-bit family -> 8 values.
template <typename T, int WF>
__device__ __forceinline__ uint4 expand8(uint32_t w0, uint32_t w1, const Scale<T>& sc) {
  using V = V2<T>;
  uint32_t r[4];
  const uint32_t ws[2] = {w0, w1};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w = ws[i >> 1];
    if constexpr (WF == WF_INT8) {
      // (1024 + (b ^ 0x80)) - 1152 = signed value, exact in fp16
      const uint32_t t = __byte_perm(w, 0x64646464u, (i & 1) ? 0x4342 : 0x4140) ^ 0x00800080u;
      const __half2 q = __hsub2(V2<__half>::bits(t), __float2half2_rn(1152.f));
      if constexpr (std::is_same<T, __half>::value) {
        r[i] = V::raw(__hmul2(q, sc.d));
      } else {
        const float2 f = __half22float2(q);
        r[i] = V::raw(__hmul2(__floats2bfloat162_rn(f.x, f.y), sc.d));
      }
    } else {
      using P = Fp8Place<T, WF>;
      const uint32_t t = __byte_perm(w, 0u, (i & 1) ? 0x3424 : 0x1404);  // bytes to the top of each 16-bit lane
      uint32_t b = t;
      if constexpr (P::sh != 0) b = (t & 0x80008000u) | ((t >> P::sh) & (0x7F007F00u >> P::sh));
      typename V::type val = V::bits(b);
      if constexpr (P::pre != 1.f) val = __hmul2(val, V::splat(P::pre));
      r[i] = V::raw(__hmul2(val, sc.d));
    }
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}

template <int WF> struct Fam {
  static constexpr bool dense = WF == WF_F16 || WF == WF_BF16;
  static constexpr bool four_bit = WF == WF_SYM_INT4 || WF == WF_ASYM_INT4 || WF == WF_LUT4;
  static constexpr int threads = dense ? kBaseThreads : kBaseThreads + kDequantThreads;
};

template <int BT>
struct Cfg {
  static constexpr int kStages = BT >= 256 ? 4 : (BT >= 128 ? 6 : 8);
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BT * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BT < 32 ? 32 : 2 * BT;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ +
                                    1024 /*pair table of the LUT families*/;
};

// ------------------------------------------------------------------------------------------------------------------
// dequantizer role: fills the weight operand of every stage for this CTA's tiles
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int BT, int WF>
__device__ __forceinline__ void dequant_role(const GemmArgs& a, uint8_t* sA, uint64_t* full, uint64_t* empty,
                                             volatile int* abort_flag, const uint32_t* lut2) {
  using C = Cfg<BT>;
  using V = V2<T>;
  constexpr bool k4 = Fam<WF>::four_bit;
  const int dt = threadIdx.x - kBaseThreads;
  const int r = dt & 127, h = dt >> 7;  // weight row of the tile, which half of its bytes
  const int lane = threadIdx.x & 31;
  const int ntiles = a.m_tiles * a.n_tiles;
  // one "unit" = 32 bytes of this thread's row: a whole 128-wide k tile for 4-bit codes (feeds two stages),
  // one 64-wide k block for bytes (feeds one stage)
  const int units = k4 ? (int)(a.Kp / 128) : (int)(a.Kp / 64);
  const int64_t tile_stride = 1024;
  int s = 0;
  uint32_t ph = 0;
  bool ok = true;

  for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
    const int nb = t / a.m_tiles;
    const int64_t rg = (int64_t)nb * kBM + r;
    const bool valid = rg < a.Np;
    const int64_t rt = valid ? (rg >> 4) : 0;
    const int rr = (int)(rg & 15);
    const int prow = pair_row(rr);
    const uint8_t* wrow = a.w + rt * units * tile_stride + rr * 64 + h * 32;
    // scale planes follow the codes
    const uint8_t* planes = a.w + (k4 ? a.Np * a.Kp / 2 : a.Np * a.Kp);
    const uint16_t* sc16 = reinterpret_cast<const uint16_t*>(planes);
    const float* sc32 = reinterpret_cast<const float*>(planes);
    const uint16_t* mins = sc16 + a.Np * (a.Kp / 64);

    auto load_unit = [&](int u, uint4& q0, uint4& q1, float& d0, float& d1, float& m0, float& m1) {
      if (!valid || u >= units) {
        q0 = make_uint4(0, 0, 0, 0); q1 = q0; d0 = d1 = m0 = m1 = 0.f;
        return;
      }
      const uint4* p = reinterpret_cast<const uint4*>(wrow + (int64_t)u * tile_stride);
      q0 = ldg_nc_v4(p);
      q1 = ldg_nc_v4(p + 1);
      if constexpr (k4) {
        const int64_t si = ((rt * units + u) * 2) * 16 + prow;
        d0 = __half2float(__ushort_as_half(sc16[si]));
        d1 = __half2float(__ushort_as_half(sc16[si + 16]));
        if constexpr (WF == WF_ASYM_INT4) {
          m0 = __half2float(__ushort_as_half(mins[si]));
          m1 = __half2float(__ushort_as_half(mins[si + 16]));
        }
      } else if constexpr (WF == WF_INT8) {
        d0 = __half2float(__ushort_as_half(sc16[(rt * units + u) * 16 + prow]));
      } else {
        d0 = sc32[(rt * (a.Kp / 128) + (u >> 1)) * 16 + prow] * Fp8Place<T, WF>::mul;
      }
    };
    auto prefetch_unit = [&](int u) {
      if (valid && u < units) asm volatile("prefetch.global.L2 [%0];" ::"l"(wrow + (int64_t)u * tile_stride));
    };

    // two units are always in flight in registers (the loads of unit u+2 are issued before unit u is expanded), later
    // ones are pulled into L2: the dequantizers must never wait for DRAM
    uint4 n0, n1, p0, p1;
    float nd0 = 0.f, nd1 = 0.f, nm0 = 0.f, nm1 = 0.f, pd0 = 0.f, pd1 = 0.f, pm0 = 0.f, pm1 = 0.f;
    load_unit(0, n0, n1, nd0, nd1, nm0, nm1);
    load_unit(1, p0, p1, pd0, pd1, pm0, pm1);
#pragma unroll 1
    for (int u = 2; u <= 1 + kPrefetchUnits; ++u) prefetch_unit(u);

#pragma unroll 1
    for (int u = 0; u < units && ok; ++u) {
      const uint4 q0 = n0, q1 = n1;
      const float d0 = nd0, d1 = nd1, m0 = nm0, m1 = nm1;
      n0 = p0; n1 = p1; nd0 = pd0; nd1 = pd1; nm0 = pm0; nm1 = pm1;
      load_unit(u + 2, p0, p1, pd0, pd1, pm0, pm1);
      prefetch_unit(u + 2 + kPrefetchUnits);
      constexpr int kSub = k4 ? 2 : 1;  // stages fed by one unit
#pragma unroll
      for (int g = 0; g < kSub; ++g) {
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
          ok = false;
          if (lane == 0) report(a.err, 11);
          break;
        }
        Scale<T> sc;
        sc.d = V::splat(g == 0 ? d0 : d1);
        sc.m = V::splat(g == 0 ? m0 : m1);
        uint4 o[4];
        if constexpr (k4) {
          // uint4 = [group0: k 16t..16t+7 | 16t+8..16t+15 | group1: same]; this thread holds t = 2h, 2h+1
          o[0] = expand4<T, WF>(g == 0 ? q0.x : q0.z, sc, lut2);
          o[1] = expand4<T, WF>(g == 0 ? q0.y : q0.w, sc, lut2);
          o[2] = expand4<T, WF>(g == 0 ? q1.x : q1.z, sc, lut2);
          o[3] = expand4<T, WF>(g == 0 ? q1.y : q1.w, sc, lut2);
        } else {
          o[0] = expand8<T, WF>(q0.x, q0.y, sc);
          o[1] = expand8<T, WF>(q0.z, q0.w, sc);
          o[2] = expand8<T, WF>(q1.x, q1.y, sc);
          o[3] = expand8<T, WF>(q1.z, q1.w, sc);
        }
        uint8_t* row = sA + s * C::kABytes + r * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = 4 * h + j;  // 16-byte chunk = 8 consecutive k
          *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = o[j];
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[s]);
        if (++s == C::kStages) { s = 0; ph ^= 1; }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// tensor-parallel epilogue, second half: wait (bounded) until every rank's partial of (tile, lane quarter) has
// arrived in the local staging buffer, sum them in fp32, add bias / residual and store the finished rows.
// The counter is reset by its only reader, so a completed launch leaves all counters zero.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename T, int BT>
__device__ bool tp_finalize(const GemmArgs& a, int t, int qd, int lane, int ntiles, volatile int* abort_flag) {
  int* flag = a.tp_flags[a.tp_rank] + t * 4 + qd;
  int arrived = 0;
  if (lane == 0) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
      if (ld_acquire_sys(flag) >= a.tp_world) { arrived = 1; break; }
      __nanosleep(64);
      if ((i & 255) == 255 && *abort_flag) break;
    }
    if (arrived) *flag = 0;
    else {
      report(a.err, 14);
      *abort_flag = 1;
    }
  }
  arrived = __shfl_sync(0xffffffffu, arrived, 0);
  if (!arrived) return false;
  const int nb = t / a.m_tiles, mb = t % a.m_tiles;
  const int n = nb * kBM + qd * 32 + lane;
  if (n >= a.N) return true;
  T* out = reinterpret_cast<T*>(a.out);
  const T* res = reinterpret_cast<const T*>(a.residual);
  const float bv = a.bias != nullptr ? to_float(reinterpret_cast<const T*>(a.bias)[n]) : 0.f;
  const size_t tile_elems = (size_t)kBM * BT;
  const T* mine = reinterpret_cast<const T*>(a.tp_stage[a.tp_rank]);
#pragma unroll 1
  for (int c = 0; c < BT / 32; ++c) {
    float acc[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[j] = bv;
    for (int rk = 0; rk < a.tp_world; ++rk) {
      const uint4* src = reinterpret_cast<const uint4*>(mine + ((size_t)rk * ntiles + t) * tile_elems +
                                                        (size_t)(qd * 32 + lane) * BT + c * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 raw = __ldcg(src + q);   // written by peers: read through L2
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[q * 8 + j] += to_float(e[j]);
      }
    }
    const int m0 = mb * BT + c * 32;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int m = m0 + j;
      if (m < a.M) {
        float f = acc[j];
        if (res != nullptr) f += to_float(res[(int64_t)m * a.ldr + n]);
        out[(int64_t)m * a.ldo + n] = from_float<T>(f);
      }
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int BT, int WF>
__global__ void __launch_bounds__(Fam<WF>::threads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, GemmArgs a) {
  using C = Cfg<BT>;
  constexpr bool kDense = Fam<WF>::dense;
  int row0 = 0;
  if (a.m_range != nullptr) {
    row0 = a.m_range[0];
    a.M = a.m_range[1];
    a.m_tiles = (a.M + BT - 1) / BT;
    a.out = reinterpret_cast<T*>(a.out) + (int64_t)row0 * a.ldo;
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + C::kStages * C::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::kStages;
  uint64_t* acc_full = bars + 2 * C::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* lut2 = reinterpret_cast<uint32_t*>(smem + C::kStages * C::kStageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = a.m_tiles * a.n_tiles;
  const int kblocks = kDense ? (a.K + kBK - 1) / kBK : (int)(a.Kp / kBK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], kDense ? 1 : 1 + kDequantThreads / 32);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if constexpr (WF == WF_LUT4) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      const T lo = from_float<T>(a.lut[i & 15]), hi = from_float<T>(a.lut[i >> 4]);
      lut2[i] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&lo)) |
                ((uint32_t)(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- loader ----------------
    if (lane == 0) {
      if constexpr (kDense) prefetch_tmap(&tm_w);
      prefetch_tmap(&tm_x);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      uint32_t ag_ready = 0;  // ranks whose rows are known to have landed
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
        const int nb = t / a.m_tiles, mb = t % a.m_tiles;
        if (a.ag_flags != nullptr) {
          const int row_hi = (mb * BT + BT < a.M ? mb * BT + BT : a.M) - 1;
          for (int r = (mb * BT) / a.ag_rows; r <= row_hi / a.ag_rows && ok; ++r) {
            if (ag_ready & (1u << r)) continue;
            bool got = false;
            for (uint32_t it = 0; it < kSpinLimit; ++it) {
              if (ld_acquire_sys(a.ag_flags + r) - a.ag_epoch >= 0) { got = true; break; }
              if (it >= 64) {
                __nanosleep(it >= 4096 ? 256 : 32);
                if (*abort_flag) break;
              }
            }
            if (got) {
              ag_ready |= 1u << r;
              // the rows were written by a peer's generic stores; the TMA engine reads through the async proxy
              asm volatile("fence.proxy.async;" ::: "memory");
            } else {
              *abort_flag = 1;
              report(a.err, 15);
              ok = false;
            }
          }
          if (!ok) break;
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) { ok = false; report(a.err, 8); break; }
          mbar_expect_tx(&full[s], kDense ? C::kStageBytes : C::kBBytes);
          if constexpr (kDense) tma_load_2d(sA + s * C::kABytes, &tm_w, kb * kBK, nb * kBM, &full[s]);
          tma_load_2d(sB + s * C::kBBytes, &tm_x, kb * kBK, row0 + mb * BT, &full[s]);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {
        // leaving early: give the copies already issued a bounded time to land before the CTA exits
        for (int i = 0; i < C::kStages; ++i) mbar_wait_quiet(&full[i], 0, 1 << 12);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16<T>(kBM, BT);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1, abort_flag)) { report(a.err, 9); break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BT;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; report(a.err, 9); break; }
          tcgen05_fence_after();
          const uint64_t adesc = make_desc_sw128(smem_u32(sA + s * C::kABytes));
          const uint64_t bdesc = make_desc_sw128(smem_u32(sB + s * C::kBBytes));
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            // +32 bytes along K inside the swizzle row = +2 in the (address >> 4) field
            umma_f16(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb | kk) != 0);
          }
          umma_commit(&empty[s]);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ---------------- epilogue ----------------
    const int qd = warp & 3;  // TMEM lane quarter this warp may read
    T* out = reinterpret_cast<T*>(a.out);
    const T* res = reinterpret_cast<const T*>(a.residual);
    const T* bias = reinterpret_cast<const T*>(a.bias);
    if (a.ag_src != nullptr) {
      // ---- all-gather half of the fused op: push this rank's rows to every rank, then publish the epoch ----
      const int te = threadIdx.x - 64;                          // 0..127 over the four epilogue warps
      const int vec_per_row = a.K / 8;                          // 16-byte vectors per row
      int my_rows = a.M - a.tp_rank * a.ag_rows;
      my_rows = my_rows < 0 ? 0 : (my_rows > a.ag_rows ? a.ag_rows : my_rows);
      const int64_t total = (int64_t)my_rows * vec_per_row;
      const T* src = reinterpret_cast<const T*>(a.ag_src);
      for (int64_t v = (int64_t)blockIdx.x * 128 + te; v < total; v += (int64_t)gridDim.x * 128) {
        const int64_t row = v / vec_per_row, c = v % vec_per_row;
        const uint4 val = *reinterpret_cast<const uint4*>(src + row * a.ag_ld_src + c * 8);
        for (int p = 0; p < a.ag_world; ++p) {
          T* dst = reinterpret_cast<T*>(a.ag_dst[p]) + ((int64_t)a.tp_rank * a.ag_rows + row) * a.K + c * 8;
          *reinterpret_cast<uint4*>(dst) = val;
        }
      }
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps only
      if (te == 0) {
        const int ticket = atomicAdd(a.ag_ticket, 1);
        if (ticket == (int)gridDim.x - 1) {
          *a.ag_ticket = 0;                                     // ready for the next launch
          __threadfence_system();
          for (int p = 0; p < a.ag_world; ++p) st_release_sys(a.ag_peer_flags[p] + a.tp_rank, a.ag_epoch);
        }
      }
    }
    int it = 0;
    int prev_t = -1;      // tensor-parallel mode: tile whose partials are pushed but not yet reduced
    bool ok_tp = true;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
      const int nb = t / a.m_tiles, mb = t % a.m_tiles;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) report(a.err, 10);
        prev_t = -1;
        break;
      }
      tcgen05_fence_after();
      const int n = nb * kBM + qd * 32 + lane;
      const float bv = (bias != nullptr && n < a.N) ? to_float(bias[n]) : 0.f;
      if (a.tp_world > 1) {
        // ---- row-parallel layer: all-reduce fused into the epilogue, over NVLink peer memory ----
        // push: this rank's partial tile goes, as T, into slot [tp_rank][tile] of EVERY rank's staging buffer
        // (layout [weight row][token], so each lane writes 64 contiguous bytes per 32-token chunk), then the
        // (tile, lane-quarter) arrival counter of every rank is bumped with release semantics.
        const size_t tile_elems = (size_t)kBM * BT;
        const size_t slot = ((size_t)a.tp_rank * ntiles + t) * tile_elems + (size_t)(qd * 32 + lane) * BT;
#pragma unroll 1
        for (int c = 0; c < BT / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + (uint32_t(qd * 32) << 16) + acc * BT + c * 32, v);
          __align__(16) T packed[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) packed[j] = from_float<T>(__uint_as_float(v[j]));
          for (int rk = 0; rk < a.tp_world; ++rk) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.tp_stage[rk]) + slot + c * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = reinterpret_cast<const uint4*>(packed)[q];
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);      // TMEM is free again: the MMA of the next tile may start
        __threadfence_system();
        __syncwarp();
        if (lane < a.tp_world) red_release_sys_add(a.tp_flags[lane] + t * 4 + qd, 1);
        // finalize the PREVIOUS tile: its partials had a whole tile time to arrive
        if (prev_t >= 0) ok_tp = ok_tp && tp_finalize<T, BT>(a, prev_t, qd, lane, ntiles, abort_flag);
        prev_t = t;
        continue;
      }
      // activation mode: lanes 0..15 hold gate rows, lanes 16..31 the matching up rows; 16 outputs per warp
      const int n_out = a.act != 0 ? (nb * kBM + qd * 32) / 2 + (lane & 15) : n;
      const int n_lim = a.act != 0 ? a.N / 2 : a.N;
      const bool writer = a.act != 0 ? (lane < 16 && n_out < n_lim) : (n < a.N);
#pragma unroll 1
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (uint32_t(qd * 32) << 16) + acc * BT + c * 32, v);
        const int m0 = mb * BT + c * 32;
        if (a.act != 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(v[j]) + bv;
            const float u = __shfl_down_sync(0xffffffffu, g, 16);
            const int m = m0 + j;
            if (writer && m < a.M) out[(int64_t)m * a.ldo + n_out] = from_float<T>(act_apply(g, a.act) * u);
          }
        } else if (writer) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = m0 + j;
            if (m < a.M) {
              float f = __uint_as_float(v[j]) + bv;
              if (res != nullptr) f += to_float(res[(int64_t)m * a.ldr + n]);
              out[(int64_t)m * a.ldo + n] = from_float<T>(f);
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    if (a.tp_world > 1 && prev_t >= 0 && ok_tp) tp_finalize<T, BT>(a, prev_t, qd, lane, ntiles, abort_flag);
  } else {
    if constexpr (!kDense) dequant_role<T, BT, WF>(a, sA, full, empty, abort_flag, lut2);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <typename T, int BT, int WF>
cudaError_t launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int sms, cudaStream_t st) {
  using C = Cfg<BT>;
  auto kern = gemm_kernel<T, BT, WF>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int ntiles = a.m_tiles * a.n_tiles;
  const int grid = ntiles < sms ? ntiles : sms;
  kern<<<grid, Fam<WF>::threads, C::kSmemBytes, st>>>(tw, tx, a);
  return cudaGetLastError();
}

template <typename T, int WF>
cudaError_t dispatch_bt(int bt, const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int sms,
                        cudaStream_t st) {
  switch (bt) {
    case 32: return launch_gemm<T, 32, WF>(tw, tx, a, sms, st);
    case 64: return launch_gemm<T, 64, WF>(tw, tx, a, sms, st);
    case 128: return launch_gemm<T, 128, WF>(tw, tx, a, sms, st);
    default: return launch_gemm<T, 256, WF>(tw, tx, a, sms, st);
  }
}

template <typename T>
cudaError_t dispatch_wf(int wf, int bt, const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int sms,
                        cudaStream_t st) {
  switch (wf) {
    case WF_SYM_INT4: return dispatch_bt<T, WF_SYM_INT4>(bt, tw, tx, a, sms, st);
    case WF_ASYM_INT4: return dispatch_bt<T, WF_ASYM_INT4>(bt, tw, tx, a, sms, st);
    case WF_LUT4: return dispatch_bt<T, WF_LUT4>(bt, tw, tx, a, sms, st);
    case WF_FP8_E4M3: return dispatch_bt<T, WF_FP8_E4M3>(bt, tw, tx, a, sms, st);
    case WF_FP8_E5M2: return dispatch_bt<T, WF_FP8_E5M2>(bt, tw, tx, a, sms, st);
    case WF_INT8: return dispatch_bt<T, WF_INT8>(bt, tw, tx, a, sms, st);
    default: return cudaErrorInvalidValue;
  }
}

int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace

// Token tile the kernels use for M tokens.
IPEX_API int ipex_gemm_tcgen05_token_tile(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)); }

// out[M,N] = x[M,K] . w[N,K]^T (+ bias[N]) (+ residual[M,N]).  x, w, out, bias, residual share one 16-bit dtype.
// Row strides (elements): ldx, ldw multiples of 8 (TMA wants 16-byte strides); x and w 16-byte aligned.
// Returns a cudaError_t, or -1 when the driver's tensor-map encoder is unavailable / rejects the arguments.
IPEX_API int ipex_gemm_tcgen05_act(const void* x, const void* w, void* out, const void* bias, const void* residual,
                                   int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int64_t ldr, int dtype,
                                   int act, int* err, void* stream);

IPEX_API int ipex_gemm_tcgen05(const void* x, const void* w, void* out, const void* bias, const void* residual, int M,
                               int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int64_t ldr, int dtype, int* err,
                               void* stream) {
  return ipex_gemm_tcgen05_act(x, w, out, bias, residual, M, N, K, ldx, ldw, ldo, ldr, dtype, 0, err, stream);
}

// Dense GEMM with the gate/up activation epilogue: act != 0 expects w rows as 16-row tiles gate, up, gate, up, ...
// and writes act(gate) * up into N/2 columns (no residual then).
IPEX_API int ipex_gemm_tcgen05_act(const void* x, const void* w, void* out, const void* bias, const void* residual,
                                   int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int64_t ldr, int dtype,
                                   int act, int* err, void* stream) {
  if (M < 1 || N < 1 || K < 1 || (ldx % 8) != 0 || (ldw % 8) != 0) return (int)cudaErrorInvalidValue;
  if (act != 0 && (residual != nullptr || (N % 32) != 0)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return (int)cudaErrorInvalidValue;
  if (dtype != DT_F16 && dtype != DT_BF16) return (int)cudaErrorInvalidValue;
  const int bt = ipex_gemm_tcgen05_token_tile(M);
  const CUtensorMapDataType tdt = dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tw, tx;
  if (!tc5::encode_2d_sw128(&tw, tdt, w, (uint64_t)K, (uint64_t)N, (uint64_t)ldw * 2, kBK, kBM)) return -1;
  if (!tc5::encode_2d_sw128(&tx, tdt, x, (uint64_t)K, (uint64_t)M, (uint64_t)ldx * 2, kBK, bt)) return -1;
  GemmArgs a = {};
  a.out = out; a.bias = bias; a.residual = residual; a.ldo = ldo; a.ldr = ldr;
  a.M = M; a.N = N; a.K = K;
  a.m_tiles = (M + bt - 1) / bt;
  a.n_tiles = (N + kBM - 1) / kBM;
  a.act = act;
  a.err = err;
  cudaStream_t st = (cudaStream_t)stream;
  return (int)(dtype == DT_F16 ? dispatch_bt<__half, WF_F16>(bt, tw, tx, a, sm_count(), st)
                               : dispatch_bt<__nv_bfloat16, WF_F16>(bt, tw, tx, a, sm_count(), st));
}

// Same contraction with packed weights in the device tile layout (family `wf`); `act` != 0 applies act(gate) * up
// to 16-row-interleaved gate/up weights and writes N/2 columns (bias allowed, residual not).
IPEX_API int ipex_gemm_lowbit_tcgen05(const void* x, const void* w, void* out, const void* bias, const void* residual,
                                      const float* lut, int M, int N, int K, int64_t ldx, int64_t ldo, int64_t ldr,
                                      int wf, int act, int dtype, int* err, void* stream) {
  if (M < 1 || N < 1 || K < 1 || (ldx % 8) != 0) return (int)cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(x) & 15) return (int)cudaErrorInvalidValue;
  if (dtype != DT_F16 && dtype != DT_BF16) return (int)cudaErrorInvalidValue;
  if (act != 0 && (residual != nullptr || (N % 32) != 0)) return (int)cudaErrorInvalidValue;
  if (wf == WF_LUT4 && lut == nullptr) return (int)cudaErrorInvalidValue;
  const int bt = ipex_gemm_tcgen05_token_tile(M);
  const CUtensorMapDataType tdt = dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tx;
  if (!tc5::encode_2d_sw128(&tx, tdt, x, (uint64_t)K, (uint64_t)M, (uint64_t)ldx * 2, kBK, bt)) return -1;
  GemmArgs a = {};
  a.w = reinterpret_cast<const uint8_t*>(w); a.lut = lut;
  a.out = out; a.bias = bias; a.residual = residual; a.ldo = ldo; a.ldr = ldr;
  a.Np = ceil_to_i64(N, 16); a.Kp = ceil_to_i64(K, 128);
  a.M = M; a.N = N; a.K = K;
  a.m_tiles = (M + bt - 1) / bt;
  a.n_tiles = (N + kBM - 1) / kBM;
  a.act = act;
  a.err = err;
  cudaStream_t st = (cudaStream_t)stream;
  return (int)(dtype == DT_F16 ? dispatch_wf<__half>(wf, bt, tx, tx, a, sm_count(), st)
                               : dispatch_wf<__nv_bfloat16>(wf, bt, tx, tx, a, sm_count(), st));
}

// Grouped form for mixture-of-experts prompts: rows [m_range[0], m_range[0] + m_range[1]) of x [M_total, K] times
// one expert's packed weight into the same rows of out [M_total, N (or N / 2 with act)].  m_range is a DEVICE pointer
// to (first row, row count): the host launches every expert without knowing its token count.  `bt` is the token
// tile (32 / 64 / 128 / 256); the grid is sized for m_upper rows, CTAs beyond the real tile count leave at once.
IPEX_API int ipex_gemm_lowbit_tcgen05_grouped(const void* x, const void* w, void* out, const float* lut,
                                              const int* m_range, int M_total, int m_upper, int N, int K, int64_t ldx,
                                              int64_t ldo, int wf, int act, int dtype, int bt, int* err, void* stream) {
  if (M_total < 1 || m_upper < 1 || N < 1 || K < 1 || (ldx % 8) != 0 || m_range == nullptr)
    return (int)cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(x) & 15) return (int)cudaErrorInvalidValue;
  if (dtype != DT_F16 && dtype != DT_BF16) return (int)cudaErrorInvalidValue;
  if (act != 0 && (N % 32) != 0) return (int)cudaErrorInvalidValue;
  if (wf == WF_LUT4 && lut == nullptr) return (int)cudaErrorInvalidValue;
  if (bt != 32 && bt != 64 && bt != 128 && bt != 256) return (int)cudaErrorInvalidValue;
  const CUtensorMapDataType tdt = dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tx;
  if (!tc5::encode_2d_sw128(&tx, tdt, x, (uint64_t)K, (uint64_t)M_total, (uint64_t)ldx * 2, kBK, bt)) return -1;
  GemmArgs a = {};
  a.w = reinterpret_cast<const uint8_t*>(w); a.lut = lut;
  a.out = out; a.bias = nullptr; a.residual = nullptr; a.ldo = ldo; a.ldr = 0;
  a.Np = ceil_to_i64(N, 16); a.Kp = ceil_to_i64(K, 128);
  a.M = m_upper; a.N = N; a.K = K;
  a.m_tiles = (m_upper + bt - 1) / bt;
  a.n_tiles = (N + kBM - 1) / kBM;
  a.act = act;
  a.err = err;
  a.m_range = m_range;
  cudaStream_t st = (cudaStream_t)stream;
  return (int)(dtype == DT_F16 ? dispatch_wf<__half>(wf, bt, tx, tx, a, sm_count(), st)
                               : dispatch_wf<__nv_bfloat16>(wf, bt, tx, tx, a, sm_count(), st));
}

// Bytes of staging every rank must provide for ipex_gemm_lowbit_tcgen05_ar (one parity), and number of counters.
IPEX_API int64_t ipex_gemm_tcgen05_ar_stage_bytes(int M, int N, int world) {
  const int bt = ipex_gemm_tcgen05_token_tile(M);
  const int64_t tiles = (int64_t)((M + bt - 1) / bt) * ((N + kBM - 1) / kBM);
  return (int64_t)world * tiles * kBM * bt * 2;
}
IPEX_API int64_t ipex_gemm_tcgen05_ar_counters(int M, int N) {
  const int bt = ipex_gemm_tcgen05_token_tile(M);
  return (int64_t)((M + bt - 1) / bt) * ((N + kBM - 1) / kBM) * 4;
}

// Row-parallel layer of a tensor-parallel model: out = sum over ranks of x_r . W_r^T (+ bias) (+ residual), the
// all-reduce running inside the GEMM's epilogue over NVLink peer memory (plain peer stores + release / acquire
// counters; no multicast).  Every rank launches the same shape.  tp_stage / tp_flags: device arrays of `world`
// pointers into the ranks' symmetric buffers for this call's parity (two parities alternate between consecutive
// calls); counters zero before the first call, left zero.  Bounded waits: *err = 14 when a peer never arrives.
IPEX_API int ipex_gemm_lowbit_tcgen05_ar(const void* x, const void* w, void* out, const void* bias,
                                         const void* residual, const float* lut, int M, int N, int K, int64_t ldx,
                                         int64_t ldo, int64_t ldr, int wf, int dtype, int* err, void* stream,
                                         int tp_rank, int tp_world, const void* tp_stage, const void* tp_flags) {
  if (M < 1 || N < 1 || K < 1 || (ldx % 8) != 0) return (int)cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(x) & 15) return (int)cudaErrorInvalidValue;
  if (dtype != DT_F16 && dtype != DT_BF16) return (int)cudaErrorInvalidValue;
  if (tp_world < 2 || tp_world > 8 || tp_rank < 0 || tp_rank >= tp_world || tp_stage == nullptr || tp_flags == nullptr)
    return (int)cudaErrorInvalidValue;
  if (wf == WF_LUT4 && lut == nullptr) return (int)cudaErrorInvalidValue;
  const int bt = ipex_gemm_tcgen05_token_tile(M);
  const CUtensorMapDataType tdt = dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tx;
  if (!tc5::encode_2d_sw128(&tx, tdt, x, (uint64_t)K, (uint64_t)M, (uint64_t)ldx * 2, kBK, bt)) return -1;
  GemmArgs a = {};
  a.w = reinterpret_cast<const uint8_t*>(w); a.lut = lut;
  a.out = out; a.bias = bias; a.residual = residual; a.ldo = ldo; a.ldr = ldr;
  a.Np = ceil_to_i64(N, 16); a.Kp = ceil_to_i64(K, 128);
  a.M = M; a.N = N; a.K = K;
  a.m_tiles = (M + bt - 1) / bt;
  a.n_tiles = (N + kBM - 1) / kBM;
  a.act = 0;
  a.err = err;
  a.tp_rank = tp_rank; a.tp_world = tp_world;
  a.tp_stage = reinterpret_cast<void* const*>(tp_stage);
  a.tp_flags = reinterpret_cast<int* const*>(tp_flags);
  cudaStream_t st = (cudaStream_t)stream;
  return (int)(dtype == DT_F16 ? dispatch_wf<__half>(wf, bt, tx, tx, a, sm_count(), st)
                               : dispatch_wf<__nv_bfloat16>(wf, bt, tx, tx, a, sm_count(), st));
}

// Column-parallel layer behind an all-gather, as ONE kernel: every rank holds `ag_rows` consecutive token rows of
// the activation (x_local, row stride ld_local; rank r owns rows [r * ag_rows, ...) of the M gathered rows).  The
// kernel's epilogue warps push those rows into every rank's gathered buffer (plain peer stores over NVLink) and
// publish `epoch` in the ranks' flag arrays; its loader waits, per token tile, for the flags of the ranks whose rows
// the tile covers and then reads the tile from THIS rank's copy with TMA, so tiles of rows that have arrived are
// multiplied while later rows are still in flight.  out = gathered_x . W^T (+ bias), optional act(gate) * up.
//   xg          this rank's gathered buffer [M, K] (row stride K), 16-byte aligned, in symmetric memory
//   ag_dst      device array of `world` pointers: every rank's gathered buffer (same parity)
//   ag_flags    device array of `world` pointers: every rank's flag array [world] ints (same parity)
//   my_flags    this rank's flag array (= ag_flags[rank]);  ticket: one zeroed int on this device, left zero
// Flags only grow (epochs increase from call to call); waits are bounded: *err = 15 when a peer never arrives.
IPEX_API int ipex_gemm_lowbit_tcgen05_ag(const void* x_local, int64_t ld_local, const void* xg, const void* w,
                                         void* out, const void* bias, const float* lut, int M, int N, int K,
                                         int64_t ldo, int wf, int act, int dtype, int* err, void* stream, int rank,
                                         int world, int ag_rows, const void* ag_dst, const void* ag_flags,
                                         const int* my_flags, int* ticket, int epoch) {
  if (M < 1 || N < 1 || K < 1 || (K % 8) != 0 || (ld_local % 8) != 0) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(xg) & 15) || (reinterpret_cast<uintptr_t>(x_local) & 15))
    return (int)cudaErrorInvalidValue;
  if (dtype != DT_F16 && dtype != DT_BF16) return (int)cudaErrorInvalidValue;
  if (world < 2 || world > 8 || rank < 0 || rank >= world || ag_rows < 1 || (int64_t)ag_rows * world < M ||
      ag_dst == nullptr || ag_flags == nullptr || my_flags == nullptr || ticket == nullptr)
    return (int)cudaErrorInvalidValue;
  if (act != 0 && (N % 32) != 0) return (int)cudaErrorInvalidValue;
  if (wf == WF_LUT4 && lut == nullptr) return (int)cudaErrorInvalidValue;
  if (wf == WF_F16 || wf == WF_BF16) return (int)cudaErrorInvalidValue;
  const int bt = ipex_gemm_tcgen05_token_tile(M);
  const CUtensorMapDataType tdt = dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tx;
  if (!tc5::encode_2d_sw128(&tx, tdt, xg, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, bt)) return -1;
  GemmArgs a = {};
  a.w = reinterpret_cast<const uint8_t*>(w); a.lut = lut;
  a.out = out; a.bias = bias; a.residual = nullptr; a.ldo = ldo; a.ldr = 0;
  a.Np = ceil_to_i64(N, 16); a.Kp = ceil_to_i64(K, 128);
  a.M = M; a.N = N; a.K = K;
  a.m_tiles = (M + bt - 1) / bt;
  a.n_tiles = (N + kBM - 1) / kBM;
  a.act = act;
  a.err = err;
  a.tp_rank = rank; a.tp_world = 1;    // no reduction of the output: every rank owns its own columns
  a.ag_flags = my_flags; a.ag_rows = ag_rows; a.ag_epoch = epoch;
  a.ag_src = x_local; a.ag_ld_src = ld_local;
  a.ag_dst = reinterpret_cast<void* const*>(ag_dst);
  a.ag_peer_flags = reinterpret_cast<int* const*>(ag_flags);
  a.ag_ticket = ticket; a.ag_world = world;
  cudaStream_t st = (cudaStream_t)stream;
  return (int)(dtype == DT_F16 ? dispatch_wf<__half>(wf, bt, tx, tx, a, sm_count(), st)
                               : dispatch_wf<__nv_bfloat16>(wf, bt, tx, tx, a, sm_count(), st));
}
