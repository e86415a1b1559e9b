// Low-bit GEMV / skinny GEMM for decode (M <= 8), register-prefetch version for the 4-bit families, sm_100a.
//
// Same contract and tile layout as gemv_lowbit.cu.  Differences, both aimed at the latency-bound nature of a
// microsecond-long weight stream:
//   * software pipelining in registers: the 16-byte tile slices (and scales) of the next PF steps are in flight
//     while the current one goes through the tensor-core pipe, so a warp keeps PF+1 kilobytes outstanding
//     instead of one;
//   * offset-free dequantization: a masked nibble pair OR-ed with the fp16 magic number is fed to the mma as is
//     (values 1024+q and 1024+16q); the activations that meet the "16q" operands are staged pre-divided by 16
//     and the constant parts are removed from the fp32 accumulator once per 64-group.  One logic instruction
//     per weight pair instead of two instructions.
// Each CTA owns RT row tiles; its 8 warps split K.
#include "common/utils.cuh"

namespace {

constexpr int kW = 8;
constexpr int kT = kW * 32;

struct DArgs {
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
  int act;
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Int4Raw {
  uint32_t p[4];
  __device__ __forceinline__ explicit Int4Raw(uint32_t u) {
    constexpr uint32_t kMagic = 0x64006400u;
    const uint32_t u2 = u >> 8;
    p[0] = (u & 0x000F000Fu) | kMagic;   // 1024 + q   : weights 0,1
    p[1] = (u & 0x00F000F0u) | kMagic;   // 1024 + 16q : weights 2,3
    p[2] = (u2 & 0x000F000Fu) | kMagic;  // weights 4,5
    p[3] = (u2 & 0x00F000F0u) | kMagic;  // weights 6,7
  }
};

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == 1) return g / (1.0f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.0f + tanhf(k0 * (g + k1 * g * g * g)));
}

// one pipeline step of a lane: its slices of one [16 rows x 128 k] tile
template <bool ASYM>
struct Frag {
  uint4 qa, qb;
  uint32_t s0, s1, m0, m1;
  __device__ __forceinline__ void load(const uint8_t* codes, const uint8_t* scales, const uint8_t* mins, size_t tile,
                                       int g, int t) {
    const uint8_t* tp = codes + tile * 1024;
    qa = ldg_nc_v4(tp + g * 64 + t * 16);
    qb = ldg_nc_v4(tp + (g + 8) * 64 + t * 16);
    s0 = ldg_nc_u32(scales + ((tile * 2 + 0) * 16 + 2 * g) * 2);
    s1 = ldg_nc_u32(scales + ((tile * 2 + 1) * 16 + 2 * g) * 2);
    if (ASYM) {
      m0 = ldg_nc_u32(mins + ((tile * 2 + 0) * 16 + 2 * g) * 2);
      m1 = ldg_nc_u32(mins + ((tile * 2 + 1) * 16 + 2 * g) * 2);
    }
  }
};

template <int WF, typename T, int RT, int PF>
__global__ void __launch_bounds__(kT) gemv_direct_kernel(DArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr bool ASYM = WF == WF_ASYM_INT4;
  const int Kp = (int)ceil_to_i64(a.K, 128);
  const int Np = (int)ceil_to_i64(a.N, 16);
  const int chunks = Kp / 128;
  const int groups = Kp / 64;
  const int xs_stride = Kp + 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tile_row0 = blockIdx.x * RT;
  const int ntiles = Np / 16;

  __half* xs = reinterpret_cast<__half*>(smem_raw);
  size_t off = ((size_t)a.M * xs_stride * sizeof(__half) + 15) & ~(size_t)15;
  float* red = reinterpret_cast<float*>(smem_raw + off);          // [kW][RT][16][8]
  off += (size_t)kW * RT * 128 * sizeof(float);
  float* scratch = reinterpret_cast<float*>(smem_raw + off);
  off += 64;
  float* xcorr = reinterpret_cast<float*>(smem_raw + off);        // [M][groups]
  off += (size_t)a.M * groups * sizeof(float);
  float* xsum = reinterpret_cast<float*>(smem_raw + off);         // asym: [M][groups]

  const uint8_t* codes = a.w;
  const uint8_t* scales = a.w + (size_t)Np * Kp / 2;
  const uint8_t* mins = scales + (size_t)Np * groups * 2;

  // ---- weights do not depend on the previous kernel: start the pipeline before waiting for it ----
  // step s of this warp = (row tile r = s % RT, chunk c = warp + kW * (s / RT))
  const int my_chunks = (chunks - warp + kW - 1) / kW;
  const int nsteps = chunks > warp ? my_chunks * RT : 0;
  Frag<ASYM> f[PF];
#pragma unroll
  for (int p = 0; p < PF; p++) {
    if (p < nsteps) {
      const int r = p % RT, c = warp + kW * (p / RT);
      if (tile_row0 + r < ntiles) f[p].load(codes, scales, mins, (size_t)(tile_row0 + r) * chunks + c, g, t);
    }
  }
  pdl_launch_dependents();
  pdl_wait();

  // ---- stage x: fp16, optionally RMS-normalised, "16q" partners pre-divided by 16 ----
  {
    const T* x = reinterpret_cast<const T*>(a.x);
    const T* nw = reinterpret_cast<const T*>(a.norm_w);
    const int nvec = a.K / 8;
    for (int m = 0; m < a.M; m++) {
      const T* xr = x + (size_t)m * a.ldx;
      float rstd = 1.0f;
      if (nw != nullptr) {
        float ss = 0.f;
        for (int v = tid; v < nvec; v += kT) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; j++) { const float fv = DT<T>::to_f(e[j]); ss += fv * fv; }
        }
        ss = warp_sum(ss);
        if (lane == 0) scratch[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kW; w++) tot += scratch[w];
        rstd = rsqrtf(tot / (float)a.K + a.eps);
        __syncthreads();
      }
      for (int v = tid; v < Kp / 8; v += kT) {
        __align__(16) __half o[8];
        if (v < nvec) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
          const T* e = reinterpret_cast<const T*>(&raw);
          uint4 wraw = make_uint4(0, 0, 0, 0);
          if (nw != nullptr) wraw = *reinterpret_cast<const uint4*>(nw + v * 8);
          const T* we = reinterpret_cast<const T*>(&wraw);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            float fv = DT<T>::to_f(e[j]);
            if (nw != nullptr) fv = fv * rstd * (DT<T>::to_f(we[j]) + a.norm_offset);
            fv = fminf(fmaxf(fv, -65504.f), 65504.f);
            if (j & 2) fv *= 0.0625f;
            o[j] = __float2half_rn(fv);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; j++) o[j] = __float2half_rn(0.f);
        }
        *reinterpret_cast<uint4*>(xs + m * xs_stride + v * 8) = *reinterpret_cast<const uint4*>(o);
      }
    }
    __syncthreads();
    const float zlo = ASYM ? 1024.f : 1032.f;
    const float zhi = ASYM ? 1024.f : 1152.f;
    for (int i = tid; i < a.M * groups; i += kT) {
      const int m = i / groups, gi = i % groups;
      float slo = 0.f, shi = 0.f;
      const __half* xp = xs + m * xs_stride + gi * 64;
#pragma unroll 8
      for (int k = 0; k < 64; k++) {
        const float v = __half2float(xp[k]);
        if (k & 2) shi += v; else slo += v;
      }
      xcorr[i] = zlo * slo + zhi * shi;
      if (ASYM) xsum[i] = slo + 16.f * shi;
    }
    __syncthreads();
  }

  float acc[RT][4];
#pragma unroll
  for (int r = 0; r < RT; r++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[r][i] = 0.f;
  const bool has_x = g < a.M;
  const int n0 = 2 * t, n1 = 2 * t + 1;

  uint4 xa0 = make_uint4(0, 0, 0, 0), xa1 = xa0, xb0 = xa0, xb1 = xa0;
  for (int s0i = 0; s0i < nsteps; s0i += PF) {
#pragma unroll
    for (int p = 0; p < PF; p++) {
      const int s = s0i + p;
      if (s < nsteps) {
        const int r = s % RT, c = warp + kW * (s / RT);
        const Frag<ASYM> cur = f[p];
        // refill this slot with the step PF ahead
        const int sn = s + PF;
        if (sn < nsteps) {
          const int rn = sn % RT, cn = warp + kW * (sn / RT);
          if (tile_row0 + rn < ntiles) f[p].load(codes, scales, mins, (size_t)(tile_row0 + rn) * chunks + cn, g, t);
        }
        if (r == 0 && has_x) {
          const __half* xp = xs + g * xs_stride + c * 128 + 16 * t;
          xa0 = *reinterpret_cast<const uint4*>(xp);
          xa1 = *reinterpret_cast<const uint4*>(xp + 8);
          xb0 = *reinterpret_cast<const uint4*>(xp + 64);
          xb1 = *reinterpret_cast<const uint4*>(xp + 72);
        }
        if (tile_row0 + r < ntiles) {
          float c0v[4] = {0.f, 0.f, 0.f, 0.f}, c0w[4] = {0.f, 0.f, 0.f, 0.f};
          float c1v[4] = {0.f, 0.f, 0.f, 0.f}, c1w[4] = {0.f, 0.f, 0.f, 0.f};
          {
            Int4Raw A(cur.qa.x), B(cur.qb.x);
            mma_f16(c0v, A.p[0], B.p[0], A.p[1], B.p[1], xa0.x, xa0.y);
            mma_f16(c0w, A.p[2], B.p[2], A.p[3], B.p[3], xa0.z, xa0.w);
          }
          {
            Int4Raw A(cur.qa.z), B(cur.qb.z);
            mma_f16(c1v, A.p[0], B.p[0], A.p[1], B.p[1], xb0.x, xb0.y);
            mma_f16(c1w, A.p[2], B.p[2], A.p[3], B.p[3], xb0.z, xb0.w);
          }
          {
            Int4Raw A(cur.qa.y), B(cur.qb.y);
            mma_f16(c0v, A.p[0], B.p[0], A.p[1], B.p[1], xa1.x, xa1.y);
            mma_f16(c0w, A.p[2], B.p[2], A.p[3], B.p[3], xa1.z, xa1.w);
          }
          {
            Int4Raw A(cur.qa.w), B(cur.qb.w);
            mma_f16(c1v, A.p[0], B.p[0], A.p[1], B.p[1], xb1.x, xb1.y);
            mma_f16(c1w, A.p[2], B.p[2], A.p[3], B.p[3], xb1.z, xb1.w);
          }
          const float k00 = n0 < a.M ? xcorr[n0 * groups + 2 * c] : 0.f;
          const float k01 = n0 < a.M ? xcorr[n0 * groups + 2 * c + 1] : 0.f;
          const float k10 = n1 < a.M ? xcorr[n1 * groups + 2 * c] : 0.f;
          const float k11 = n1 < a.M ? xcorr[n1 * groups + 2 * c + 1] : 0.f;
          const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&cur.s0));
          const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&cur.s1));
          acc[r][0] += d0.x * (c0v[0] + c0w[0] - k00) + d1.x * (c1v[0] + c1w[0] - k01);
          acc[r][1] += d0.x * (c0v[1] + c0w[1] - k10) + d1.x * (c1v[1] + c1w[1] - k11);
          acc[r][2] += d0.y * (c0v[2] + c0w[2] - k00) + d1.y * (c1v[2] + c1w[2] - k01);
          acc[r][3] += d0.y * (c0v[3] + c0w[3] - k10) + d1.y * (c1v[3] + c1w[3] - k11);
          if (ASYM) {
            const float2 mn0 = __half22float2(*reinterpret_cast<const __half2*>(&cur.m0));
            const float2 mn1 = __half22float2(*reinterpret_cast<const __half2*>(&cur.m1));
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
    for (int i = tid; i < RT * 128; i += kT) {
      const int r = i / 128, col = (i % 128) / 16, row = i % 16;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kW; w++) s += red[((size_t)(w * RT + r) * 16 + row) * 8 + col];
      const int n = (tile_row0 + r) * 16 + row;
      if (n < a.N && col < a.M) {
        if (a.bias != nullptr) s += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[n]);
        if (a.residual != nullptr) s += DT<T>::to_f(reinterpret_cast<const T*>(a.residual)[(size_t)col * a.ldr + n]);
        y[(size_t)col * a.ldy + n] = DT<T>::from_f(s);
      }
    }
  } else if (RT == 2) {
    if (tid < 128) {
      const int col = tid / 16, row = tid % 16;
      float gsum = 0.f, usum = 0.f;
#pragma unroll
      for (int w = 0; w < kW; w++) {
        gsum += red[((size_t)(w * RT + 0) * 16 + row) * 8 + col];
        usum += red[((size_t)(w * RT + 1) * 16 + row) * 8 + col];
      }
      const int n = blockIdx.x * 16 + row;
      if (n < a.N / 2 && col < a.M) {
        if (a.bias != nullptr) {
          gsum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)blockIdx.x * 32 + row]);
          usum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)blockIdx.x * 32 + 16 + row]);
        }
        y[(size_t)col * a.ldy + n] = DT<T>::from_f(act_apply(gsum, a.act) * usum);
      }
    }
  }
}

int g_pf = 4;

template <int WF, typename T, int RT, int PF>
cudaError_t launch_pf(const DArgs& a, cudaStream_t stream, bool pdl) {
  const int Kp = (int)ceil_to_i64(a.K, 128);
  const int Np = (int)ceil_to_i64(a.N, 16);
  size_t smem = (((size_t)a.M * (Kp + 8) * 2 + 15) & ~(size_t)15) + (size_t)kW * RT * 128 * 4 + 64 +
                (size_t)a.M * (Kp / 64) * 4 * (WF == WF_ASYM_INT4 ? 2 : 1);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  auto kern = gemv_direct_kernel<WF, T, RT, PF>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  dim3 grid((Np / 16 + RT - 1) / RT);
  return launch_kernel(kern, grid, dim3(kT), smem, stream, pdl, a);
}

template <int WF, typename T, int RT>
cudaError_t launch_d(const DArgs& a, cudaStream_t s, bool pdl) {
  switch (g_pf) {
    case 2: return launch_pf<WF, T, RT, 2>(a, s, pdl);
    case 6: return launch_pf<WF, T, RT, 6>(a, s, pdl);
    default: return launch_pf<WF, T, RT, 4>(a, s, pdl);
  }
}

template <typename T>
cudaError_t dispatch(int wf, const DArgs& a, cudaStream_t s, bool pdl) {
  if (wf == WF_SYM_INT4) return a.act ? launch_d<WF_SYM_INT4, T, 2>(a, s, pdl) : launch_d<WF_SYM_INT4, T, 1>(a, s, pdl);
  if (wf == WF_ASYM_INT4)
    return a.act ? launch_d<WF_ASYM_INT4, T, 2>(a, s, pdl) : launch_d<WF_ASYM_INT4, T, 1>(a, s, pdl);
  return cudaErrorInvalidValue;
}

}  // namespace

// prefetch depth (2, 4 or 6 pipeline steps per warp)
IPEX_API void ipex_gemv_direct_tune(int prefetch_steps) {
  if (prefetch_steps == 2 || prefetch_steps == 4 || prefetch_steps == 6) g_pf = prefetch_steps;
}

// Integer 4-bit families only (sym_int4 / asym_int4); same arguments as ipex_gemv_lowbit.
IPEX_API int ipex_gemv_int4_direct(const void* w, int wf, const void* x, void* y, int M, int N, int K, int ldx, int ldy,
                                   const void* norm_w, float eps, float norm_offset, const void* bias,
                                   const void* residual, int ldr, int act, const float* lut, int dtype, int pdl,
                                   void* stream) {
  if (M < 1 || M > 8 || (K % 64) != 0) return (int)cudaErrorInvalidValue;
  if ((ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return (int)cudaErrorInvalidValue;
  DArgs a;
  a.w = (const uint8_t*)w; a.x = x; a.y = y; a.norm_w = norm_w; a.bias = bias; a.residual = residual; a.lut = lut;
  a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.ldr = ldr; a.eps = eps; a.norm_offset = norm_offset;
  a.act = act;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) return (int)dispatch<__half>(wf, a, s, pdl != 0);
  if (dtype == DT_BF16) return (int)dispatch<__nv_bfloat16>(wf, a, s, pdl != 0);
  return (int)cudaErrorInvalidValue;
}
