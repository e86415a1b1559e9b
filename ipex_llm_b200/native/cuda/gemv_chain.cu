// A chain of dependent decode GEMVs in ONE persistent kernel (symmetric int4 weights, integer tensor-core path).
//
// A decoder layer's token step is   ... attention -> o_proj -> gate/up (+act) -> down -> next layer's qkv ...
// Run as separate kernels, each of these pays a launch, a prologue (stage and normalise x), a cold start of its
// weight stream and a tail, which together cost more than streaming the weights.  Here up to four GEMVs run
// inside one launch of one CTA per SM:
//   * the producer warp walks the CTA's weight tiles of ALL ops back to back with cp.async.bulk into one ring of
//     stages, so the HBM stream never drains between ops: while the consumers are in the grid barrier that
//     separates two ops, the next op's weights are already landing in shared memory;
//   * sixteen consumer warps stage x for the op (RMS norm fused, activations quantised to 15-bit hi/lo int8 pairs
//     with one scale per token), run the s8 tensor-core pipeline out of shared memory, reduce across warps with the
//     ticket scheme of the single-op kernel and apply the epilogue (bias, residual, act(gate) * up);
//   * between ops a grid-wide barrier (one global arrival counter, monotonically increasing within the launch,
//     bounded spin) makes every CTA's outputs visible before anyone stages them as the next op's x.
// All CTAs are co-resident (grid <= number of SMs, one CTA per SM), which the barrier needs; kernels launched before
// this one always terminate on their own, so late-starting CTAs only delay the barrier.
// Every wait is bounded; on expiry the kernel records a code in *err (21 producer, 22 consumer, 23 reduction
// buffer, 24 grid barrier) and every role leaves.
//
// Reference counterpart: none as one kernel; the reference launches xe_linear.forward_new per projection
// (python/llm/src/ipex_llm/transformers/low_bit_linear.py:640-668).
#include "common/utils.cuh"

namespace {

constexpr int kCW = 16;                       // consumer warps
constexpr int kCThreads = kCW * 32;           // 512
constexpr int kThreads = kCThreads + 32;      // + producer warp
constexpr int kSpin = 1 << 22;
constexpr int kNB = 4;                        // reduction buffers in flight
constexpr int kCPS = 16;                      // 128-k chunks per stage
constexpr int kCB = 1024, kSB = 64;           // code / scale bytes per chunk
constexpr int kStageBytes = kCPS * (kCB + kSB);
constexpr int kPad = 64;                      // extra bytes per staged token row (bank spread)
constexpr int kMaxOps = 4;

struct ChainOp {
  const uint8_t* w;
  const void* x;
  void* y;
  const void* norm_w;
  const void* bias;
  const void* residual;
  int N, K, ldx, ldy, ldr, act;
  float eps, norm_offset;
};

struct ChainArgs {
  ChainOp op[kMaxOps];
  int nops, M, stages, kp_max;
  unsigned int* barrier;  // [2]: arrival counter, exit counter (both zero between launches)
  int* err;
};

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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
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
    if (i >= 2) {
      __nanosleep(i < 32 ? 32 : 128);
      if ((i & 63) == 0 && *abort_flag) return false;
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCThreads) : "memory"); }

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float act_apply(float g, int act) {
  if (act == 1) return g / (1.0f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.0f + tanhf(k0 * (g + k1 * g * g * g)));
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct Ctx {
  uint8_t* ring;
  uint64_t* full_bar;
  uint64_t* empty_bar;
  int8_t* xh;
  int8_t* xl;
  float* red;      // [kNB][2][128]
  int* red_cnt;    // [kNB]
  int* red_gen;    // [kNB]
  float* scratch;  // [2 * kCW]
  float* dxs;      // [8]
  int2* seeds;     // [kp_max / 64][8]
  volatile int* abort_flag;
  int stages;
  int xs_stride;
};

// x -> (hi, lo) int8 rows in the octet order (k0,k4,k1,k5 | k2,k6,k3,k7), per-token scale, accumulator seeds.
template <typename T>
__device__ void stage_x_i8(const ChainOp& a, int M, const Ctx& c, int Kp) {
  const int tid = threadIdx.x;
  const T* x = reinterpret_cast<const T*>(a.x);
  const T* nw = reinterpret_cast<const T*>(a.norm_w);
  const int nvec = a.K / 8;
  const int groups = Kp / 64;
  for (int i = tid; i < groups * 8; i += kCThreads)
    if ((i & 7) >= M) c.seeds[i] = make_int2(0, 0);
  if (tid < 8) c.dxs[tid] = 0.f;
  for (int m = 0; m < M; m++) {
    const T* xr = x + (size_t)m * a.ldx;
    float ss = 0.f, mx = 0.f;
    for (int v = tid; v < nvec; v += kCThreads) {
      const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(xr + v * 8));  // L2: written by other SMs
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
    const float rstd = nw != nullptr ? rsqrtf(tot / (float)a.K + a.eps) : 1.0f;
    amax *= rstd;
    const float dx = amax > 0.f ? amax / 16383.f : 1.0f;
    const float inv = rstd / dx;
    if (tid == 0) c.dxs[m] = dx;
    consumer_sync();
    for (int v0 = 0; v0 < Kp / 8; v0 += kCThreads) {
      const int v = v0 + tid;
      int sh = 0, sl = 0;
      if (v < Kp / 8) {
        uint32_t ph[2] = {0, 0}, pl[2] = {0, 0};
        if (v < nvec) {
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(xr + v * 8));  // L2: written by other SMs
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
        *reinterpret_cast<uint2*>(c.xh + (size_t)m * c.xs_stride + v * 8) = make_uint2(ph[0], ph[1]);
        *reinterpret_cast<uint2*>(c.xl + (size_t)m * c.xs_stride + v * 8) = make_uint2(pl[0], pl[1]);
      }
      sh += __shfl_xor_sync(0xffffffffu, sh, 1); sl += __shfl_xor_sync(0xffffffffu, sl, 1);
      sh += __shfl_xor_sync(0xffffffffu, sh, 2); sl += __shfl_xor_sync(0xffffffffu, sl, 2);
      sh += __shfl_xor_sync(0xffffffffu, sh, 4); sl += __shfl_xor_sync(0xffffffffu, sl, 4);
      if ((tid & 7) == 0 && v < Kp / 8) c.seeds[(v >> 3) * 8 + m] = make_int2(-8 * sh, -8 * sl);
    }
  }
}

// One op on the consumer side.  `it` (stage iteration) and `giter` (reduction-buffer generation) run on across ops.
template <typename T, int RT>
__device__ bool consume_op(const ChainOp& a, int M, const Ctx& c, int& it, int& giter, int* err) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int Kp = (int)ceil_to_i64(a.K, 128), Np = (int)ceil_to_i64(a.N, 16);
  const int chunks = Kp / 128;
  const int stages_per_tile = (chunks + kCPS - 1) / kCPS;
  const int ntiles = Np / 16;
  const int ngroups = (ntiles + RT - 1) / RT;
  const bool has_x = g < M;
  T* y = reinterpret_cast<T*>(a.y);
  constexpr uint32_t kM = 0x0F0F0F0Fu;

  for (int grp = blockIdx.x; grp < ngroups; grp += gridDim.x, giter++) {
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
        const int slot = it % c.stages;
        if (!mbar_wait(&c.full_bar[slot], (it / c.stages) & 1, c.abort_flag)) {
          atomicCAS(err, 0, 22);
          return false;
        }
        const int c0 = sp * kCPS;
        const int nch = min(kCPS, chunks - c0);
        const uint8_t* st = c.ring + (size_t)slot * kStageBytes;
        const uint8_t* st_scales = st + kCPS * kCB;
        for (int ch = warp; ch < nch; ch += kCW) {
          const int cg = c0 + ch;
          const uint8_t* tp = st + ch * kCB;
          const uint4 qa = *reinterpret_cast<const uint4*>(tp + g * 64 + t * 16);
          const uint4 qb = *reinterpret_cast<const uint4*>(tp + (g + 8) * 64 + t * 16);
          const uint32_t s0 = *reinterpret_cast<const uint32_t*>(st_scales + ch * kSB + (0 * 16 + 2 * g) * 2);
          const uint32_t s1 = *reinterpret_cast<const uint32_t*>(st_scales + ch * kSB + (1 * 16 + 2 * g) * 2);
          uint4 h0 = make_uint4(0, 0, 0, 0), h1 = h0, l0 = h0, l1 = h0;
          if (has_x) {
            const int8_t* ph = c.xh + (size_t)g * c.xs_stride + cg * 128 + 16 * t;
            const int8_t* pl = c.xl + (size_t)g * c.xs_stride + cg * 128 + 16 * t;
            h0 = *reinterpret_cast<const uint4*>(ph);
            h1 = *reinterpret_cast<const uint4*>(ph + 64);
            l0 = *reinterpret_cast<const uint4*>(pl);
            l1 = *reinterpret_cast<const uint4*>(pl + 64);
          }
          const int4 sd0 = *reinterpret_cast<const int4*>(c.seeds + (2 * cg) * 8 + 2 * t);
          const int4 sd1 = *reinterpret_cast<const int4*>(c.seeds + (2 * cg + 1) * 8 + 2 * t);
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
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.empty_bar[slot]);
      }
    }
    {
      const float dxa = c.dxs[2 * t], dxb = c.dxs[2 * t + 1];
#pragma unroll
      for (int r = 0; r < RT; r++) {
        acc[r][0] *= dxa; acc[r][1] *= dxb; acc[r][2] *= dxa; acc[r][3] *= dxb;
      }
    }
    // ---- cross-warp reduction: shared float atomics + tickets; the last arriver finalises the tile group ----
    const int b = giter % kNB;
    {
      volatile int* genp = c.red_gen + b;
      bool ready = false;
      for (int i = 0; i < kSpin; i++) {
        if (*genp == giter / kNB) { ready = true; break; }
        __nanosleep(64);
        if ((i & 63) == 63 && *c.abort_flag) break;
      }
      if (!ready) {
        atomicCAS(err, 0, 23);
        *c.abort_flag = 1;
        return false;
      }
    }
    float* rbuf = c.red + (size_t)b * 2 * 128;
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
    if (lane == 0) ticket = atomicAdd(c.red_cnt + b, 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket == kCW - 1) {
      __threadfence_block();
      if (RT == 1) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int i = lane + 32 * j;  // [16 rows][8 cols]
          const int row = i / 8, col = i % 8;
          float sv = atomicExch(&rbuf[i], 0.f);
          const int n = grp * 16 + row;
          if (n < a.N && col < M) {
            if (a.bias != nullptr) sv += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[n]);
            if (a.residual != nullptr)
              sv += DT<T>::to_f(__ldcg(reinterpret_cast<const T*>(a.residual) + (size_t)col * a.ldr + n));
            y[(size_t)col * a.ldy + n] = DT<T>::from_f(sv);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int i = lane + 32 * j;
          const int row = i / 8, col = i % 8;
          float gsum = atomicExch(&rbuf[i], 0.f), usum = atomicExch(&rbuf[128 + i], 0.f);
          const int n = grp * 16 + row;
          if (n < a.N / 2 && col < M) {
            if (a.bias != nullptr) {
              gsum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)grp * 32 + row]);
              usum += DT<T>::to_f(reinterpret_cast<const T*>(a.bias)[(size_t)grp * 32 + 16 + row]);
            }
            y[(size_t)col * a.ldy + n] = DT<T>::from_f(act_apply(gsum, a.act) * usum);
          }
        }
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) {
        c.red_cnt[b] = 0;
        __threadfence_block();
        *(volatile int*)(c.red_gen + b) = giter / kNB + 1;
      }
    }
  }
  return true;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) gemv_chain_kernel(const __grid_constant__ ChainArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  Ctx c;
  c.stages = a.stages;
  c.xs_stride = a.kp_max + kPad;
  c.ring = smem_raw;
  size_t off = (size_t)a.stages * kStageBytes;
  c.full_bar = reinterpret_cast<uint64_t*>(smem_raw + off);
  c.empty_bar = c.full_bar + a.stages;
  off += (size_t)2 * a.stages * sizeof(uint64_t);
  off = (off + 15) & ~(size_t)15;
  c.xh = reinterpret_cast<int8_t*>(smem_raw + off);
  c.xl = c.xh + (size_t)a.M * c.xs_stride;
  off += (size_t)2 * a.M * c.xs_stride;
  off = (off + 15) & ~(size_t)15;
  c.red = reinterpret_cast<float*>(smem_raw + off);
  off += (size_t)kNB * 2 * 128 * sizeof(float);
  c.red_cnt = reinterpret_cast<int*>(smem_raw + off);
  c.red_gen = c.red_cnt + kNB;
  off += 2 * kNB * sizeof(int);
  c.scratch = reinterpret_cast<float*>(smem_raw + off);
  off += 2 * kCW * sizeof(float);
  c.dxs = reinterpret_cast<float*>(smem_raw + off);
  off += 8 * sizeof(float);
  c.seeds = reinterpret_cast<int2*>(smem_raw + off);
  off += (size_t)(a.kp_max / 64) * 8 * sizeof(int2);
  c.abort_flag = reinterpret_cast<volatile int*>(smem_raw + off);

  if (tid == 0) {
    for (int s = 0; s < a.stages; s++) {
      mbar_init(&c.full_bar[s], 1);
      mbar_init(&c.empty_bar[s], kCW);
    }
    *c.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kCW) {
    // ---------------- producer: weights of every op, never waits for another kernel or for the grid barrier ----
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int o = 0; o < a.nops && ok; o++) {
        const ChainOp& op = a.op[o];
        const int RT = op.act != 0 ? 2 : 1;
        const int Kp = (int)ceil_to_i64(op.K, 128), Np = (int)ceil_to_i64(op.N, 16);
        const int chunks = Kp / 128;
        const int stages_per_tile = (chunks + kCPS - 1) / kCPS;
        const int ntiles = Np / 16;
        const int ngroups = (ntiles + RT - 1) / RT;
        const uint8_t* codes = op.w;
        const uint8_t* scales = op.w + (size_t)Np * Kp / 2;
        for (int grp = blockIdx.x; grp < ngroups && ok; grp += gridDim.x) {
          for (int r = 0; r < RT && ok; r++) {
            const int tile = grp * RT + r;
            if (tile >= ntiles) break;
            for (int sp = 0; sp < stages_per_tile; sp++, it++) {
              const int slot = it % a.stages;
              if (it >= a.stages) {
                if (!mbar_wait(&c.empty_bar[slot], ((it / a.stages) - 1) & 1, c.abort_flag)) {
                  atomicCAS(a.err, 0, 21);
                  ok = false;
                  break;
                }
              }
              const int c0 = sp * kCPS;
              const int nch = min(kCPS, chunks - c0);
              uint8_t* dst = c.ring + (size_t)slot * kStageBytes;
              mbar_expect_tx(&c.full_bar[slot], (uint32_t)(nch * (kCB + kSB)));
              const size_t chunk_index = (size_t)tile * chunks + c0;
              bulk_g2s(dst, codes + chunk_index * kCB, (uint32_t)(nch * kCB), &c.full_bar[slot]);
              bulk_g2s(dst + kCPS * kCB, scales + chunk_index * kSB, (uint32_t)(nch * kSB), &c.full_bar[slot]);
            }
          }
        }
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  pdl_wait();
  for (int i = tid; i < kNB * 2 * 128; i += kCThreads) c.red[i] = 0.f;
  if (tid < 2 * kNB) c.red_cnt[tid] = 0;
  int it = 0, giter = 0;
  bool ok = true;
  for (int o = 0; o < a.nops && ok; o++) {
    const ChainOp& op = a.op[o];
    const int Kp = (int)ceil_to_i64(op.K, 128);
    consumer_sync();
    stage_x_i8<T>(op, a.M, c, Kp);
    consumer_sync();
    ok = op.act != 0 ? consume_op<T, 2>(op, a.M, c, it, giter, a.err) : consume_op<T, 1>(op, a.M, c, it, giter, a.err);
    if (o + 1 < a.nops) {
      // ---- grid barrier: every CTA's outputs of op o are complete and visible before op o+1 stages them ----
      consumer_sync();
      if (tid == 0) {
        __threadfence();
        atomicAdd(a.barrier, 1u);
        const unsigned int target = (unsigned int)(o + 1) * gridDim.x;
        bool arrived = false;
        for (int i = 0; i < kSpin; i++) {
          if (ld_acquire_gpu(a.barrier) >= target) { arrived = true; break; }
          __nanosleep(40);
          if ((i & 255) == 255 && *c.abort_flag) break;
        }
        if (!arrived) {
          atomicCAS(a.err, 0, 24);
          *c.abort_flag = 1;
        }
        __threadfence();
      }
      consumer_sync();
      if (*c.abort_flag) ok = false;
    }
  }
  // ---- leave the counters zero for the next launch: the last CTA out resets them ----
  consumer_sync();
  if (tid == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(a.barrier + 1, 1u);
    if (prev == gridDim.x - 1) {
      a.barrier[0] = 0u;
      a.barrier[1] = 0u;
      __threadfence();
    }
  }
}

size_t chain_smem(int M, int kp_max, int stages) {
  size_t off = (size_t)stages * kStageBytes + (size_t)2 * stages * 8;
  off = (off + 15) & ~(size_t)15;
  off += (size_t)2 * M * (kp_max + kPad);
  off = (off + 15) & ~(size_t)15;
  off += (size_t)kNB * 2 * 128 * 4 + 2 * kNB * 4 + 2 * kCW * 4 + 8 * 4 + (size_t)(kp_max / 64) * 8 * 8 + 16;
  return off;
}

}  // namespace

// Descriptor passed from the host: `nops` (1..4) GEMVs run in order, op i+1 may read what op i wrote.
// All weights are symmetric int4 in the device tile layout; K % 64 == 0; M <= 8 tokens (shared memory permitting).
// `barrier`: two zero-initialised unsigned ints owned by the caller (left zero by every completed launch).
struct IpexChainOpDesc {
  const void* w; const void* x; void* y; const void* norm_w; const void* bias; const void* residual;
  int N, K, ldx, ldy, ldr, act;
  float eps, norm_offset;
};

IPEX_API int ipex_gemv_chain_max_ops(void) { return kMaxOps; }

IPEX_API int ipex_gemv_chain(const IpexChainOpDesc* ops, int nops, int M, int dtype, unsigned int* barrier, int pdl,
                             int* err, void* stream) {
  if (nops < 1 || nops > kMaxOps || M < 1 || M > 8 || barrier == nullptr || err == nullptr)
    return (int)cudaErrorInvalidValue;
  ChainArgs a;
  int kp_max = 0;
  for (int i = 0; i < nops; i++) {
    const IpexChainOpDesc& d = ops[i];
    if ((d.K % 64) != 0 || (d.ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(d.x) & 15) != 0 || d.N < 1)
      return (int)cudaErrorInvalidValue;
    if (d.act != 0 && (d.residual != nullptr || (d.N % 32) != 0)) return (int)cudaErrorInvalidValue;
    ChainOp& o = a.op[i];
    o.w = reinterpret_cast<const uint8_t*>(d.w); o.x = d.x; o.y = d.y; o.norm_w = d.norm_w; o.bias = d.bias;
    o.residual = d.residual; o.N = d.N; o.K = d.K; o.ldx = d.ldx; o.ldy = d.ldy; o.ldr = d.ldr; o.act = d.act;
    o.eps = d.eps; o.norm_offset = d.norm_offset;
    const int kp = (int)ceil_to_i64(d.K, 128);
    if (kp > kp_max) kp_max = kp;
  }
  a.nops = nops; a.M = M; a.kp_max = kp_max; a.barrier = barrier; a.err = err;
  int stages = 12;
  while (stages > 2 && chain_smem(M, kp_max, stages) > 200 * 1024) stages--;
  if (chain_smem(M, kp_max, stages) > 227 * 1024) return (int)cudaErrorInvalidValue;
  a.stages = stages;
  const size_t smem = chain_smem(M, kp_max, stages);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) {
    auto kern = gemv_chain_kernel<__half>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_kernel(kern, dim3(sms), dim3(kThreads), smem, s, pdl != 0, a);
  }
  if (dtype == DT_BF16) {
    auto kern = gemv_chain_kernel<__nv_bfloat16>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_kernel(kern, dim3(sms), dim3(kThreads), smem, s, pdl != 0, a);
  }
  return (int)cudaErrorInvalidValue;
}
