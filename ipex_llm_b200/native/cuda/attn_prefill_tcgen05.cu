// Prompt-pass (Sq == Skv) flash attention on the 5th-generation tensor cores, sm_100a.
//
// Stand-in for the reference's closed `xe_addons.sdp_causal` / `sdp_non_causal`
// (python/llm/src/ipex_llm/transformers/models/common.py:270-285).  Both GEMMs of attention run as tcgen05.mma with
// their accumulators in tensor memory:
//
//   S  = Q K^T   A = Q tile [128 queries x D]        B = K tile  [128 keys x D]     -> TMEM columns [0, 128)
//   PV = P V     A = P tile [128 queries x 128 keys] B = V^T tile [D x 128 keys]    -> TMEM columns [128, 128 + D)
//
// Every operand is K-major in the 128-byte swizzle: Q and K tiles come straight from the fused qkv activation
// through TMA, V is read from a transposed copy ([B, Hkv, D, S]) so that its tile is K-major too, and P is written
// by the softmax threads in the same swizzle.  One CTA owns 128 queries of one head and walks the key blocks:
//
//   warp 8 (one lane): TMA loads, K / V^T double buffered
//   warp 9 (one lane): issues the MMAs, S(j+1) is issued before the softmax threads have folded PV(j) into O
//   warps 0-7        : two threads per query row (warps w and w + 4 read the same TMEM lanes), each owning 64 of
//                      the block's 128 score columns and half of the output columns: row max (exchanged through
//                      shared memory), exp2, row sum, P to shared memory, running output O[D/2] in registers
//                      rescaled by exp2(m_old - m_new) per block
//
// No cluster multicast.  Every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, the
// error word gets a code (31 loader, 32 MMA issuer, 33 softmax) and all roles leave, after which TMEM is freed.
#include "common/utils.cuh"
#include "tcgen05_common.cuh"

namespace {

using namespace tc5;

constexpr int kBQ = 128;   // queries per CTA (MMA M)
constexpr int kBKV = 128;  // keys per block
constexpr int kThreads = 320;  // 8 softmax warps, loader warp, MMA warp

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct PrefillArgs {
  void* out;          // [B, S, Hq, D] with row stride ldo (elements) between tokens
  int* err;
  int64_t ldo;
  int B, S, Hq, Hkv;
  int causal;
  float scale_log2;   // softmax scale * log2(e)
  // optional: tanh soft-cap of the scaled scores (Gemma-2), sliding window (a query sees the `window` newest keys up
  // to itself), and left padding (batch b's keys and queries below kv_lo[b] do not exist)
  float cap_log2;          // softcap * log2(e), 0 = off
  float scale_over_cap;    // softmax scale / softcap
  int window;              // 0 = off
  const int* kv_lo;        // [B] or null
};

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T, int D, bool EXT /* soft-cap / window / left padding compiled in */>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_vt, PrefillArgs a) {
  constexpr int kDB = D / 64;                       // 64-element k-blocks along the head dim
  constexpr int kQBytes = kBQ * D * 2;
  constexpr int kKBytes = kBKV * D * 2;
  constexpr int kVBytes = D * kBKV * 2;
  constexpr int kPBytes = kBQ * kBKV * 2;
  constexpr int kStageBytes = kKBytes + kVBytes;
  constexpr uint32_t kTmemCols = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + kQBytes;
  uint8_t* sKV = sP + kPBytes;                      // 2 stages of [K tile | V^T tile]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + 2 * kStageBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                     // [2]
  uint64_t* kv_empty = bars + 3;                    // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint64_t* o_free = bars + 8;
  uint64_t* x_full = bars + 9;                      // row-maximum exchange inside a thread pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(bars + 32);  // [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (a.S + kBQ - 1) / kBQ;
  // Blocks are dispatched x-fastest: heads run along x and query blocks, longest first, along y, so every head's
  // longest rows start before any shorter ones (longest-processing-time-first over the SMs).
  const int qb = nqb - 1 - (int)blockIdx.y;
  const int h = blockIdx.x, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int nkv = a.causal ? qb + 1 : (a.S + kBKV - 1) / kBKV;
  // first key block any query of this block can see (sliding window, left padding); all roles walk [j0, nkv)
  const int klo_b = EXT && a.kv_lo != nullptr ? a.kv_lo[b] : 0;
  int j0 = klo_b / kBKV;
  if (EXT && a.window > 0) j0 = max(j0, (qb * kBQ - a.window + 1) / kBKV);
  j0 = EXT ? max(0, min(j0, nkv)) : 0;
  const int nblk = nkv - j0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 256);
    mbar_init(o_full, 1);
    mbar_init(o_free, 256);
    mbar_init(x_full, 256);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---------------- loader ----------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_vt);
      const int row0 = b * a.S + qb * kBQ;          // token row of the first query
      mbar_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int kb = 0; kb < kDB; ++kb) tma_load_2d(sQ + kb * (kBQ * 128), &tm_q, h * D + kb * 64, row0, q_full);
      bool ok = true;
      for (int jj = 0; jj < nblk && ok; ++jj) {
        const int j = j0 + jj;
        const int st = jj & 1;
        const uint32_t ph = (jj >> 1) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag)) { ok = false; report(a.err, 31); break; }
        uint8_t* sK = sKV + st * kStageBytes;
        uint8_t* sV = sK + kKBytes;
        mbar_expect_tx(&kv_full[st], kStageBytes);
#pragma unroll
        for (int kb = 0; kb < kDB; ++kb)
          tma_load_2d(sK + kb * (kBKV * 128), &tm_k, kvh * D + kb * 64, b * a.S + j * kBKV, &kv_full[st]);
#pragma unroll
        for (int kb = 0; kb < kBKV / 64; ++kb)
          tma_load_2d(sV + kb * (D * 128), &tm_vt, j * kBKV + kb * 64, (b * a.Hkv + kvh) * D, &kv_full[st]);
      }
      if (!ok) {
        mbar_wait_quiet(q_full, 0, 1 << 12);
        for (int i = 0; i < 2; ++i) mbar_wait_quiet(&kv_full[i], 0, 1 << 12);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16<T>(kBQ, kBKV);
      const uint32_t idesc_o = make_idesc_f16<T>(kBQ, D);
      const uint32_t tm_s = tmem_base, tm_o = tmem_base + kBKV;
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (!ok) report(a.err, 32);
      for (int jj = 0; jj < nblk && ok; ++jj) {
        const int st = jj & 1;
        const uint32_t ph = (jj >> 1) & 1, jp = jj & 1;
        uint8_t* sK = sKV + st * kStageBytes;
        uint8_t* sV = sK + kKBytes;
        if (!mbar_wait(&kv_full[st], ph, abort_flag)) { ok = false; report(a.err, 32); break; }
        tcgen05_fence_after();
        // S = Q K^T (the softmax threads released S(j-1) before they signalled p_full(j-1), waited on below)
#pragma unroll
        for (int kb = 0; kb < kDB; ++kb) {
          const uint64_t adesc = make_desc_sw128(smem_u32(sQ + kb * (kBQ * 128)));
          const uint64_t bdesc = make_desc_sw128(smem_u32(sK + kb * (kBKV * 128)));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f16(tm_s, adesc + 2 * kk, bdesc + 2 * kk, idesc_s, (kb | kk) != 0);
        }
        umma_commit(s_full);
        // PV = P V: needs P(j) in shared memory and the previous PV read out of TMEM
        if (!mbar_wait(p_full, jp, abort_flag)) { ok = false; report(a.err, 32); break; }
        if (jj > 0 && !mbar_wait(o_free, jp ^ 1, abort_flag)) { ok = false; report(a.err, 32); break; }
        tcgen05_fence_after();
#pragma unroll
        for (int kb = 0; kb < kBKV / 64; ++kb) {
          const uint64_t adesc = make_desc_sw128(smem_u32(sP + kb * (kBQ * 128)));
          const uint64_t bdesc = make_desc_sw128(smem_u32(sV + kb * (D * 128)));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_f16(tm_o, adesc + 2 * kk, bdesc + 2 * kk, idesc_o, (kb | kk) != 0);
        }
        umma_commit(o_full);
        umma_commit(&kv_empty[st]);
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax + output: two threads per query row, each owns half of the columns ----------------
    const int r = threadIdx.x & 127, hf = threadIdx.x >> 7;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int qpos = qb * kBQ + r;
    constexpr int kOH = D / 2;                        // output columns of this thread: [hf * kOH, (hf + 1) * kOH)
    float o[kOH];
#pragma unroll
    for (int d = 0; d < kOH; ++d) o[d] = 0.f;
    float m = -INFINITY, l = 0.f;                     // m: row maximum (shared by the pair), l: this thread's part
    bool ok = true;
    // score -> exponent (base 2): plain scale, or the tanh soft-cap of the scaled score (monotonic, so the row
    // maximum can be taken on the raw scores and transformed once)
    const bool capped = EXT && a.cap_log2 > 0.f;
    auto expo = [&](float sv) {
      return capped ? a.cap_log2 * tanh_approx(sv * a.scale_over_cap) : sv * a.scale_log2;
    };
    for (int jj = 0; jj < nblk; ++jj) {
      const int j = j0 + jj;
      const uint32_t jp = jj & 1;
      if (!mbar_wait(s_full, jp, abort_flag)) { ok = false; if (lane == 0) report(a.err, 33); break; }
      tcgen05_fence_after();
      const int k0 = j * kBKV;
      // keys this row may see in the block: [k0 + klow, k0 + klim); this thread looks at block columns
      // [hf*64, hf*64+64), of which the local columns in [lo, lim) are visible
      int klim = a.S - k0;
      if (a.causal) klim = min(klim, qpos - k0 + 1);
      int klow = klo_b - k0;
      if (EXT && a.window > 0) klow = max(klow, qpos - a.window + 1 - k0);
      if (EXT && qpos < klo_b) klim = 0;              // a padding row sees nothing (its output is zero)
      const int lim = min(klim, kBKV) - hf * 64;
      const int lo = EXT ? klow - hf * 64 : 0;
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(tmem_base + lane_addr + hf * 64, v0);
      tmem_ld_32x32(tmem_base + lane_addr + hf * 64 + 32, v1);
      float mx = -INFINITY;
      const bool full = lim >= 64 && (!EXT || lo <= 0);
      if (full) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < lim && (!EXT || i >= lo)) mx = fmaxf(mx, __uint_as_float(v0[i]));
          if (32 + i < lim && (!EXT || 32 + i >= lo)) mx = fmaxf(mx, __uint_as_float(v1[i]));
        }
      }
      mx = mx == -INFINITY ? mx : expo(mx);           // the transform is increasing: max commutes with it
      xch[hf * 128 + r] = mx;
      mbar_arrive(x_full);
      if (!mbar_wait(x_full, jp, abort_flag)) { ok = false; if (lane == 0) report(a.err, 33); break; }
      mx = fmaxf(fmaxf(mx, xch[(hf ^ 1) * 128 + r]), m);
      // a row that sees nothing yet keeps m = -inf; use 0 as the reference so that exp2 stays finite
      const float mref = mx == -INFINITY ? 0.f : mx;
      const float corr = ex2(m - mref);               // m = -inf -> 0
      float psum = 0.f;
      uint8_t* prow = sP + hf * (kBQ * 128) + r * 128;  // P k-block `hf` holds block columns [hf*64, hf*64+64)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        __align__(16) T pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float sv = __uint_as_float(half == 0 ? v0[i] : v1[i]);
          float p = ex2(expo(sv) - mref);
          if (!full && (half * 32 + i >= lim || (EXT && half * 32 + i < lo))) p = 0.f;
          const T pt = from_float<T>(p);
          pk[i] = pt;
          psum += to_float<T>(pt);                   // the sum the tensor cores will see
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = half * 4 + q;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = reinterpret_cast<const uint4*>(pk)[q];
        }
      }
      l = l * corr + psum;
      m = mx;
      fence_proxy_async_smem();
      tcgen05_fence_before();
      mbar_arrive(p_full);
      // fold this thread's half of PV(j) into the running output
      if (!mbar_wait(o_full, jp, abort_flag)) { ok = false; if (lane == 0) report(a.err, 33); break; }
      tcgen05_fence_after();
#pragma unroll
      for (int c = 0; c < kOH / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_addr + kBKV + hf * kOH + c * 32, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], corr, __uint_as_float(v[i]));
      }
      tcgen05_fence_before();
      mbar_arrive(o_free);
    }
    if (ok) {
      // the pair's row sum: one more exchange through the same slots
      xch[hf * 128 + r] = l;
      mbar_arrive(x_full);
      ok = mbar_wait(x_full, nblk & 1, abort_flag);
      if (!ok && lane == 0) report(a.err, 33);
      l += xch[(hf ^ 1) * 128 + r];
    }
    if (ok && qpos < a.S) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* op = reinterpret_cast<T*>(a.out) + ((int64_t)b * a.S + qpos) * a.ldo + (int64_t)h * D + hf * kOH;
#pragma unroll
      for (int c = 0; c < kOH / 8; ++c) {
        __align__(16) T ov[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) ov[i] = from_float<T>(o[c * 8 + i] * inv);
        *reinterpret_cast<uint4*>(op + c * 8) = *reinterpret_cast<const uint4*>(ov);
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, kTmemCols);
}

// V (token-major, element (b, s, h, d) at v[(b*S + s) * ldv + h*D + d]) -> V^T [B, Hkv, D, s_pad], zeros for
// s in [S, s_pad).  64 x 64 tiles through shared memory: 128-byte contiguous reads along d and writes along s.
template <typename T>
__global__ void __launch_bounds__(256) transpose_v_kernel(const T* __restrict__ v, T* __restrict__ vt, int S, int Hkv,
                                                          int D, int64_t ldv, int64_t s_pad) {
  __shared__ T tile[64][66];
  const int s0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  const int bh = blockIdx.z, b = bh / Hkv, h = bh % Hkv;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int sl = ty + 4 * i, s = s0 + sl;
    T val = DT<T>::from_f(0.f);
    if (s < S) val = v[((int64_t)b * S + s) * ldv + (int64_t)h * D + d0 + tx];
    tile[sl][tx] = val;
  }
  __syncthreads();
  if (s0 + tx < s_pad) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int dl = ty + 4 * i;
      vt[((int64_t)bh * D + d0 + dl) * s_pad + s0 + tx] = tile[tx][dl];
    }
  }
}

template <typename T, int D>
int launch(const void* q, const void* k, const void* vt, void* out, int B, int S, int Hq, int Hkv, int64_t ldq,
           int64_t ldk, int64_t s_pad, int64_t ldo, float scale, int causal, float softcap, int window,
           const int* kv_lo, int* err, cudaStream_t stream) {
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_q, tm_k, tm_vt;
  if (!encode_2d_sw128(&tm_q, dt, q, (uint64_t)Hq * D, (uint64_t)B * S, (uint64_t)ldq * 2, 64, kBQ) ||
      !encode_2d_sw128(&tm_k, dt, k, (uint64_t)Hkv * D, (uint64_t)B * S, (uint64_t)ldk * 2, 64, kBKV) ||
      !encode_2d_sw128(&tm_vt, dt, vt, (uint64_t)s_pad, (uint64_t)B * Hkv * D, (uint64_t)s_pad * 2, 64, D))
    return (int)cudaErrorInvalidValue;
  PrefillArgs a;
  a.out = out; a.err = err; a.ldo = ldo; a.B = B; a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.cap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  a.scale_over_cap = softcap > 0.f ? scale / softcap : 0.f;
  a.window = window > 0 ? window : 0;
  a.kv_lo = kv_lo;
  const size_t smem = 1024 + (size_t)kBQ * D * 2 + (size_t)kBQ * kBKV * 2 + 2 * ((size_t)kBKV * D * 2 * 2) + 256 + 1024;
  const bool ext = a.cap_log2 > 0.f || a.window > 0 || a.kv_lo != nullptr;
  auto kern = ext ? attn_prefill_kernel<T, D, true> : attn_prefill_kernel<T, D, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(Hq, (S + kBQ - 1) / kBQ, B);
  kern<<<grid, kThreads, smem, stream>>>(tm_q, tm_k, tm_vt, a);
  return (int)cudaGetLastError();
}

}  // namespace

// q: token-major activation, element (b, s, h, d) at q[((b*S + s) * ldq) + h*D + d] (already rotated); k likewise
// with Hkv heads and row stride ldk; vt: V transposed, [B, Hkv, D, s_pad] contiguous with zeros past S (s_pad a
// multiple of 8, >= S); out: [B, S, Hq, D] with token stride ldo.  D is 64 or 128, Hq a multiple of Hkv.  All base
// pointers 16-byte aligned, ldq / ldk / ldo multiples of 8.  `err` receives a code when a bounded wait runs out.
// softcap > 0: scores become softcap * tanh(score * scale / softcap); window > 0: a query sees only the `window`
// newest keys up to itself; kv_lo (device, [B], may be null): keys and queries of batch b below kv_lo[b] are padding
// (padding queries produce zeros).  Returns a cudaError_t.
IPEX_API int ipex_attn_prefill_tcgen05_ex(const void* q, const void* k, const void* vt, void* out, int B, int S, int Hq,
                                          int Hkv, int D, int64_t ldq, int64_t ldk, int64_t s_pad, int64_t ldo,
                                          float scale, int causal, float softcap, int window, const int* kv_lo,
                                          int dtype, int* err, void* stream) {
  if (B < 1 || S < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0 || B > 65535 || Hq > 65535) return (int)cudaErrorInvalidValue;
  if ((ldq % 8) != 0 || (ldk % 8) != 0 || (ldo % 8) != 0 || (s_pad % 8) != 0 || s_pad < S)
    return (int)cudaErrorInvalidValue;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)vt | (uintptr_t)out) & 15) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) {
    if (D == 128)
      return launch<__half, 128>(q, k, vt, out, B, S, Hq, Hkv, ldq, ldk, s_pad, ldo, scale, causal, softcap, window,
                                 kv_lo, err, s);
    if (D == 64)
      return launch<__half, 64>(q, k, vt, out, B, S, Hq, Hkv, ldq, ldk, s_pad, ldo, scale, causal, softcap, window,
                                kv_lo, err, s);
  } else if (dtype == DT_BF16) {
    if (D == 128)
      return launch<__nv_bfloat16, 128>(q, k, vt, out, B, S, Hq, Hkv, ldq, ldk, s_pad, ldo, scale, causal, softcap,
                                        window, kv_lo, err, s);
    if (D == 64)
      return launch<__nv_bfloat16, 64>(q, k, vt, out, B, S, Hq, Hkv, ldq, ldk, s_pad, ldo, scale, causal, softcap,
                                       window, kv_lo, err, s);
  }
  return (int)cudaErrorInvalidValue;
}

// Plain form: no soft-cap, no window, no padding.
IPEX_API int ipex_attn_prefill_tcgen05(const void* q, const void* k, const void* vt, void* out, int B, int S, int Hq,
                                       int Hkv, int D, int64_t ldq, int64_t ldk, int64_t s_pad, int64_t ldo,
                                       float scale, int causal, int dtype, int* err, void* stream) {
  return ipex_attn_prefill_tcgen05_ex(q, k, vt, out, B, S, Hq, Hkv, D, ldq, ldk, s_pad, ldo, scale, causal, 0.f, 0,
                                      nullptr, dtype, err, stream);
}

// The transposed V the kernel above reads: v is token-major (row stride ldv elements), vt [B, Hkv, D, s_pad] gets
// zeros past S.  D a multiple of 64, 16-bit dtype.
IPEX_API int ipex_attn_transpose_v(const void* v, void* vt, int B, int S, int Hkv, int D, int64_t ldv, int64_t s_pad,
                                   int dtype, void* stream) {
  if (B < 1 || S < 1 || Hkv < 1 || (D % 64) != 0 || s_pad < S || (int64_t)B * Hkv > 65535)
    return (int)cudaErrorInvalidValue;
  dim3 grid((unsigned)((s_pad + 63) / 64), D / 64, B * Hkv);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16)
    transpose_v_kernel<__half><<<grid, 256, 0, s>>>((const __half*)v, (__half*)vt, S, Hkv, D, ldv, s_pad);
  else if (dtype == DT_BF16)
    transpose_v_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)v, (__nv_bfloat16*)vt, S, Hkv, D, ldv,
                                                          s_pad);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}
