// Prefill GEMM on the 5th-generation tensor cores:  out[M, N] = x[M, K] . w[N, K]^T  (+ bias, + residual).
//
// The weight rows sit on the MMA's M side (128 rows per tile) and the tokens on its N side (32..256 per tile), so a
// short prompt still fills the instruction: D[TMEM lane = weight row][TMEM column = token].  Both operands are
// K-major in shared memory in the 128-byte swizzle that TMA writes and tcgen05.mma reads directly.
//
// One persistent CTA per SM, three roles:
//   warp 0      one lane issues the TMA loads of both operands into a ring of stages (full/empty mbarriers);
//   warp 1      allocates TMEM, one lane issues tcgen05.mma (4 per 64-wide k block) and commits: a commit releases
//               the stage to the loader, the last commit of a tile hands the accumulator to the epilogue;
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp owns one 32-lane quarter), add bias / residual,
//               convert and store.  Two accumulators alternate in TMEM, so the epilogue of tile i overlaps the
//               main loop of tile i+1.
// Every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, records a code in the global
// error flag, and every role leaves its loop; TMEM is released on all paths.
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
constexpr int kThreads = 192;

struct GemmArgs {
  void* out;
  const void* bias;      // [N] or null
  const void* residual;  // [M, ldr] or null
  int64_t ldo, ldr;
  int M, N, K;
  int m_tiles, n_tiles;
  int* err;
};

template <int BT>
struct Cfg {
  static constexpr int kStages = BT >= 256 ? 4 : (BT >= 128 ? 6 : 8);
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BT * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BT < 32 ? 32 : 2 * BT;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <typename T, int BT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, GemmArgs a) {
  using C = Cfg<BT>;
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = a.m_tiles * a.n_tiles;
  const int kblocks = (a.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- loader ----------------
    if (lane == 0) {
      prefetch_tmap(&tm_w);
      prefetch_tmap(&tm_x);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
        const int nb = t / a.m_tiles, mb = t % a.m_tiles;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) { ok = false; report(a.err, 8); break; }
          mbar_expect_tx(&full[s], C::kStageBytes);
          tma_load_2d(sA + s * C::kABytes, &tm_w, kb * kBK, nb * kBM, &full[s]);
          tma_load_2d(sB + s * C::kBBytes, &tm_x, kb * kBK, mb * BT, &full[s]);
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
  } else {
    // ---------------- epilogue ----------------
    const int qd = warp & 3;  // TMEM lane quarter this warp may read
    T* out = reinterpret_cast<T*>(a.out);
    const T* res = reinterpret_cast<const T*>(a.residual);
    const T* bias = reinterpret_cast<const T*>(a.bias);
    int it = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
      const int nb = t / a.m_tiles, mb = t % a.m_tiles;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) report(a.err, 10);
        break;
      }
      tcgen05_fence_after();
      const int n = nb * kBM + qd * 32 + lane;
      const float bv = (bias != nullptr && n < a.N) ? to_float(bias[n]) : 0.f;
#pragma unroll 1
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (uint32_t(qd * 32) << 16) + acc * BT + c * 32, v);
        const int m0 = mb * BT + c * 32;
        if (n < a.N) {
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
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <typename T, int BT>
cudaError_t launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int sms, cudaStream_t st) {
  using C = Cfg<BT>;
  auto kern = gemm_tn_kernel<T, BT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int ntiles = a.m_tiles * a.n_tiles;
  const int grid = ntiles < sms ? ntiles : sms;
  kern<<<grid, kThreads, C::kSmemBytes, st>>>(tw, tx, a);
  return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch_bt(int bt, const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int sms,
                        cudaStream_t st) {
  switch (bt) {
    case 32: return launch_gemm<T, 32>(tw, tx, a, sms, st);
    case 64: return launch_gemm<T, 64>(tw, tx, a, sms, st);
    case 128: return launch_gemm<T, 128>(tw, tx, a, sms, st);
    default: return launch_gemm<T, 256>(tw, tx, a, sms, st);
  }
}

}  // namespace

// Token tile the kernel will use for M tokens.
IPEX_API int ipex_gemm_tcgen05_token_tile(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)); }

// out[M,N] = x[M,K] . w[N,K]^T (+ bias[N]) (+ residual[M,N]).  x, w, out, bias, residual share one 16-bit dtype.
// Row strides (elements): ldx, ldw multiples of 8 (TMA wants 16-byte strides); x and w 16-byte aligned.
// Returns a cudaError_t, or -1 when the driver's tensor-map encoder is unavailable / rejects the arguments.
IPEX_API int ipex_gemm_tcgen05(const void* x, const void* w, void* out, const void* bias, const void* residual, int M,
                               int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int64_t ldr, int dtype, int* err,
                               void* stream) {
  if (M < 1 || N < 1 || K < 1 || (ldx % 8) != 0 || (ldw % 8) != 0) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return (int)cudaErrorInvalidValue;
  if (dtype != DT_F16 && dtype != DT_BF16) return (int)cudaErrorInvalidValue;
  const int bt = ipex_gemm_tcgen05_token_tile(M);
  const CUtensorMapDataType tdt = dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tw, tx;
  if (!tc5::encode_2d_sw128(&tw, tdt, w, (uint64_t)K, (uint64_t)N, (uint64_t)ldw * 2, kBK, kBM)) return -1;
  if (!tc5::encode_2d_sw128(&tx, tdt, x, (uint64_t)K, (uint64_t)M, (uint64_t)ldx * 2, kBK, bt)) return -1;
  GemmArgs a;
  a.out = out; a.bias = bias; a.residual = residual; a.ldo = ldo; a.ldr = ldr;
  a.M = M; a.N = N; a.K = K;
  a.m_tiles = (M + bt - 1) / bt;
  a.n_tiles = (N + kBM - 1) / kBM;
  a.err = err;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaStream_t st = (cudaStream_t)stream;
  return (int)(dtype == DT_F16 ? dispatch_bt<__half>(bt, tw, tx, a, sms, st)
                               : dispatch_bt<__nv_bfloat16>(bt, tw, tx, a, sms, st));
}
