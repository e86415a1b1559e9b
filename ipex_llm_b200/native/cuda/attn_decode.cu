// Split-KV decode attention with fused RoPE + KV-cache append (+ fp8 e5m2 quantization), sm_100a.
//
// One launch does what the reference does with four closed kernels per layer: `rotary_half_inplaced`,
// `quantize_key_value` (cache append), and `sdp` / `sdp_fp8` (python/llm/src/ipex_llm/transformers/models/
// llama.py:158-194, models/utils.py:133-146, models/common.py:276-280).  It serves every "short query against a
// long cache" case: plain decode (Sq = 1), self-speculative verification and prompt-lookup (Sq <= 32).
//
// Grid (x = split * row_block, y = kv head, z = batch).  A CTA owns one KV range of one kv head for up to 16
// (query position, q head) rows of that head's GQA group.  Inside a warp, 8 lanes share a token (each owns D/8
// dims) so a 16-byte load per lane covers a full 128-dim fp8 row; 4 token slots per warp step.  Warps are split
// between row groups and token sub-ranges.  Partial (m, l, acc) per split go to a scratch buffer; the CTA that
// draws the last ticket of its (batch, kv head, row block) merges them and resets the ticket, so the whole op
// is one kernel and the scratch needs no clearing between calls.
//
// mode A (engine): new K/V rows come from the qkv GEMV output, are rotated, written to the cache by row block 0
//                  of the last split, and attended to from shared memory (causal among themselves).
// mode B (module path): the cache already holds every token; q is already rotated.
#include <cstdlib>

#include "common/utils.cuh"

namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kMaxRows = 16;

struct AttnArgs {
  const void* q;      // [B, Sq, Hq, D] via strides (elements)
  const void* knew;   // [B, Sq, Hkv, D] via strides, or null (mode B)
  const void* vnew;
  void* kcache;       // [B, Hkv, Smax, D]
  void* vcache;
  void* out;          // [B, Sq, Hq, D] via strides
  const int* past_len;  // [B] device, or null -> past_scalar
  const float* cosp;  // [max_pos, R/2] fp32 rotary table (mode A with rope != 0)
  const float* sinp;
  float* scratch;
  int* counters;
  int64_t q_b, q_s, q_h, kn_b, kn_s, kn_h, c_b, c_h, c_s, o_b, o_s, o_h;
  int past_scalar;
  int B, Sq, Hq, Hkv, nsplit, nrb;
  int rope;        // 0 none, 1 half (NeoX), 2 interleaved (GPT-J)
  int R;           // rotary dims
  int causal;      // mode B: 1 causal (query i sees kv_len - Sq + i), 0 full
  int window;      // sliding window (0 = off)
  float scale;     // softmax scale
  float softcap;   // 0 = off
};

__device__ __forceinline__ uint8_t to_e5m2(float v) {
  v = fminf(fmaxf(v, -57344.f), 57344.f);
  uint16_t h = __half_as_ushort(__float2half_rn(v));
  uint32_t r = (uint32_t)h + 0x7F + ((h >> 8) & 1);
  uint8_t o = (uint8_t)(r >> 8);
  if ((o & 0x7F) > 0x7B) o = (o & 0x80) | 0x7B;
  return o;
}
__device__ __forceinline__ float from_e5m2(uint8_t b) { return __half2float(__ushort_as_half((uint16_t)b << 8)); }

// DPL consecutive cache elements of one token held as raw 32-bit words (loaded early, decoded late)
template <typename T, bool FP8, int DPL>
struct RawKV {
  static constexpr int kBytes = FP8 ? DPL : DPL * 2;
  static constexpr int kWords = kBytes / 4;
  static_assert(kBytes % 8 == 0, "unsupported head dim");
  uint32_t w[kWords];

  __device__ __forceinline__ void load(const void* base, int64_t elem_off) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(base) + elem_off * (FP8 ? 1 : 2);
    if constexpr (kBytes % 16 == 0) {
#pragma unroll
      for (int i = 0; i < kBytes / 16; i++) {
        const uint4 v = *reinterpret_cast<const uint4*>(p + 16 * i);
        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < kBytes / 8; i++) {
        const uint2 v = *reinterpret_cast<const uint2*>(p + 8 * i);
        w[2 * i] = v.x; w[2 * i + 1] = v.y;
      }
    }
  }

  __device__ __forceinline__ void decode(float (&out)[DPL]) const {
    if constexpr (FP8) {
#pragma unroll
      for (int j = 0; j < kWords; j++) {
        // e5m2 byte -> fp16 by moving it to the upper byte of a 16-bit lane
        uint32_t lo = __byte_perm(w[j], 0, 0x1404), hi = __byte_perm(w[j], 0, 0x3424);
        const float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
        const float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
        out[4 * j + 0] = a.x; out[4 * j + 1] = a.y; out[4 * j + 2] = b.x; out[4 * j + 3] = b.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < kWords; j++) {
        const T* e = reinterpret_cast<const T*>(&w[j]);
        out[2 * j] = DT<T>::to_f(e[0]);
        out[2 * j + 1] = DT<T>::to_f(e[1]);
      }
    }
  }
};

template <typename T, bool FP8, int D, int RW>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnArgs a) {
  constexpr int DPL = D / 8;
  extern __shared__ __align__(16) float sm[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tg = lane >> 3, ds = lane & 7;
  const int split = blockIdx.x / a.nrb, rb = blockIdx.x % a.nrb;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int rows_total = G * a.Sq;
  const int row0 = rb * kMaxRows;
  const int rows_blk = min(kMaxRows, rows_total - row0);
  const bool modeA = a.knew != nullptr;

  pdl_launch_dependents();
  pdl_wait();

  const int past = a.past_len != nullptr ? a.past_len[b] : a.past_scalar;   // tokens held by the cache
  const int n_new = modeA ? a.Sq : 0;
  const int causal_base = modeA ? past : (a.causal ? past - a.Sq : past);
  const bool causal = modeA || a.causal;

  // shared memory carve-up
  float* knew_s = sm;                                   // [Sq][D]  (mode A, last split)
  float* vnew_s = knew_s + (modeA ? a.Sq * D : 0);
  float* part_acc = vnew_s + (modeA ? a.Sq * D : 0);    // [kAttnWarps][RW][D]
  float* part_ml = part_acc + kAttnWarps * RW * D;      // [kAttnWarps][RW][2]
  __shared__ int s_last;

  // ---- row-group / token-sub-range assignment of this warp ----
  const int row_groups = (rows_blk + RW - 1) / RW;
  const int rg_p2 = row_groups <= 1 ? 1 : (row_groups <= 2 ? 2 : 4);
  const int TS = kAttnWarps / rg_p2;
  const int rg = warp % rg_p2, tsub = warp / rg_p2;

  // ---- q rows of this warp, rotated, pre-scaled, in registers ----
  float qr[RW][DPL];
  int qpos[RW];     // query position index i of each row (for the causal limit), -1 = inactive row
#pragma unroll
  for (int r = 0; r < RW; r++) {
    const int row = row0 + rg * RW + r;
    qpos[r] = -1;
#pragma unroll
    for (int d = 0; d < DPL; d++) qr[r][d] = 0.f;
    if (rg * RW + r < rows_blk) {
      const int i = row / G, gq = row % G;
      qpos[r] = i;
      const T* qp = reinterpret_cast<const T*>(a.q) + b * a.q_b + (int64_t)i * a.q_s + (int64_t)(kvh * G + gq) * a.q_h;
      const int pos = past + i;
#pragma unroll
      for (int d = 0; d < DPL; d++) {
        const int e = ds * DPL + d;
        float v = DT<T>::to_f(qp[e]);
        if (modeA && a.rope != 0 && e < a.R) {
          const int half = a.R / 2;
          if (a.rope == 1) {
            const int j = e < half ? e : e - half;
            const float c = a.cosp[(int64_t)pos * half + j], s = a.sinp[(int64_t)pos * half + j];
            const float o = DT<T>::to_f(qp[e < half ? e + half : e - half]);
            v = e < half ? v * c - o * s : v * c + o * s;
          } else {
            const int j = e >> 1;
            const float c = a.cosp[(int64_t)pos * half + j], s = a.sinp[(int64_t)pos * half + j];
            const float o = DT<T>::to_f(qp[e ^ 1]);
            v = (e & 1) ? v * c + o * s : v * c - o * s;
          }
          v = DT<T>::to_f(DT<T>::from_f(v));
        }
        qr[r][d] = v * a.scale;
      }
    }
  }

  // ---- mode A, last split: rotate + stage the new K/V rows (through the cache's precision) ----
  const bool last_split = split == a.nsplit - 1;
  if (modeA && last_split) {
    for (int idx = tid; idx < a.Sq * D; idx += kAttnThreads) {
      const int i = idx / D, e = idx % D;
      const T* kp = reinterpret_cast<const T*>(a.knew) + b * a.kn_b + (int64_t)i * a.kn_s + (int64_t)kvh * a.kn_h;
      const T* vp = reinterpret_cast<const T*>(a.vnew) + b * a.kn_b + (int64_t)i * a.kn_s + (int64_t)kvh * a.kn_h;
      float kv = DT<T>::to_f(kp[e]);
      const int pos = past + i;
      if (a.rope != 0 && e < a.R) {
        const int half = a.R / 2;
        if (a.rope == 1) {
          const int j = e < half ? e : e - half;
          const float c = a.cosp[(int64_t)pos * half + j], s = a.sinp[(int64_t)pos * half + j];
          const float o = DT<T>::to_f(kp[e < half ? e + half : e - half]);
          kv = e < half ? kv * c - o * s : kv * c + o * s;
        } else {
          const int j = e >> 1;
          const float c = a.cosp[(int64_t)pos * half + j], s = a.sinp[(int64_t)pos * half + j];
          const float o = DT<T>::to_f(kp[e ^ 1]);
          kv = (e & 1) ? kv * c + o * s : kv * c - o * s;
        }
      }
      float vv = DT<T>::to_f(vp[e]);
      const int64_t coff = b * a.c_b + (int64_t)kvh * a.c_h + (int64_t)pos * a.c_s + e;
      if constexpr (FP8) {
        const uint8_t kq = to_e5m2(kv), vq = to_e5m2(vv);
        kv = from_e5m2(kq);
        vv = from_e5m2(vq);
        if (rb == 0) {
          reinterpret_cast<uint8_t*>(a.kcache)[coff] = kq;
          reinterpret_cast<uint8_t*>(a.vcache)[coff] = vq;
        }
      } else {
        const T kt = DT<T>::from_f(kv), vt = DT<T>::from_f(vv);
        kv = DT<T>::to_f(kt);
        vv = DT<T>::to_f(vt);
        if (rb == 0) {
          reinterpret_cast<T*>(a.kcache)[coff] = kt;
          reinterpret_cast<T*>(a.vcache)[coff] = vt;
        }
      }
      knew_s[idx] = kv;
      vnew_s[idx] = vv;
    }
    __syncthreads();
  }

  // ---- online softmax state ----
  float m[RW], l[RW], acc[RW][DPL];
#pragma unroll
  for (int r = 0; r < RW; r++) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; d++) acc[r][d] = 0.f;
  }
  const float cap = a.softcap;
  const float inv_cap_scaled = cap > 0.f ? 1.f / cap : 0.f;

  auto consume = [&](const float (&kf)[DPL], const float (&vf)[DPL], int pos, bool valid) {
#pragma unroll
    for (int r = 0; r < RW; r++) {
      float s = 0.f;
#pragma unroll
      for (int d = 0; d < DPL; d++) s += qr[r][d] * kf[d];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (cap > 0.f) s = cap * tanhf(s * inv_cap_scaled);
      bool ok = valid && qpos[r] >= 0;
      if (ok && causal) {
        const int limit = causal_base + qpos[r] + 1;
        ok = pos < limit && (a.window <= 0 || pos >= limit - a.window);
      }
      if (ok) {
        const float mn = fmaxf(m[r], s);
        const float corr = __expf(m[r] - mn);
        const float p = __expf(s - mn);
        l[r] = l[r] * corr + p;
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[r][d] = acc[r][d] * corr + p * vf[d];
        m[r] = mn;
      }
    }
  };

  // ---- cached tokens of this split ----
  {
    int chunk = (past + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + 15) & ~15;
    const int t0 = split * chunk;
    const int t1 = min(past, t0 + chunk);
    const uint8_t* kc = reinterpret_cast<const uint8_t*>(a.kcache);
    const uint8_t* vc = reinterpret_cast<const uint8_t*>(a.vcache);
    const int64_t head_off = b * a.c_b + (int64_t)kvh * a.c_h + ds * DPL;
    // software pipeline on the raw cache words, kPF steps deep: a step's loads are issued kPF steps before the
    // (serial) online-softmax update consumes them.  One step ahead left every step waiting for most of an L2
    // round trip (about 1 us per step measured: 59 us for the 32-step walks of one kv head with 8 query heads).
    using Raw = RawKV<T, FP8, DPL>;
    constexpr int kStepWords = 2 * Raw::kWords;            // registers one step in flight holds
    constexpr int kState = 2 * RW * DPL;                   // registers of the q rows and their accumulators
    constexpr int kBudget = kState <= 64 ? 48 : (kState <= 128 ? 32 : 16);
    constexpr int kWant = kBudget / kStepWords;
    constexpr int kPF = kWant >= 4 ? 4 : (kWant >= 2 ? kWant : 2);
    Raw kq[kPF], vq[kPF];
    const int stride = 4 * TS;
    int base = t0 + tsub * 4;
#pragma unroll
    for (int i = 0; i < kPF; i++) {
      const int p = base + i * stride + tg;
      if (p < t1) {
        kq[i].load(kc, head_off + (int64_t)p * a.c_s);
        vq[i].load(vc, head_off + (int64_t)p * a.c_s);
      }
    }
    while (base < t1) {
#pragma unroll
      for (int i = 0; i < kPF; i++) {
        const int cur = base + i * stride;                 // warp-uniform
        if (cur < t1) {
          const int pos = cur + tg;
          const bool valid = pos < t1;
          float kf[DPL], vf[DPL];
          if (valid) {
            kq[i].decode(kf);
            vq[i].decode(vf);
          } else {
#pragma unroll
            for (int d = 0; d < DPL; d++) { kf[d] = 0.f; vf[d] = 0.f; }
          }
          // the slot is free again: refill it with the step kPF ahead before the softmax update
          const int np = cur + kPF * stride + tg;
          if (np < t1) {
            kq[i].load(kc, head_off + (int64_t)np * a.c_s);
            vq[i].load(vc, head_off + (int64_t)np * a.c_s);
          }
          consume(kf, vf, pos, valid);
        }
      }
      base += kPF * stride;
    }
  }
  // ---- new tokens (mode A, last split) from shared memory ----
  if (modeA && last_split) {
    for (int base = tsub * 4; base < n_new; base += 4 * TS) {
      const int j = base + tg;
      const bool valid = j < n_new;
      float kf[DPL], vf[DPL];
#pragma unroll
      for (int d = 0; d < DPL; d++) {
        kf[d] = valid ? knew_s[j * D + ds * DPL + d] : 0.f;
        vf[d] = valid ? vnew_s[j * D + ds * DPL + d] : 0.f;
      }
      consume(kf, vf, past + j, valid);
    }
  }

  // ---- merge the 4 token slots of the warp ----
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
#pragma unroll
    for (int r = 0; r < RW; r++) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[r], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[r], o);
      const float mn = fmaxf(m[r], mo);
      const float ca = mn == -INFINITY ? 0.f : __expf(m[r] - mn);
      const float cb = mn == -INFINITY ? 0.f : __expf(mo - mn);
      l[r] = l[r] * ca + lo * cb;
#pragma unroll
      for (int d = 0; d < DPL; d++) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[r][d], o);
        acc[r][d] = acc[r][d] * ca + ao * cb;
      }
      m[r] = mn;
    }
  }
  if (tg == 0) {
#pragma unroll
    for (int r = 0; r < RW; r++) {
#pragma unroll
      for (int d = 0; d < DPL; d++) part_acc[(warp * RW + r) * D + ds * DPL + d] = acc[r][d];
      if (ds == 0) {
        part_ml[(warp * RW + r) * 2 + 0] = m[r];
        part_ml[(warp * RW + r) * 2 + 1] = l[r];
      }
    }
  }
  __syncthreads();

  // ---- merge the token sub-ranges (warps with the same row group) and emit the CTA partial ----
  // thread -> (row in block, dim)
  const int64_t part_stride = D + 2;
  float* my_scratch = a.scratch +
      ((((int64_t)b * a.Hkv + kvh) * a.nrb + rb) * kMaxRows) * a.nsplit * part_stride;
  for (int idx = tid; idx < rows_blk * D; idx += kAttnThreads) {
    const int rrow = idx / D, e = idx % D;
    const int rgi = rrow / RW, r = rrow % RW;
    float mm = -INFINITY;
    for (int ts = 0; ts < TS; ts++) mm = fmaxf(mm, part_ml[((ts * rg_p2 + rgi) * RW + r) * 2]);
    float ll = 0.f, av = 0.f;
    for (int ts = 0; ts < TS; ts++) {
      const int w = ts * rg_p2 + rgi;
      const float mw = part_ml[(w * RW + r) * 2];
      const float c = (mm == -INFINITY) ? 0.f : __expf(mw - mm);
      ll += part_ml[(w * RW + r) * 2 + 1] * c;
      av += part_acc[(w * RW + r) * D + e] * c;
    }
    if (a.nsplit == 1) {
      const int row = row0 + rrow;
      const int i = row / G, gq = row % G;
      T* op = reinterpret_cast<T*>(a.out) + b * a.o_b + (int64_t)i * a.o_s + (int64_t)(kvh * G + gq) * a.o_h;
      op[e] = DT<T>::from_f(ll > 0.f ? av / ll : 0.f);
    } else {
      float* dst = my_scratch + ((int64_t)rrow * a.nsplit + split) * part_stride;
      dst[e] = av;
      if (e == 0) { dst[D] = mm; dst[D + 1] = ll; }
    }
  }
  if (a.nsplit == 1) return;

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* ctr = a.counters + ((int64_t)b * a.Hkv + kvh) * a.nrb + rb;
    const int ticket = atomicAdd(ctr, 1);
    s_last = ticket == a.nsplit - 1;
    if (s_last) *ctr = 0;  // self-cleaning: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Merge of the splits by the CTA that drew the last ticket.  The per-(row, split) weights exp(m_s - M_row) and
  // the row sums are computed once (they used to be recomputed for every output element, which made the merge the
  // longest part of the kernel for grouped-query heads: 59 us for 8 rows x 18 splits), then every thread
  // accumulates its output elements with independent, coalesced loads.
  float* w_s = part_ml + kAttnWarps * RW * 2;          // [rows_blk][nsplit]: m_s, then the weight
  float* l_s = w_s + kMaxRows * a.nsplit;              // [rows_blk][nsplit]: l_s
  float* Lrow = l_s + kMaxRows * a.nsplit;             // [kMaxRows]
  const int np = rows_blk * a.nsplit;
  for (int p = tid; p < np; p += kAttnThreads) {
    const float* src = my_scratch + (int64_t)p * part_stride;      // p = rrow * nsplit + s
    w_s[p] = __ldcg(src + D);
    l_s[p] = __ldcg(src + D + 1);
  }
  __syncthreads();
  if (tid < rows_blk) {
    float mm = -INFINITY;
    for (int s = 0; s < a.nsplit; s++) mm = fmaxf(mm, w_s[tid * a.nsplit + s]);
    float ll = 0.f;
    for (int s = 0; s < a.nsplit; s++) {
      const float ms = w_s[tid * a.nsplit + s];
      const float c = (mm == -INFINITY || ms == -INFINITY) ? 0.f : __expf(ms - mm);
      w_s[tid * a.nsplit + s] = c;
      ll += l_s[tid * a.nsplit + s] * c;
    }
    Lrow[tid] = ll;
  }
  __syncthreads();
  for (int idx = tid; idx < rows_blk * D; idx += kAttnThreads) {
    const int rrow = idx / D, e = idx % D;
    const float* src = my_scratch + (int64_t)rrow * a.nsplit * part_stride + e;
    const float* wr = w_s + rrow * a.nsplit;
    float av = 0.f;
#pragma unroll 4
    for (int s = 0; s < a.nsplit; s++) av += __ldcg(src + s * part_stride) * wr[s];
    const float ll = Lrow[rrow];
    const int row = row0 + rrow;
    const int i = row / G, gq = row % G;
    T* op = reinterpret_cast<T*>(a.out) + b * a.o_b + (int64_t)i * a.o_s + (int64_t)(kvh * G + gq) * a.o_h;
    op[e] = DT<T>::from_f(ll > 0.f ? av / ll : 0.f);
  }
}

// IPEX_LLM_ATTN_RW4=1: 5..8 query rows per kv head use four rows per warp (two row groups, the warps of a group
// split the tokens) instead of two rows per warp with every warp walking all tokens of the split.
static bool wide_rows() {
  static const bool on = [] {
    const char* v = getenv("IPEX_LLM_ATTN_RW4");
    return v != nullptr && v[0] == '1';
  }();
  return on;
}

template <typename T, bool FP8, int D>
cudaError_t launch_rw(const AttnArgs& a, cudaStream_t s, bool pdl) {
  const int G = a.Hq / a.Hkv;
  const int rows = min(kMaxRows, G * a.Sq);
  dim3 grid(a.nsplit * a.nrb, a.Hkv, a.B);
  const bool modeA = a.knew != nullptr;
  auto smem_for = [&](int RW) {
    return (size_t)((modeA ? 2 * a.Sq * D : 0) + kAttnWarps * RW * D + kAttnWarps * RW * 2 +
                    2 * kMaxRows * a.nsplit + kMaxRows /* merge: weights, row sums */) * sizeof(float);
  };
  if (rows <= 1) {
    auto k = attn_decode_kernel<T, FP8, D, 1>;
    size_t sm = smem_for(1);
    if (sm > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    return launch_kernel(k, grid, dim3(kAttnThreads), sm, s, pdl, a);
  } else if (rows <= 8 && !(rows > 4 && wide_rows())) {
    auto k = attn_decode_kernel<T, FP8, D, 2>;
    size_t sm = smem_for(2);
    if (sm > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    return launch_kernel(k, grid, dim3(kAttnThreads), sm, s, pdl, a);
  } else {
    auto k = attn_decode_kernel<T, FP8, D, 4>;
    size_t sm = smem_for(4);
    if (sm > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    return launch_kernel(k, grid, dim3(kAttnThreads), sm, s, pdl, a);
  }
}

template <typename T, bool FP8>
cudaError_t launch_d(int D, const AttnArgs& a, cudaStream_t s, bool pdl) {
  switch (D) {
    case 64: return launch_rw<T, FP8, 64>(a, s, pdl);
    case 128: return launch_rw<T, FP8, 128>(a, s, pdl);
    case 256: return launch_rw<T, FP8, 256>(a, s, pdl);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// Scratch requirement for a launch: floats for the split partials and ints for the tickets.
IPEX_API int64_t ipex_attn_decode_scratch_floats(int B, int Hkv, int G, int Sq, int D, int nsplit) {
  const int rows_total = G * Sq;
  const int nrb = (rows_total + kMaxRows - 1) / kMaxRows;
  return (int64_t)B * Hkv * nrb * kMaxRows * nsplit * (D + 2);
}
IPEX_API int64_t ipex_attn_decode_counter_ints(int B, int Hkv, int G, int Sq) {
  const int rows_total = G * Sq;
  const int nrb = (rows_total + kMaxRows - 1) / kMaxRows;
  return (int64_t)B * Hkv * nrb;
}

// See AttnArgs for the meaning of the arguments.  `counters` must be zero before the first call; the kernel
// leaves it zero.  Returns a cudaError_t.
IPEX_API int ipex_attn_decode(const void* q, const void* knew, const void* vnew, void* kcache, void* vcache, void* out,
                              const int* past_len, int past_scalar, const float* cosp, const float* sinp,
                              float* scratch, int* counters, const int64_t* strides /*12*/, int B, int Sq, int Hq,
                              int Hkv, int D, int nsplit, int rope, int R, int causal, int window, float scale,
                              float softcap, int fp8_kv, int dtype, int pdl, void* stream) {
  if (Hq % Hkv != 0 || Sq < 1 || nsplit < 1) return (int)cudaErrorInvalidValue;
  AttnArgs a;
  a.q = q; a.knew = knew; a.vnew = vnew; a.kcache = kcache; a.vcache = vcache; a.out = out;
  a.past_len = past_len; a.past_scalar = past_scalar; a.cosp = cosp; a.sinp = sinp;
  a.scratch = scratch; a.counters = counters;
  a.q_b = strides[0]; a.q_s = strides[1]; a.q_h = strides[2];
  a.kn_b = strides[3]; a.kn_s = strides[4]; a.kn_h = strides[5];
  a.c_b = strides[6]; a.c_h = strides[7]; a.c_s = strides[8];
  a.o_b = strides[9]; a.o_s = strides[10]; a.o_h = strides[11];
  a.B = B; a.Sq = Sq; a.Hq = Hq; a.Hkv = Hkv; a.nsplit = nsplit;
  const int rows_total = (Hq / Hkv) * Sq;
  a.nrb = (rows_total + kMaxRows - 1) / kMaxRows;
  a.rope = rope; a.R = R; a.causal = causal; a.window = window; a.scale = scale; a.softcap = softcap;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DT_F16) {
    return (int)(fp8_kv ? launch_d<__half, true>(D, a, s, pdl != 0) : launch_d<__half, false>(D, a, s, pdl != 0));
  } else if (dtype == DT_BF16) {
    return (int)(fp8_kv ? launch_d<__nv_bfloat16, true>(D, a, s, pdl != 0)
                        : launch_d<__nv_bfloat16, false>(D, a, s, pdl != 0));
  }
  return (int)cudaErrorInvalidValue;
}
