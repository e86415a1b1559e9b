"""Python entry points of the sm_100a kernels (torch tensors in, torch tensors out).

This is the layer the reference fills with ``xe_linear`` / ``xe_batch`` / ``xe_addons`` calls
(python/llm/src/ipex_llm/transformers/xpu_ops.py:23-162).  Every function launches on the current CUDA stream
through the C ABI of ``libipex_llm_cuda.so`` and raises if the library is missing — there is no eager
fallback on a GPU.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from ..native import cuda_api as api
from ..native.lib import cuda_lib, current_stream, ptr
from ..quant import qtypes as qt
from ..quant.params import FP4Params, get_block_size, get_type_size

_NF4 = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
        -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
        0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
        0.7229568362236023, 1.0]
_FP4 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]

QTYPE_TO_WF = {
    qt.SYM_INT4: api.WF_SYM_INT4, qt.ASYM_INT4: api.WF_ASYM_INT4, qt.NF4: api.WF_LUT4, qt.FP4: api.WF_LUT4,
    qt.FP8E4: api.WF_FP8_E4M3, qt.FP8E5: api.WF_FP8_E5M2, qt.SYM_INT8: api.WF_INT8,
}

_lut_cache = {}
_USE_PDL = os.environ.get("IPEX_LLM_PDL", "1") != "0"
_GEMV_IMPL = os.environ.get("IPEX_LLM_GEMV", "stream")   # stream | tma | v1
_err_flags = {}


def error_flag(device) -> torch.Tensor:
    """Device int the kernels with bounded waits set when a wait expires (0 = healthy)."""
    key = str(device)
    if key not in _err_flags:
        _err_flags[key] = torch.zeros(4, dtype=torch.int32, device=device)
        tune = os.environ.get("IPEX_LLM_GEMV_TUNE")  # "ctas_per_sm,budget_kb,chunks_per_stage"
        if tune:
            a, b, c = (int(v) for v in tune.split(","))
            cuda_lib().ipex_gemv_tma_tune(a, b, c)
        tune = os.environ.get("IPEX_LLM_GEMV_STREAM_TUNE")  # "ring_kb,chunks_per_stage,warps_per_tile"
        if tune and hasattr(cuda_lib(), "ipex_gemv_stream_tune"):
            fn = cuda_lib().ipex_gemv_stream_tune
            fn.argtypes, fn.restype = [ctypes.c_int] * 3, None
            fn(*(int(v) for v in tune.split(",")))
    return _err_flags[key]


def check_error_flag(device):
    """Raise if a kernel recorded an expired wait (synchronises the device)."""
    flag = _err_flags.get(str(device))
    if flag is not None:
        v = int(flag[0].item())
        if v != 0:
            flag.zero_()
            raise RuntimeError(f"ipex_llm_b200: a kernel wait expired (code {v}); results are invalid")
GEMV_MAX_M = 8
_SMEM_LIMIT = 200 * 1024


def lut_for(qtype: int, device) -> torch.Tensor | None:
    if qtype not in (qt.NF4, qt.FP4):
        return None
    key = (qtype, str(device))
    if key not in _lut_cache:
        _lut_cache[key] = torch.tensor(_NF4 if qtype == qt.NF4 else _FP4, dtype=torch.float32, device=device)
    return _lut_cache[key]


def _dt(t: torch.Tensor) -> int:
    return api.dtype_code(t.dtype)


def is_tiled(qtype: int) -> bool:
    return qtype in QTYPE_TO_WF


# ------------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------------
def gemv_lowbit(x: torch.Tensor, w_data: torch.Tensor, qtype: int, N: int, K: int, out: torch.Tensor = None,
                norm_weight: torch.Tensor = None, eps: float = 1e-6, norm_offset: float = 0.0,
                bias: torch.Tensor = None, residual: torch.Tensor = None, act: int = 0, pdl: bool = False,
                wf: int = None) -> torch.Tensor:
    """``x [M<=8, K]`` times a tiled low-bit (or dense half) weight.  ``act``: 0 none, 1 SiLU(gate)*up,
    2 GELU(gate)*up with gate/up row tiles interleaved in ``w_data`` (then the output has N/2 columns)."""
    lib = cuda_lib()
    M = x.shape[0]
    assert 1 <= M <= GEMV_MAX_M and x.stride(-1) == 1
    if wf is None:
        wf = QTYPE_TO_WF[qtype]
    n_out = N // 2 if act else N
    if out is None:
        out = torch.empty((M, n_out), dtype=x.dtype, device=x.device)
    lut = lut_for(qtype, x.device) if wf == api.WF_LUT4 else None
    if _GEMV_IMPL == "stream" and wf in (api.WF_SYM_INT4, api.WF_FP8_E4M3) and x.stride(0) % 8 == 0 and \
            getattr(lib, "ipex_gemv_lowbit_stream", None) is not None:
        # warp-private rings, one tensor-core instruction per 512 weights for up to four tokens
        rc = lib.ipex_gemv_lowbit_stream(ptr(w_data), wf, ptr(x), ptr(out), M, N, K, x.stride(0), out.stride(0),
                                         ptr(norm_weight), eps, norm_offset, ptr(bias), ptr(residual),
                                         residual.stride(0) if residual is not None else 0, act, None, _dt(x),
                                         int(pdl and _USE_PDL), ptr(error_flag(x.device)), current_stream())
        if rc == 0:
            return out
        if rc != 1:
            api.check(rc, "gemv_lowbit_stream")
        # cudaErrorInvalidValue: the staged activations leave no room for the rings -> the other kernels
    if _GEMV_IMPL in ("tma", "stream") and wf not in (api.WF_F16, api.WF_BF16):
        rc = lib.ipex_gemv_lowbit_tma(ptr(w_data), wf, ptr(x), ptr(out), M, N, K, x.stride(0), out.stride(0),
                                      ptr(norm_weight), eps, norm_offset, ptr(bias), ptr(residual),
                                      residual.stride(0) if residual is not None else 0, act, ptr(lut), _dt(x),
                                      int(pdl and _USE_PDL), ptr(error_flag(x.device)), current_stream())
        if rc == 0:
            return out
        if rc != 1:
            api.check(rc, "gemv_lowbit_tma")
        # cudaErrorInvalidValue: x does not fit beside the ring -> non-pipelined kernel
    rc = lib.ipex_gemv_lowbit(ptr(w_data), wf, ptr(x), ptr(out), M, N, K, x.stride(0), out.stride(0),
                              ptr(norm_weight), eps, norm_offset, ptr(bias), ptr(residual),
                              residual.stride(0) if residual is not None else 0, act, ptr(lut), _dt(x),
                              int(pdl and _USE_PDL), current_stream())
    api.check(rc, "gemv_lowbit")
    return out


def gemv_lowbit_ar(x: torch.Tensor, w_data: torch.Tensor, qtype: int, N: int, K: int, out: torch.Tensor, comm,
                   bias: torch.Tensor = None, residual: torch.Tensor = None, pdl: bool = False, wf: int = None):
    """Row-parallel GEMV fused with its all-reduce: ``out = sum_over_ranks(x_r @ W_r.T) (+ bias) (+ residual)``.
    ``comm`` is the group's ``SymmComm``; every rank must issue the same sequence of calls."""
    lib = cuda_lib()
    M = x.shape[0]
    assert 1 <= M <= GEMV_MAX_M and x.stride(-1) == 1
    if wf is None:
        wf = QTYPE_TO_WF[qtype]
    lut = lut_for(qtype, x.device) if wf == api.WF_LUT4 else None
    rank, world, npad, bufs, flags = comm.gemv_ar_args()
    args = (ptr(w_data), wf, ptr(x), ptr(out), M, N, K, x.stride(0), out.stride(0), None, 0.0, 0.0, ptr(bias),
            ptr(residual), residual.stride(0) if residual is not None else 0, ptr(lut), _dt(x),
            int(pdl and _USE_PDL), ptr(error_flag(x.device)), current_stream(), rank, world, npad, ptr(bufs),
            ptr(flags))
    rc = 1
    sfn = getattr(lib, "ipex_gemv_lowbit_stream_ar", None)
    if _GEMV_IMPL == "stream" and sfn is not None and wf in (api.WF_SYM_INT4, api.WF_FP8_E4M3) and \
            x.stride(0) % 8 == 0:
        sfn.argtypes, sfn.restype = lib.ipex_gemv_lowbit_tma_ar.argtypes, ctypes.c_int
        rc = sfn(*args)         # 1 (invalid value) = shape it does not take; nothing was launched
    if rc == 1:
        rc = lib.ipex_gemv_lowbit_tma_ar(*args)
    api.check(rc, "gemv_lowbit_tma_ar")
    return out


def _gemv_rows_per_call(K: int, dtype_size: int = 2) -> int:
    kp = (K + 127) // 128 * 128
    return max(1, min(GEMV_MAX_M, (_SMEM_LIMIT - 8192) // ((kp + 8) * 2)))


def lowbit_linear(x: torch.Tensor, weight: FP4Params) -> torch.Tensor:
    """``x [M, K] @ dequant(weight).T`` for any qtype, any M."""
    N, K = int(weight._shape[0]), int(weight._shape[1])
    qtype = weight.qtype
    M = x.shape[0]
    if x.dtype == torch.float32:
        return lowbit_linear(x.to(torch.float16), weight).to(torch.float32)
    if is_tiled(qtype):
        if M <= GEMV_MAX_M:
            per = _gemv_rows_per_call(K)
            if M <= per:
                return gemv_lowbit(x, weight.data, qtype, N, K)
            out = torch.empty((M, N), dtype=x.dtype, device=x.device)
            for s in range(0, M, per):
                gemv_lowbit(x[s:s + per], weight.data, qtype, N, K, out=out[s:s + per])
            return out
        return gemm_lowbit(x, weight.data, qtype, N, K)
    # qtypes without a tile layout: dequantize the canonical blocks, then the dense GEMM / GEMV
    w = dequantize_device(weight.data, (N, K), qtype, x.dtype)
    return dense_linear(x, w)


_DEQUANT_ONCE_MIN_TOKENS = 1 << 30


def dequant_once_min_tokens() -> int:
    """From this many tokens on, a low-bit GEMM expands its weight once into a transient half-precision matrix and
    runs the dense tcgen05 kernel instead of dequantizing inside the GEMM's producer warps.  Off by default: in
    isolation the dense kernel is faster at 1024 tokens (1012-1143 TFLOP/s against 744), but with the expansion
    pass in front the 1024-token prompt pass of a 7B int4 model measured 32.0 ms against 30.5 ms with the
    dequantizers in the loop.  ``IPEX_LLM_PREFILL_DEQUANT_MIN_TOKENS`` sets the threshold (e.g. 4096 for very long
    prompts, where the expansion is amortised over four times the math)."""
    return int(os.environ.get("IPEX_LLM_PREFILL_DEQUANT_MIN_TOKENS", str(_DEQUANT_ONCE_MIN_TOKENS)))


def gemm_lowbit(x: torch.Tensor, w_data: torch.Tensor, qtype: int, N: int, K: int, out: torch.Tensor = None,
                bias: torch.Tensor = None, residual: torch.Tensor = None) -> torch.Tensor:
    """M > 8: tcgen05 GEMM with in-kernel dequantization when the kernel is built; otherwise dequantize to the
    activation dtype and run the dense tensor-core GEMM."""
    lib = cuda_lib()
    M = x.shape[0]
    fn = getattr(lib, "ipex_gemm_lowbit_tcgen05", None)
    if fn is not None and os.environ.get("IPEX_LLM_TCGEN05", "1") != "0" and x.dtype in (torch.float16, torch.bfloat16):
        from . import tcgen05_gemm
        if M >= dequant_once_min_tokens() and is_tiled(qtype) and K % 8 == 0:
            # many tokens: expand the weight once and use the dense TMA-fed kernel (see dequant_once_min_tokens)
            wd = dequantize_device(w_data, (N, K), qtype, x.dtype)
            return tcgen05_gemm.gemm_dense(x, wd, bias=bias, residual=residual, out=out)
        if tcgen05_gemm.supported(M, N, K, qtype):
            return tcgen05_gemm.gemm_lowbit(x, w_data, qtype, N, K, out=out, bias=bias, residual=residual)
    w = dequantize_device(w_data, (N, K), qtype, x.dtype)
    y = dense_linear(x, w)
    if bias is not None:
        y = y + bias
    if residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


def dense_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x [M, K] @ w[N, K].T`` for half-precision weights: own GEMV for M <= 8, own tcgen05 GEMM above when
    available, cuBLAS as the plain library GEMM otherwise."""
    M, K = x.shape
    N = w.shape[0]
    if M <= GEMV_MAX_M and K % 64 == 0 and w.is_contiguous() and x.dtype == w.dtype and \
            x.dtype in (torch.float16, torch.bfloat16) and M <= _gemv_rows_per_call(K):
        wf = api.WF_F16 if w.dtype == torch.float16 else api.WF_BF16
        return gemv_lowbit(x, w, None, N, K, wf=wf)
    lib = cuda_lib()
    if getattr(lib, "ipex_gemm_tcgen05", None) is not None and os.environ.get("IPEX_LLM_TCGEN05", "1") != "0":
        from . import tcgen05_gemm
        if tcgen05_gemm.dense_supported(M, N, K, x.dtype) and x.dtype == w.dtype:
            return tcgen05_gemm.gemm_dense(x, w)
    return torch.matmul(x, w.t())


def lowbit_linear_backward(grad_output: torch.Tensor, weight: FP4Params) -> torch.Tensor:
    """``grad_x = grad_y @ dequant(W)`` (QLoRA backward, reference low_bit_linear.py:522-540)."""
    N, K = int(weight._shape[0]), int(weight._shape[1])
    go = grad_output.reshape(-1, N)
    w = dequantize_device(weight.data, (N, K), weight.qtype, go.dtype if go.dtype != torch.float32
                          else torch.bfloat16)
    return torch.matmul(go.to(w.dtype), w).to(grad_output.dtype).view(*grad_output.shape[:-1], K)


def dequantize_device(w_data: torch.Tensor, shape, qtype: int, dtype=torch.float16) -> torch.Tensor:
    """Full dense weight from device-resident packed bytes."""
    N, K = int(shape[0]), int(shape[1])
    if qtype in qt.IQ_QTYPES:
        # code-book formats: the look-up is tensor code (quant/iq_codebooks.py), the product then runs dense
        from ..quant import iq_codebooks
        return iq_codebooks.dequantize(w_data, (N, K), qtype, dtype)
    lib = cuda_lib()
    out = torch.empty((N, K), dtype=dtype, device=w_data.device)
    if is_tiled(qtype):
        rc = lib.ipex_dequantize_tiles(ptr(w_data), ptr(out), N, K, K, QTYPE_TO_WF[qtype],
                                       ptr(lut_for(qtype, w_data.device)), api.dtype_code(dtype), current_stream())
        api.check(rc, "dequantize_tiles")
    else:
        qk, ts = get_block_size(qtype), get_type_size(qtype)
        raw = w_data.view(torch.uint8)
        rc = lib.ipex_dequantize_blocks(ptr(raw), ptr(out), N * K // qk, qk, ts, qtype, api.dtype_code(dtype),
                                        current_stream())
        api.check(rc, "dequantize_blocks")
    return out


def dequantize_rows(ids: torch.Tensor, weight: FP4Params, dim: int, vocab: int, dtype) -> torch.Tensor:
    lib = cuda_lib()
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    out_dtype = dtype if dtype in (torch.float16, torch.bfloat16, torch.float32) else torch.float32
    out = torch.empty((flat.numel(), dim), dtype=out_dtype, device=ids.device)
    qk, ts = get_block_size(weight.qtype), get_type_size(weight.qtype)
    raw = weight.data.view(torch.uint8)
    rc = lib.ipex_dequantize_rows(ptr(flat), ptr(raw), ptr(out), flat.numel(), dim, qk, ts, weight.qtype,
                                  api.dtype_code(out_dtype), current_stream())
    api.check(rc, "dequantize_rows")
    return out.view(*ids.shape, dim)


# ------------------------------------------------------------------------------------------------
# norms / activations / softmax / rope
# ------------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float = 0.0, residual: torch.Tensor = None,
             residual_out: torch.Tensor = None, pdl: bool = False) -> torch.Tensor:
    lib = cuda_lib()
    xc = x.contiguous()
    H = xc.shape[-1]
    rows = xc.numel() // H
    out = torch.empty_like(xc)
    w = weight if weight.dtype == xc.dtype else weight.to(xc.dtype)
    rc = lib.ipex_rms_norm(ptr(xc), ptr(w), ptr(residual), ptr(out), ptr(residual_out), rows, H, eps, offset, _dt(xc),
                           int(pdl and _USE_PDL), current_stream())
    api.check(rc, "rms_norm")
    return out


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    lib = cuda_lib()
    xc = x.contiguous()
    H = xc.shape[-1]
    out = torch.empty_like(xc)
    w = weight.to(xc.dtype) if weight is not None else None
    b = bias.to(xc.dtype) if bias is not None else None
    rc = lib.ipex_layer_norm(ptr(xc), ptr(w), ptr(b), ptr(out), xc.numel() // H, H, eps, _dt(xc), current_stream())
    api.check(rc, "layer_norm")
    return out


def act_mul(gate: torch.Tensor, up: torch.Tensor, act: int) -> torch.Tensor:
    lib = cuda_lib()
    g, u = gate.contiguous(), up.contiguous()
    out = torch.empty_like(g)
    rc = lib.ipex_act_mul(ptr(g), ptr(u), ptr(out), g.numel(), act, _dt(g), 0, current_stream())
    api.check(rc, "act_mul")
    return out


def softmax_inplace(x: torch.Tensor) -> torch.Tensor:
    lib = cuda_lib()
    cols = x.shape[-1]
    rc = lib.ipex_softmax_inplace(ptr(x), x.numel() // cols, cols, _dt(x), current_stream())
    api.check(rc, "softmax_inplace")
    return x


def rotary_inplace(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved=False):
    """RoPE in place on ``q [B,Hq,S,D]`` / ``k [B,Hk,S,D]`` (arbitrary outer strides, unit inner stride);
    ``cos``/``sin`` ``[B or 1, S, R]``.  Returns (q, k)."""
    lib = cuda_lib()
    if q.stride(-1) != 1:
        q = q.contiguous()
    if k.stride(-1) != 1:
        k = k.contiguous()
    B, Hq, S, D = q.shape
    Hk = k.shape[1]
    R = cos.shape[-1]
    # transformers passes cos/sin duplicated over the two halves ([.., R] with R = rotary dim): use the first half
    cosc = cos[..., : R // 2].contiguous() if not interleaved else cos[..., 0::2].contiguous()
    sinc = sin[..., : R // 2].contiguous() if not interleaved else sin[..., 0::2].contiguous()
    cs_b = cosc.stride(0) if cosc.shape[0] == B and B > 1 else 0
    cos_dt = api.DT_F32 if cosc.dtype == torch.float32 else _dt(cosc)
    if cos_dt != api.DT_F32 and cosc.dtype != q.dtype:
        cosc, sinc, cos_dt = cosc.float(), sinc.float(), api.DT_F32
    rc = lib.ipex_rope_inplace(ptr(q), ptr(k), ptr(cosc), ptr(sinc), B, Hq, Hk, S, R, q.stride(0), q.stride(1),
                               q.stride(2), k.stride(0), k.stride(1), k.stride(2), cs_b, cosc.stride(1),
                               int(interleaved), _dt(q), cos_dt, current_stream())
    api.check(rc, "rope_inplace")
    return q, k


def quantize_kv_e5m2(x: torch.Tensor) -> torch.Tensor:
    lib = cuda_lib()
    xc = x.contiguous()
    D = xc.shape[-1]
    out = torch.empty(xc.shape, dtype=torch.uint8, device=xc.device)
    rc = lib.ipex_kv_quant_e5m2(ptr(xc), ptr(out), xc.numel() // D, D, D, _dt(xc), current_stream())
    api.check(rc, "kv_quant_e5m2")
    return out


def dequantize_kv_e5m2(x: torch.Tensor, dtype) -> torch.Tensor:
    lib = cuda_lib()
    D = x.shape[-1]
    if x.stride(-1) != 1 or not _rows_uniform(x):
        x = x.contiguous()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    if x.is_contiguous():
        rc = lib.ipex_kv_dequant_e5m2(ptr(x), ptr(out), x.numel() // D, D, D, api.dtype_code(dtype), current_stream())
        api.check(rc, "kv_dequant_e5m2")
        return out
    # [B, H, S, D] view into a larger [B, H, cap, D] buffer: convert per (b, h) slab
    B, H, S, _ = x.shape
    for b in range(B):
        for h in range(H):
            src = x[b, h]
            rc = lib.ipex_kv_dequant_e5m2(ptr(src), ptr(out[b, h]), S, D, src.stride(0), api.dtype_code(dtype),
                                          current_stream())
            api.check(rc, "kv_dequant_e5m2")
    return out


def _rows_uniform(x):
    return x.dim() == 4


def repetition_penalty_inplace(logits: torch.Tensor, input_ids: torch.Tensor, penalty: float):
    lib = cuda_lib()
    B, V = logits.shape
    ids = input_ids.to(torch.int64).contiguous()
    rc = lib.ipex_repetition_penalty(ptr(logits), ptr(ids), B, V, ids.shape[1], penalty, _dt(logits),
                                     current_stream())
    api.check(rc, "repetition_penalty")
    return logits


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
_attn_ws = {}


def sdpa_decode_supported(head_dim: int, v_head_dim: int) -> bool:
    return head_dim == v_head_dim and head_dim in (64, 128, 256)


def pick_nsplit(B: int, Hkv: int, kv_len: int, n_sm: int = 148, rows: int = 1) -> int:
    """Number of KV splits.  A warp walks its tokens serially (4 per step, one step prefetched), so the split
    count is chosen to keep that chain short: about ``IPEX_LLM_ATTN_STEPS`` steps per warp.  ``rows`` = q rows
    per kv head (GQA group x query length): with more rows the warps of a CTA divide rows, not tokens."""
    # measured: 8 steps is best for one query row per kv head (Llama-2-7B, 2.37 vs 2.39 ms/token at 16); grouped-query
    # heads do better with longer walks and fewer partials to combine (70B shape at TP=2: 2.67 ms at 32 vs 3.15 at 8)
    steps = int(os.environ.get("IPEX_LLM_ATTN_STEPS", "8" if rows <= 1 else "32"))
    rows_blk = min(16, max(1, rows))
    rw = 1 if rows_blk <= 1 else (2 if rows_blk <= 8 else 4)
    row_groups = -(-rows_blk // rw)
    rg_p2 = 1 if row_groups <= 1 else (2 if row_groups <= 2 else 4)
    ts = 4 // rg_p2                      # warps sharing a row group split the tokens
    tokens_per_split = 4 * ts * steps
    by_len = max(1, -(-kv_len // tokens_per_split))
    # few kv heads per GPU (tensor parallel over many ranks) leave most SMs idle under the rule above (18 CTAs for
    # one kv head of the 70B model at 8 ranks).  Splitting further, down to 8 steps per walk, is available through
    # IPEX_LLM_ATTN_MIN_CTAS but off: measured on that shape, 64 splits took 54 us against 44 us for 18 (the merge
    # by the last CTA grows with the split count), and the 8-rank decode step went from 12.8 to 15.8 ms with it
    min_ctas = int(os.environ.get("IPEX_LLM_ATTN_MIN_CTAS", "0"))
    if B * Hkv * by_len < min_ctas:
        finest = max(1, kv_len // (4 * ts * 8))
        by_len = max(by_len, min(-(-min_ctas // max(1, B * Hkv)), finest))
    return int(max(1, min(by_len, 128)))


_attn_ws_retired = []


def attn_workspace(device, floats: int, ints: int):
    """Per-device scratch of the split-KV kernel (grown on demand, tickets zeroed once).

    A captured CUDA graph bakes in the addresses it was given, so a workspace that has been handed out is never
    returned to the allocator: when a larger request arrives the old pair is parked in ``_attn_ws_retired`` and
    stays valid for every graph that references it."""
    key = str(device)
    ws = _attn_ws.get(key)
    if ws is None or ws[0].numel() < floats or ws[1].numel() < ints:
        if ws is not None:
            _attn_ws_retired.append(ws)
        ws = (torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=device),
              torch.zeros(max(ints, 4096), dtype=torch.int32, device=device))
        _attn_ws[key] = ws
    return ws


def sdpa_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask, scale: float, softcap, sliding_window,
                causal: bool = True) -> torch.Tensor:
    """Module-path decode attention: the cache views ``k``/``v`` ``[B,Hkv,Skv,D]`` (activation dtype or e5m2
    bytes) already hold every token; ``q [B,Hq,Sq<=32,D]`` is already rotated."""
    generic = False
    if mask is not None:
        if mask.dtype == torch.bool:
            generic = not bool(mask.all())
        elif bool((mask != 0).any()):
            if _is_causal_mask(mask, q.shape[2], k.shape[2]):
                causal = True            # the mask spells out the causal pattern: the kernel applies it itself
            else:
                generic = True
    if generic:
        # arbitrary masks (padding) take the generic path
        from .kv_cache import fp8_e5m2_dequantize
        from ..models.common import repeat_kv
        if k.dtype == torch.uint8:
            k, v = fp8_e5m2_dequantize(k, q.dtype), fp8_e5m2_dequantize(v, q.dtype)
        kk, vv = repeat_kv(k, q.shape[1] // k.shape[1]), repeat_kv(v, q.shape[1] // k.shape[1])
        m = mask[..., : k.shape[2]]
        return torch.nn.functional.scaled_dot_product_attention(q, kk, vv, attn_mask=m.to(q.dtype) if
                                                                m.dtype != torch.bool else m, scale=scale)
    lib = cuda_lib()
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    fp8 = k.dtype == torch.uint8
    if k.stride(-1) != 1 or v.stride(-1) != 1 or k.stride() != v.stride():
        k, v = k.contiguous(), v.contiguous()
    if q.stride(-1) != 1:
        q = q.contiguous()
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    G = Hq // Hkv
    nsplit = pick_nsplit(B, Hkv, Skv, rows=G * Sq)
    floats = lib.ipex_attn_decode_scratch_floats(B, Hkv, G, Sq, D, nsplit)
    ints = lib.ipex_attn_decode_counter_ints(B, Hkv, G, Sq)
    scratch, counters = attn_workspace(q.device, floats, ints)
    strides = (ctypes.c_int64 * 12)(q.stride(0), q.stride(2), q.stride(1), 0, 0, 0,
                                    k.stride(0), k.stride(1), k.stride(2),
                                    out.stride(0), out.stride(1), out.stride(2))
    rc = lib.ipex_attn_decode(ptr(q), None, None, ptr(k), ptr(v), ptr(out), None, Skv, None, None, ptr(scratch),
                              ptr(counters), strides, B, Sq, Hq, Hkv, D, nsplit, 0, 0, int(causal),
                              int(sliding_window or 0), float(scale), float(softcap or 0.0), int(fp8), _dt(q), 0,
                              current_stream())
    api.check(rc, "attn_decode")
    return out.transpose(1, 2)


def _is_causal_mask(mask, q_len, kv_len) -> bool:
    """True when an additive/bool mask is exactly the causal pattern for the last ``q_len`` positions."""
    m = mask[..., :kv_len]
    if m.shape[-2] != q_len:
        return False
    allowed = (m if m.dtype == torch.bool else (m == 0))
    qi = torch.arange(kv_len - q_len, kv_len, device=m.device).view(-1, 1)
    ki = torch.arange(kv_len, device=m.device).view(1, -1)
    return bool((allowed == (ki <= qi)).all())


def _token_major(t: torch.Tensor) -> bool:
    """``t [B, H, S, D]`` is a view of a token-major activation: element (b, h, s, d) at
    ``(b * S + s) * ld + h * D + d`` (what slicing the fused qkv output and transposing gives)."""
    B, H, S, D = t.shape
    ld = t.stride(2)
    return t.stride(3) == 1 and t.stride(1) == D and (B == 1 or t.stride(0) == S * ld) and ld % 8 == 0 and \
        t.data_ptr() % 16 == 0


def attn_prefill_tcgen05_ok(q, k, v) -> bool:
    """Shapes and layouts the tcgen05 prompt-attention kernel takes; ``IPEX_LLM_TCGEN05_ATTN=0`` switches it off."""
    if os.environ.get("IPEX_LLM_TCGEN05_ATTN", "1") == "0" or not q.is_cuda or q.requires_grad:
        return False
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        return False
    B, Hq, S, D = q.shape
    if D not in (64, 128) or k.shape[2] != S or S < 64 or Hq % k.shape[1] != 0 or B > 65535:
        return False
    if not hasattr(cuda_lib(), "ipex_attn_prefill_tcgen05"):
        return False
    return _token_major(q) and _token_major(k)


def attn_prefill_tcgen05(q, k, v, scale: float, causal: bool = True, softcap: float = 0.0, window: int = 0,
                         kv_lo: torch.Tensor = None) -> torch.Tensor:
    """Prompt attention (Sq == Skv) on the tcgen05 kernel.  ``q [B, Hq, S, D]`` and ``k [B, Hkv, S, D]`` are
    token-major views (see ``_token_major``), already rotated; ``v`` any layout.  Returns ``[B, Hq, S, D]`` as a
    view of a ``[B, S, Hq, D]`` buffer, so the ``transpose(1, 2).reshape(T, Hq * D)`` that feeds the output
    projection is free.  ``softcap`` (Gemma-2 tanh cap of the scaled scores), ``window`` (sliding window) and
    ``kv_lo`` (int32 ``[B]``: first real token of each left-padded row) are applied inside the kernel."""
    lib = cuda_lib()
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    s_pad = (S + 7) // 8 * 8
    if _token_major(v) and B * Hkv <= 65535 and hasattr(lib, "ipex_attn_transpose_v"):
        # tiled transpose kernel (a strided torch copy of this shape runs at a fraction of the memory rate and
        # cost as much as the attention itself)
        vt = torch.empty(B, Hkv, D, s_pad, dtype=q.dtype, device=q.device)
        rc = lib.ipex_attn_transpose_v(ptr(v), ptr(vt), B, S, Hkv, D, v.stride(2), s_pad, _dt(q), current_stream())
        api.check(rc, "attn_transpose_v")
    else:
        vt = torch.zeros(B, Hkv, D, s_pad, dtype=q.dtype, device=q.device) if s_pad != S else \
            torch.empty(B, Hkv, D, S, dtype=q.dtype, device=q.device)
        vt[..., :S].copy_(v.transpose(-1, -2))
    out = torch.empty(B, S, Hq, D, dtype=q.dtype, device=q.device)
    if softcap or window or kv_lo is not None:
        fn = lib.ipex_attn_prefill_tcgen05_ex
        vp, ci, i64, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
        fn.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, i64, i64, i64, i64, cf, ci, cf, ci, vp, ci, vp, vp]
        fn.restype = ci
        rc = fn(ptr(q), ptr(k), ptr(vt), ptr(out), B, S, Hq, Hkv, D, q.stride(2), k.stride(2), s_pad, Hq * D,
                float(scale), int(bool(causal)), float(softcap or 0.0), int(window or 0), ptr(kv_lo), _dt(q),
                ptr(error_flag(q.device)), current_stream())
    else:
        rc = lib.ipex_attn_prefill_tcgen05(ptr(q), ptr(k), ptr(vt), ptr(out), B, S, Hq, Hkv, D, q.stride(2),
                                           k.stride(2), s_pad, Hq * D, float(scale), int(bool(causal)), _dt(q),
                                           ptr(error_flag(q.device)), current_stream())
    api.check(rc, "attn_prefill_tcgen05")
    return out.transpose(1, 2)


_mask_shape_cache = {}


def left_pad_mask_bounds(mask: torch.Tensor, S: int, window: int = 0):
    """If ``mask`` (``[B, 1, S, S]``, boolean "may attend" or additive) is exactly a left-padding mask, i.e.
    ``key >= lo[b]`` (and ``key <= query`` when causal, and ``key > query - window`` with a sliding window) for
    every real query row, return ``(lo int32 [B], causal)``; else ``None``.  Rows of padding queries are ignored
    (their content differs between mask builders and their outputs are never used).  One comparison and one host
    synchronisation per distinct mask: the result is cached for the layers that follow."""
    if mask.dim() != 4 or mask.shape[1] != 1 or mask.shape[2] != S or mask.shape[3] < S:
        return None
    # cached per live tensor object (a weak reference, not the address: the allocator hands a freed mask's memory to
    # the next one) and per in-place version
    import weakref
    key = (id(mask), mask._version, S, window)
    hit = _mask_shape_cache.get(key)
    if hit is not None and hit[0]() is mask:
        return hit[1]
    vis = mask[:, 0, :, :S]
    if vis.dtype == torch.bool:
        other = None
    else:
        # an additive mask is 0 where a key may be seen and a large negative number where not (-inf, the dtype's
        # minimum, the minimum of another dtype after a cast, the -10000 of older models); any other value is a bias
        # that the kernel cannot express
        add = vis
        vis = add == 0
        other = ~(vis | (add <= -1e4))
    # keys that some query sees; rows that see everything are left out (mask builders "unmask" the rows of padding
    # queries completely), and a batch row without any other kind of row has no padding
    partial = vis & ~vis.all(dim=-1, keepdim=True)
    any_col = partial.any(dim=-2)
    lo = torch.where(any_col.any(dim=-1), any_col.int().argmax(dim=-1), torch.zeros_like(any_col[:, 0].int()))
    qi = torch.arange(S, device=mask.device).view(1, S, 1)
    ki = torch.arange(S, device=mask.device).view(1, 1, S)
    real_q = qi >= lo.view(-1, 1, 1)
    result = None
    for causal in (True, False):
        exp = ki >= lo.view(-1, 1, 1)
        if causal:
            exp = exp & (ki <= qi)
        if window:
            exp = exp & (ki > qi - window)
        agree = (vis == exp) | ~real_q
        if other is not None:
            agree = agree & ~other
        if bool(agree.all()):
            result = (lo.to(torch.int32).contiguous(), causal)
            break
    if len(_mask_shape_cache) > 8:
        _mask_shape_cache.clear()
    _mask_shape_cache[key] = (weakref.ref(mask), result)
    return result


def sdpa_prefill(q, k, v, mask, scale, softcap, sliding_window, causal=True):
    """Prefill attention.  Uses the package's tcgen05 flash kernel when built and applicable; otherwise the
    library SDPA (flash) on repeated KV heads — the same fallback the reference takes off its own device
    (models/common.py:288-305)."""
    from ..models.common import repeat_kv
    n_rep = q.shape[1] // k.shape[1]
    D = q.shape[-1]
    if D in (72, 80, 96, 112) and q.is_cuda and not q.requires_grad and q.shape[2] == k.shape[2] and \
            q.shape[2] >= 64 and q.dtype in (torch.float16, torch.bfloat16) and \
            hasattr(cuda_lib(), "ipex_attn_prefill_tcgen05") and os.environ.get("IPEX_LLM_TCGEN05_ATTN", "1") != "0":
        # head dims between the kernel's sizes (Phi-2 / StableLM 80, Phi-3-mini 96, SigLIP 72): zero-pad to 128 in a
        # token-major buffer (the padded dims add nothing to q.k and produce zero output columns), as the
        # reference pads them for its own kernels (models/utils.py:218-240)
        B, Hq, S, _ = q.shape
        Hkv = k.shape[1]
        buf = torch.zeros(B, S, Hq + 2 * Hkv, 128, dtype=q.dtype, device=q.device)
        buf[:, :, :Hq, :D] = q.transpose(1, 2)
        buf[:, :, Hq:Hq + Hkv, :D] = k.transpose(1, 2)
        buf[:, :, Hq + Hkv:, :D] = v.transpose(1, 2)
        out = sdpa_prefill(buf[:, :, :Hq].transpose(1, 2), buf[:, :, Hq:Hq + Hkv].transpose(1, 2),
                           buf[:, :, Hq + Hkv:].transpose(1, 2), mask, scale, softcap, sliding_window, causal)
        return out[..., :D]
    if (softcap or sliding_window or mask is not None) and attn_prefill_tcgen05_ok(q, k, v) and \
            hasattr(cuda_lib(), "ipex_attn_prefill_tcgen05_ex") and \
            os.environ.get("IPEX_LLM_TCGEN05_ATTN_EXT", "1") != "0":
        # soft-capped (Gemma-2), sliding-window and left-padded prompts stay on the tcgen05 kernel
        S = q.shape[2]
        window = int(sliding_window) if sliding_window and sliding_window < S else 0
        bounds = left_pad_mask_bounds(mask, S, window) if mask is not None else (None, causal)
        if bounds is not None and bounds[0] is not None and bounds[0].shape[0] != q.shape[0]:
            # a mask shared by the whole batch ([1, 1, S, S]): the kernel reads one bound per batch row
            bounds = (bounds[0].expand(q.shape[0]).contiguous(), bounds[1]) if bounds[0].shape[0] == 1 else None
        if bounds is not None:
            lo, is_causal = bounds
            return attn_prefill_tcgen05(q, k, v, scale, is_causal, softcap or 0.0, window, lo)
    if softcap or sliding_window:
        kk, vv = repeat_kv(k, n_rep), repeat_kv(v, n_rep)
        w = torch.matmul(q, kk.transpose(2, 3)).float() * scale
        if softcap:
            w = torch.tanh(w / softcap) * softcap
        q_len, kv_len = q.shape[2], k.shape[2]
        if mask is not None:
            m = mask[..., :kv_len]
            w = w.masked_fill(~m, float("-inf")) if m.dtype == torch.bool else w + m.float()
        else:
            qi = torch.arange(kv_len - q_len, kv_len, device=w.device).view(-1, 1)
            ki = torch.arange(kv_len, device=w.device).view(1, -1)
            allowed = ki <= qi if causal else torch.ones_like(ki <= qi)
            if sliding_window:
                allowed = allowed & (ki > qi - sliding_window)
            w = w.masked_fill(~allowed, float("-inf"))
        # (rows without any visible key, e.g. left padding under a sliding window, attend to nothing instead of NaN)
        return torch.matmul(torch.nan_to_num(torch.softmax(w, dim=-1), nan=0.0).to(q.dtype), vv)
    if mask is not None:
        m = mask[..., : k.shape[2]]
        if m.dtype != torch.bool and m.dtype != q.dtype:
            m = m.to(q.dtype)
        return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=m, scale=scale,
                                                                enable_gqa=n_rep > 1)
    if attn_prefill_tcgen05_ok(q, k, v):
        return attn_prefill_tcgen05(q, k, v, scale, causal)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal and q.shape[2] > 1,
                                                            scale=scale, enable_gqa=n_rep > 1)


# ------------------------------------------------------------------------------------------------
# MoE (the fused kernels register themselves here when built)
# ------------------------------------------------------------------------------------------------
_MOE_MAX_SLOTS = 64       # tokens x experts-per-token handled by the per-slot GEMV launch (decode / small batches)


class _MoeBank:
    """Device-side view of a ``LowBitExperts`` bank: per-expert gate/up merged into interleaved 16-row tiles (so
    the GEMV epilogue can apply act(gate) * up) and pointer tables indexed by expert id."""

    def __init__(self, experts):
        from ..engine.decoder_engine import _W, _interleave_row_tiles
        q = experts.qtype
        wf = QTYPE_TO_WF[q]
        H, I = experts.hidden_dim, experts.intermediate_dim
        self.gate_up, gu_ptrs, dn_ptrs = [], [], []
        for i in range(experts.num_experts):     # (an activation module may be registered beside the experts)
            e = experts[i]
            merged = _interleave_row_tiles(_W(e.w1.weight.data, wf, q, I, H), _W(e.w3.weight.data, wf, q, I, H))
            self.gate_up.append(merged.data)
            gu_ptrs.append(merged.data.data_ptr())
            dn_ptrs.append(e.w2.weight.data.data_ptr())
        dev = experts[0].w1.weight.data.device
        self.gu_ptrs_host, self.dn_ptrs_host = gu_ptrs, dn_ptrs
        self.gu_ptrs = torch.tensor(gu_ptrs, dtype=torch.int64, device=dev)
        self.dn_ptrs = torch.tensor(dn_ptrs, dtype=torch.int64, device=dev)
        self.wf, self.qtype, self.H, self.I = wf, q, H, I


def moe_supported(experts) -> bool:
    lib = cuda_lib()
    if getattr(lib, "ipex_moe_gemv", None) is None or not is_tiled(experts.qtype):
        return False
    w = experts[0].w1.weight
    return bool(getattr(w, "quantized", False)) and w.data.is_cuda and experts.hidden_dim % 64 == 0 and \
        experts.intermediate_dim % 64 == 0 and experts.intermediate_dim % 16 == 0


def moe_forward(experts, hidden_states, top_k_index, top_k_weights, residual=None, out=None):
    """Sparse-MoE block ``(residual +) sum_k w_k * expert_k(x)`` without host synchronisation.

    * one token: every (token, choice) slot is a GEMV whose expert is picked on the device;
    * a few tokens: the slots are sorted by expert on the device and each expert's weights are read once for up to
      eight of its tokens (``ipex_moe_gemv_grouped``);
    * prompts: expert-sorted rows through the tcgen05 GEMM with device-side row ranges."""
    lib = cuda_lib()
    T, k = top_k_index.shape
    slots = T * k
    if slots > _MOE_MAX_SLOTS:
        out = _moe_forward_grouped(experts, hidden_states, top_k_index, top_k_weights)
        return out if residual is None else out.add_(residual)
    bank = _moe_bank(experts)
    x = hidden_states.contiguous()
    dt = x.dtype
    act_code = _moe_act_code(experts)
    ids = top_k_index.reshape(-1).to(torch.int64).contiguous()
    act = torch.empty((slots, bank.I), dtype=dt, device=x.device)
    y = torch.empty((slots, bank.H), dtype=dt, device=x.device)
    lut = lut_for(bank.qtype, x.device)
    E = experts.num_experts
    vp, ci = ctypes.c_void_p, ctypes.c_int
    tfn = getattr(lib, "ipex_moe_gemv_tma", None)
    gfn = getattr(lib, "ipex_moe_gemv_grouped", None)
    mode = os.environ.get("IPEX_LLM_MOE_GROUPED_GEMV", "tma")        # tma | tiled | 0 (per-slot launches)
    if (tfn is not None or gfn is not None) and T >= 2 and E <= 4 * slots and E <= 256 and mode != "0":
        order = torch.empty(slots, dtype=torch.int32, device=x.device)
        ranges = torch.empty((E, 2), dtype=torch.int32, device=x.device)
        sfn = lib.ipex_moe_sort_slots
        sfn.argtypes, sfn.restype = [vp, ci, ci, vp, vp, vp], ci
        api.check(sfn(ptr(ids), slots, E, ptr(order), ptr(ranges), current_stream()), "moe_sort_slots")
        if tfn is not None and mode != "tiled":
            # one persistent launch per projection: the weight ring keeps streaming across the experts
            sig = [vp, ci, vp, vp, ci, ci, ci, vp, ci, ci, ci, vp, ci, ci, ci, ci, ci, vp, ci, vp, vp]
            tfn.argtypes, tfn.restype = sig, ci
            sfn2 = getattr(lib, "ipex_moe_gemv_stream", None)      # warp-private rings (sym_int4 / fp8_e4m3)
            if sfn2 is not None:
                sfn2.argtypes, sfn2.restype = sig, ci
            err = ptr(error_flag(x.device))

            def walk(args, what):
                rc = 1
                if sfn2 is not None and mode != "tma-shared":
                    rc = sfn2(*args)            # 1 (invalid value): a format or shape it does not take
                if rc == 1:
                    rc = tfn(*args)
                api.check(rc, what)

            walk((ptr(bank.gu_ptrs), bank.wf, ptr(ranges), ptr(order), E, slots, T, ptr(x), k, 1, 0, ptr(act),
                  2 * bank.I, bank.H, x.stride(0), act.stride(0), act_code, ptr(lut), _dt(x), err,
                  current_stream()), "moe_gemv(gate_up)")
            walk((ptr(bank.dn_ptrs), bank.wf, ptr(ranges), ptr(order), E, slots, T, ptr(act), 1, 0, 1, ptr(y),
                  bank.H, bank.I, act.stride(0), y.stride(0), 0, ptr(lut), _dt(x), err, current_stream()),
                 "moe_gemv(down)")
        else:
            gfn.argtypes = [vp, ci, vp, vp, ci, ci, vp, ci, ci, ci, vp, ci, ci, ci, ci, ci, vp, ci, vp]
            gfn.restype = ci
            rows = lib.ipex_moe_gemv_group_rows      # a token picks an expert at most once: <= T slots per expert
            rows.argtypes, rows.restype = [ci], ci
            z = -(-T // rows(bank.H))
            rc = gfn(ptr(bank.gu_ptrs), bank.wf, ptr(ranges), ptr(order), E, z, ptr(x), k, 1, 0, ptr(act),
                     2 * bank.I, bank.H, x.stride(0), act.stride(0), act_code, ptr(lut), _dt(x), current_stream())
            api.check(rc, "moe_gemv_grouped(gate_up)")
            z = -(-T // rows(bank.I))
            rc = gfn(ptr(bank.dn_ptrs), bank.wf, ptr(ranges), ptr(order), E, z, ptr(act), 1, 0, 1, ptr(y), bank.H,
                     bank.I, act.stride(0), y.stride(0), 0, ptr(lut), _dt(x), current_stream())
            api.check(rc, "moe_gemv_grouped(down)")
    else:
        fn = lib.ipex_moe_gemv
        fn.argtypes = [vp, ci, vp, ci, vp, ci, vp] + [ci] * 5 + [vp, ci, ci, vp]
        fn.restype = ci
        rc = fn(ptr(bank.gu_ptrs), bank.wf, ptr(ids), slots, ptr(x), k, ptr(act), 2 * bank.I, bank.H, x.stride(0),
                act.stride(0), act_code, ptr(lut), _dt(x), 0, current_stream())
        api.check(rc, "moe_gemv(gate_up)")
        rc = fn(ptr(bank.dn_ptrs), bank.wf, ptr(ids), slots, ptr(act), 1, ptr(y), bank.H, bank.I, act.stride(0),
                y.stride(0), 0, ptr(lut), _dt(x), 0, current_stream())
        api.check(rc, "moe_gemv(down)")
    if out is None or not out.is_contiguous() or out.shape != x.shape or out.dtype != x.dtype:
        out = torch.empty_like(x)
    w = top_k_weights.to(torch.float32).contiguous()
    if residual is not None:
        residual = residual.contiguous()
    cfn = lib.ipex_moe_combine_add
    cfn.argtypes = [vp] * 4 + [ci] * 4 + [vp]
    cfn.restype = ci
    rc = cfn(ptr(y), ptr(w), ptr(residual), ptr(out), T, k, bank.H, _dt(x), current_stream())
    api.check(rc, "moe_combine")
    return out


def _moe_bank(experts):
    bank = experts.__dict__.get("_cuda_bank")
    if bank is None:
        bank = _MoeBank(experts)
        experts.__dict__["_cuda_bank"] = bank
    return bank


def _moe_act_code(experts) -> int:
    return 1 if getattr(experts.act_fn, "__name__", "silu") in ("silu", "SiLU") or \
        type(experts.act_fn).__name__ in ("SiLU", "SiLUActivation") else 2


def _moe_forward_grouped(experts, hidden_states, top_k_index, top_k_weights):
    """Prompt-sized inputs.  The (token, choice) slots are sorted by expert on the device; every expert's rows then
    go through the low-bit tcgen05 GEMM, which reads its row range (first row, row count) from device memory, so the
    host launches 2 x num_experts GEMMs without ever learning the routing (no synchronisation, graph-capturable).
    gate/up is one GEMM with ``act(gate) * up`` in its epilogue."""
    from . import tcgen05_gemm
    lib = cuda_lib()
    fn = getattr(lib, "ipex_gemm_lowbit_tcgen05_grouped", None)
    H, I = experts.hidden_dim, experts.intermediate_dim
    if fn is None or not tcgen05_gemm.supported(1, 2 * I, H, experts.qtype) or \
            not tcgen05_gemm.supported(1, H, I, experts.qtype) or (2 * I) % 32 != 0 or \
            hidden_states.dtype not in (torch.float16, torch.bfloat16):
        return _moe_forward_per_expert(experts, hidden_states, top_k_index, top_k_weights)
    bank = _moe_bank(experts)
    E = experts.num_experts
    T, k = top_k_index.shape
    slots = T * k
    x = hidden_states.contiguous()
    flat = top_k_index.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    ranges = torch.stack([torch.cumsum(counts, 0) - counts, counts], dim=1).to(torch.int32).contiguous()   # [E, 2]
    xs = x[order // k]                                         # [slots, H], rows grouped by expert
    act = torch.empty((slots, I), dtype=x.dtype, device=x.device)
    ys = torch.empty((slots, H), dtype=x.dtype, device=x.device)
    lut = lut_for(bank.qtype, x.device)
    vp, ci, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    fn.argtypes, fn.restype = [vp, vp, vp, vp, vp, ci, ci, ci, ci, i64, i64, ci, ci, ci, ci, vp, vp], ci
    bt = tcgen05_gemm.token_tile(max(1, (slots + E - 1) // E))
    err, st, dt, code = ptr(error_flag(x.device)), current_stream(), _dt(x), _moe_act_code(experts)
    for e in range(E):
        rc = fn(ptr(xs), bank.gu_ptrs_host[e], ptr(act), ptr(lut), ranges[e].data_ptr(), slots, slots, 2 * I, H,
                xs.stride(0), act.stride(0), bank.wf, code, dt, bt, err, st)
        api.check(rc, "gemm_lowbit_tcgen05_grouped(gate_up)")
    for e in range(E):
        rc = fn(ptr(act), bank.dn_ptrs_host[e], ptr(ys), ptr(lut), ranges[e].data_ptr(), slots, slots, H, I,
                act.stride(0), ys.stride(0), bank.wf, 0, dt, bt, err, st)
        api.check(rc, "gemm_lowbit_tcgen05_grouped(down)")
    y = torch.empty_like(ys)
    y[order] = ys                                              # back to (token, choice) order
    out = torch.empty_like(x)
    w = top_k_weights.to(torch.float32).contiguous()
    cfn = lib.ipex_moe_combine
    cfn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
    cfn.restype = ctypes.c_int
    rc = cfn(ptr(y), ptr(w), ptr(out), T, k, H, dt, st)
    api.check(rc, "moe_combine")
    return out


def _moe_forward_per_expert(experts, hidden_states, top_k_index, top_k_weights):
    """Expert-by-expert form with one host synchronisation (kept for weight formats the grouped GEMM lacks)."""
    from ..models.common import SILU, _act_mul
    final = torch.zeros_like(hidden_states)
    E = experts.num_experts
    flat = top_k_index.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E).tolist()       # one host sync per MoE block
    k = top_k_index.shape[1]
    start = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        sel = order[start:start + c]
        start += c
        tok, pos = sel // k, sel % k
        x = hidden_states[tok]
        exp = experts[e]
        h = _act_mul(exp.w1(x), exp.w3(x), SILU)
        yy = exp.w2(h) * top_k_weights[tok, pos, None].to(h.dtype)
        final.index_add_(0, tok, yy.to(final.dtype))
    return final


def moe_softmax_topk(router_logits, top_k, renormalize):
    lib = cuda_lib()
    fn = getattr(lib, "ipex_moe_softmax_topk", None)
    T, E = router_logits.shape
    if fn is None or E > 256 or top_k > 8:
        probs = torch.softmax(router_logits.float(), dim=-1)
        w, idx = torch.topk(probs, top_k, dim=-1)
        if renormalize:
            w = w / w.sum(dim=-1, keepdim=True)
        return probs, w, idx
    logits = router_logits.contiguous()
    probs = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    idx = torch.empty((T, top_k), dtype=torch.int64, device=logits.device)
    rc = fn(ptr(logits), ptr(probs), ptr(w), ptr(idx), T, E, top_k, int(renormalize), _dt(logits), current_stream())
    api.check(rc, "moe_softmax_topk")
    return probs, w, idx


def moe_group_topk(scores, bias, n_group, topk_group, top_k, norm_topk_prob, routed_scaling_factor):
    """DeepSeek-V3 grouped routing on the device: one kernel (a warp per token) when the shape fits it, tensor ops
    otherwise.  Returns ``(indices [T, k] int64, weights [T, k] fp32)``."""
    from .moe import _group_topk_impl
    lib = cuda_lib()
    fn = getattr(lib, "ipex_moe_group_topk", None)
    T, E = scores.shape
    if fn is None or not scores.is_cuda or scores.requires_grad or E > 256 or n_group > 32 or E % n_group or \
            top_k > 8 or top_k > topk_group * (E // n_group) or \
            scores.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        return _group_topk_impl(scores, bias, n_group, topk_group, top_k, norm_topk_prob, routed_scaling_factor)
    sc = scores.contiguous()
    b = bias.to(torch.float32).contiguous()
    idx = torch.empty((T, top_k), dtype=torch.int64, device=sc.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=sc.device)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes, fn.restype = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, cf, ci, vp], ci
    rc = fn(ptr(sc), ptr(b), ptr(idx), ptr(w), T, E, int(n_group), int(topk_group), int(top_k),
            int(bool(norm_topk_prob)), float(routed_scaling_factor), _dt(sc), current_stream())
    api.check(rc, "moe_group_topk")
    return idx, w
