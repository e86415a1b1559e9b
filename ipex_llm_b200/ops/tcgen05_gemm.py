"""Python front of the tcgen05 (5th-gen tensor core) GEMM kernels used for prompts and batches.

``gemm_dense``  : ``x[M,K] @ w[N,K].T`` for fp16/bf16 weights (TMA -> swizzled shared memory -> tcgen05.mma -> TMEM).
``gemm_lowbit`` : the same contraction with packed low-bit weights dequantized inside the kernel's producer warps.

Reference counterpart: the GEMM branch of ``xe_linear.forward_new`` that the reference takes for prompts
(python/llm/src/ipex_llm/transformers/low_bit_linear.py:640-668) and ``xe_batch.batch_forward``.
"""
from __future__ import annotations

import ctypes

import torch

from ..native import cuda_api as api
from ..native.lib import cuda_lib, current_stream, ptr


def _err(device):
    from . import cuda_ops
    return cuda_ops.error_flag(device)


def dense_supported(M: int, N: int, K: int, dtype) -> bool:
    return dtype in (torch.float16, torch.bfloat16) and K % 8 == 0 and M >= 1 and N >= 8


def gemm_dense(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor = None, residual: torch.Tensor = None,
               out: torch.Tensor = None, act: int = 0) -> torch.Tensor:
    """``x [M, K] @ w[N, K].T (+ bias) (+ residual)``; ``x``/``w`` row strides must be multiples of 8 elements.
    ``act`` != 0: ``w`` holds gate / up rows interleaved in 16-row tiles and the result is ``act(gate) * up`` with
    ``N / 2`` columns (1 = SiLU, 2 = GELU-tanh)."""
    lib = cuda_lib()
    M, K = x.shape
    N = w.shape[0]
    if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    if w.stride(1) != 1 or w.stride(0) % 8 != 0 or w.data_ptr() % 16 != 0:
        w = w.contiguous()
    if out is None:
        out = torch.empty((M, N // 2 if act else N), dtype=x.dtype, device=x.device)
    if residual is not None and residual.stride(1) != 1:
        residual = residual.contiguous()
    fn = lib.ipex_gemm_tcgen05_act
    vp, ci, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    fn.argtypes, fn.restype = [vp, vp, vp, vp, vp, ci, ci, ci, i64, i64, i64, i64, ci, ci, vp, vp], ci
    rc = fn(ptr(x), ptr(w), ptr(out), ptr(bias), ptr(residual), M, N, K, x.stride(0), w.stride(0), out.stride(0),
            residual.stride(0) if residual is not None else 0, api.dtype_code(x.dtype), int(act), ptr(_err(x.device)),
            current_stream())
    if rc == -1:
        raise RuntimeError("ipex_llm_b200: the driver's tensor-map encoder rejected the GEMM operands")
    api.check(rc, "gemm_tcgen05")
    return out


def token_tile(M: int) -> int:
    """Token tile (32 / 64 / 128 / 256) the kernels use for ``M`` rows."""
    return 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256


# weight families the in-kernel dequantizer handles (codes of native/cuda/common/utils.cuh)
_LOWBIT_FAMILIES = ("WF_SYM_INT4", "WF_ASYM_INT4", "WF_LUT4", "WF_FP8_E4M3", "WF_FP8_E5M2", "WF_INT8")


def supported(M: int, N: int, K: int, qtype: int) -> bool:
    from .cuda_ops import QTYPE_TO_WF
    lib = cuda_lib()
    if getattr(lib, "ipex_gemm_lowbit_tcgen05", None) is None or qtype not in QTYPE_TO_WF:
        return False
    ok = {getattr(api, n) for n in _LOWBIT_FAMILIES if hasattr(api, n)}
    return QTYPE_TO_WF[qtype] in ok and K % 128 == 0 and N % 16 == 0


def gemm_lowbit(x: torch.Tensor, w_data: torch.Tensor, qtype: int, N: int, K: int, out: torch.Tensor = None,
                bias: torch.Tensor = None, residual: torch.Tensor = None, act: int = 0, wf: int = None) -> torch.Tensor:
    """``x [M, K] @ dequant(w).T`` with the packed device tiles of ``qtype`` (or of family ``wf``).  ``act`` 1/2
    (silu / gelu-tanh) treats the rows as 16-row-interleaved gate/up and returns ``[M, N/2]``."""
    from .cuda_ops import QTYPE_TO_WF, lut_for
    lib = cuda_lib()
    M = x.shape[0]
    if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    if out is None:
        out = torch.empty((M, N // 2 if act else N), dtype=x.dtype, device=x.device)
    if residual is not None and residual.stride(1) != 1:
        residual = residual.contiguous()
    if wf is None:
        wf = QTYPE_TO_WF[qtype]
    lut = lut_for(qtype, x.device) if qtype is not None else None
    rc = lib.ipex_gemm_lowbit_tcgen05(ptr(x), ptr(w_data), ptr(out), ptr(bias), ptr(residual), ptr(lut), M, N, K,
                                      x.stride(0), out.stride(0),
                                      residual.stride(0) if residual is not None else 0, wf, int(act),
                                      api.dtype_code(x.dtype), ptr(_err(x.device)), current_stream())
    if rc == -1:
        raise RuntimeError("ipex_llm_b200: the driver's tensor-map encoder rejected the GEMM operands")
    api.check(rc, "gemm_lowbit_tcgen05")
    return out



def gemm_lowbit_ar(x: torch.Tensor, w_data: torch.Tensor, qtype: int, N: int, K: int, comm, out: torch.Tensor = None,
                   bias: torch.Tensor = None, residual: torch.Tensor = None, wf: int = None) -> torch.Tensor:
    """Row-parallel projection of a tensor-parallel model: ``sum_over_ranks(x_r @ dequant(W_r).T) (+ bias)
    (+ residual)`` with the all-reduce fused into the GEMM's epilogue (peer stores over NVLink).  ``comm`` is the
    group's ``SymmComm``; every rank issues the same calls in the same order."""
    from .cuda_ops import QTYPE_TO_WF, lut_for
    lib = cuda_lib()
    M = x.shape[0]
    if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if residual is not None and residual.stride(1) != 1:
        residual = residual.contiguous()
    if wf is None:
        wf = QTYPE_TO_WF[qtype]
    lut = lut_for(qtype, x.device) if qtype is not None else None
    sb = lib.ipex_gemm_tcgen05_ar_stage_bytes
    sb.argtypes, sb.restype = [ctypes.c_int] * 3, ctypes.c_int64
    cn = lib.ipex_gemm_tcgen05_ar_counters
    cn.argtypes, cn.restype = [ctypes.c_int] * 2, ctypes.c_int64
    rank, world, stage, flags = comm.gemm_ar_args(int(sb(M, N, comm.world)), int(cn(M, N)))
    fn = lib.ipex_gemm_lowbit_tcgen05_ar
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 3 + [ctypes.c_int64] * 3 + [ctypes.c_int, ctypes.c_int,
                                                                                    ctypes.c_void_p, ctypes.c_void_p,
                                                                                    ctypes.c_int, ctypes.c_int,
                                                                                    ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    rc = fn(ptr(x), ptr(w_data), ptr(out), ptr(bias), ptr(residual), ptr(lut), M, N, K, x.stride(0), out.stride(0),
            residual.stride(0) if residual is not None else 0, wf, api.dtype_code(x.dtype), ptr(_err(x.device)),
            current_stream(), rank, world, ptr(stage), ptr(flags))
    if rc == -1:
        raise RuntimeError("ipex_llm_b200: the driver's tensor-map encoder rejected the GEMM operands")
    api.check(rc, "gemm_lowbit_tcgen05_ar")
    return out


def gemm_lowbit_ag(x_local: torch.Tensor, w_data: torch.Tensor, qtype: int, N: int, K: int, M_total: int, comm,
                   out: torch.Tensor = None, bias: torch.Tensor = None, act: int = 0, wf: int = None) -> torch.Tensor:
    """Column-parallel projection behind an all-gather, fused: ``x_local`` holds this rank's
    ``ceil(M_total / world)`` consecutive token rows (fewer on the last ranks); the kernel pushes them to every
    rank over NVLink, and multiplies each token tile of the gathered activation as soon as the ranks it covers have
    arrived.  Returns ``gathered_x @ dequant(W).T (+ bias)`` (or ``act(gate) * up``) for all ``M_total`` tokens.
    ``comm`` is the group's ``SymmComm``; every rank issues the same calls in the same order."""
    from .cuda_ops import QTYPE_TO_WF, lut_for
    lib = cuda_lib()
    world = comm.world
    ag_rows = (M_total + world - 1) // world
    if x_local.stride(1) != 1 or x_local.stride(0) % 8 != 0 or x_local.data_ptr() % 16 != 0:
        x_local = x_local.contiguous()
    n_out = N // 2 if act else N
    if out is None:
        out = torch.empty((M_total, n_out), dtype=x_local.dtype, device=x_local.device)
    if wf is None:
        wf = QTYPE_TO_WF[qtype]
    lut = lut_for(qtype, x_local.device) if qtype is not None else None
    rank, world, xg, dst, flags, my_flags, ticket, epoch = comm.gemm_ag_args(M_total * K * 2)
    fn = lib.ipex_gemm_lowbit_tcgen05_ag
    vp, ci, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    fn.argtypes = [vp, i64, vp, vp, vp, vp, vp, ci, ci, ci, i64, ci, ci, ci, vp, vp, ci, ci, ci, vp, vp, vp, vp, ci]
    fn.restype = ci
    rc = fn(ptr(x_local), x_local.stride(0), xg, ptr(w_data), ptr(out), ptr(bias), ptr(lut), M_total, N, K,
            out.stride(0), wf, act, api.dtype_code(x_local.dtype), ptr(_err(x_local.device)), current_stream(), rank,
            world, ag_rows, ptr(dst), ptr(flags), my_flags, ticket, epoch)
    if rc == -1:
        raise RuntimeError("ipex_llm_b200: the driver's tensor-map encoder rejected the GEMM operands")
    api.check(rc, "gemm_lowbit_tcgen05_ag")
    return out
