"""ctypes signatures of the CUDA kernel library (``libipex_llm_cuda.so``).

Every launcher returns a ``cudaError_t`` (0 = success); ``check`` turns a failure into a Python exception.
"""
from __future__ import annotations

import ctypes

vp = ctypes.c_void_p
ci = ctypes.c_int
i64 = ctypes.c_int64
cf = ctypes.c_float

DT_F16, DT_BF16, DT_F32 = 0, 1, 2
WF_SYM_INT4, WF_ASYM_INT4, WF_LUT4, WF_FP8_E4M3, WF_FP8_E5M2, WF_INT8, WF_F16, WF_BF16 = range(8)

_SIGS = {
    "ipex_gemv_lowbit": [vp, ci, vp, vp, ci, ci, ci, ci, ci, vp, cf, cf, vp, vp, ci, ci, vp, ci, ci, vp],
    "ipex_gemv_lowbit_tma": [vp, ci, vp, vp, ci, ci, ci, ci, ci, vp, cf, cf, vp, vp, ci, ci, vp, ci, ci, vp, vp],
    "ipex_gemv_lowbit_stream": [vp, ci, vp, vp, ci, ci, ci, ci, ci, vp, cf, cf, vp, vp, ci, ci, vp, ci, ci, vp, vp],
    "ipex_gemv_lowbit_tma_ar": [vp, ci, vp, vp, ci, ci, ci, ci, ci, vp, cf, cf, vp, vp, ci, vp, ci, ci, vp, vp,
                                ci, ci, ci, vp, vp],
    "ipex_allreduce_oneshot": [vp, vp, vp, i64, ci, ci, ci, vp, ci, ci, vp],
    "ipex_allreduce_oneshot_epi": [vp, vp, vp, i64, ci, ci, ci, vp, ci, ci, vp, vp, ci, vp],
    "ipex_symm_barrier": [vp, ci, ci, vp, vp],
    "ipex_wait_timeout_probe": [vp, ci, ci, vp, vp],
    "ipex_rms_norm": [vp, vp, vp, vp, vp, i64, ci, cf, cf, ci, ci, vp],
    "ipex_layer_norm": [vp, vp, vp, vp, i64, ci, cf, ci, vp],
    "ipex_act_mul": [vp, vp, vp, i64, ci, ci, ci, vp],
    "ipex_softmax_inplace": [vp, i64, ci, ci, vp],
    "ipex_attn_prefill_tcgen05": [vp, vp, vp, vp, ci, ci, ci, ci, ci, i64, i64, i64, i64, cf, ci, ci, vp, vp],
    "ipex_attn_transpose_v": [vp, vp, ci, ci, ci, ci, i64, i64, ci, vp],
    "ipex_rwkv_wkv_v4": [vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp],
    "ipex_rwkv_linear_attention_v5": [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp],
    "ipex_rwkv_time_shift": [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp],
    "ipex_rope_inplace": [vp, vp, vp, vp, ci, ci, ci, ci, ci, i64, i64, i64, i64, i64, i64, i64, i64, ci, ci, ci, vp],
    "ipex_kv_quant_e5m2": [vp, vp, i64, ci, i64, ci, vp],
    "ipex_kv_dequant_e5m2": [vp, vp, i64, ci, i64, ci, vp],
    "ipex_repetition_penalty": [vp, vp, ci, ci, ci, cf, ci, vp],
    "ipex_embedding": [vp, vp, vp, i64, ci, cf, ci, ci, vp],
    "ipex_argmax": [vp, vp, ci, ci, i64, ci, ci, vp],
    "ipex_attn_decode": [vp, vp, vp, vp, vp, vp, vp, ci, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, ci,
                         cf, cf, ci, ci, ci, vp],
    "ipex_quantize_to_tiles": [vp, vp, i64, i64, i64, ci, ci, ci, vp],
    "ipex_dequantize_tiles": [vp, vp, i64, i64, i64, ci, vp, ci, vp],
    "ipex_dequantize_blocks": [vp, vp, i64, ci, ci, ci, ci, vp],
    "ipex_dequantize_rows": [vp, vp, vp, i64, ci, ci, ci, ci, ci, vp],
}

_I64_RET = {
    "ipex_attn_decode_scratch_floats": [ci, ci, ci, ci, ci, ci],
    "ipex_attn_decode_counter_ints": [ci, ci, ci, ci],
}

# optional entry points: declared when the library exports them (kernels added over time)
_OPTIONAL = {
    "ipex_gemm_tcgen05": [vp, vp, vp, vp, vp, ci, ci, ci, i64, i64, i64, i64, ci, vp, vp],
    "ipex_gemm_tcgen05_token_tile": [ci],
    "ipex_gemm_lowbit_tcgen05": [vp, vp, vp, vp, vp, vp, ci, ci, ci, i64, i64, i64, ci, ci, ci, vp, vp],
    "ipex_gemm_lowbit_tcgen05_grouped": [vp, vp, vp, vp, vp, ci, ci, ci, ci, i64, i64, ci, ci, ci, ci, vp, vp],
    "ipex_lora_rs_adamw": [vp, vp, vp, vp, vp, vp, vp, vp, i64, ci, ci, cf, cf, cf, cf, cf, ci, ci, ci, vp, vp],
    "ipex_moe_softmax_topk": [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp],
}


def declare(lib: ctypes.CDLL):
    for name, args in _SIGS.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ci
    for name, args in _I64_RET.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = i64
    lib.ipex_gemv_tma_tune.argtypes = [ci, ci, ci]
    lib.ipex_gemv_tma_tune.restype = None
    for name, args in _OPTIONAL.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = ci


_CUDA_ERRORS = {1: "invalid value", 2: "out of memory", 98: "invalid device function", 700: "illegal address",
                701: "launch out of resources", 715: "illegal instruction", 719: "launch failure"}


def check(code: int, what: str):
    if code != 0:
        raise RuntimeError(f"ipex_llm_b200 CUDA kernel '{what}' failed: cudaError {code} "
                           f"({_CUDA_ERRORS.get(code, 'see cuda_runtime_api.h')})")


def dtype_code(torch_dtype) -> int:
    import torch
    if torch_dtype == torch.float16:
        return DT_F16
    if torch_dtype == torch.bfloat16:
        return DT_BF16
    if torch_dtype == torch.float32:
        return DT_F32
    raise TypeError(f"unsupported activation dtype {torch_dtype}")
