"""Low-bit type registry.

Name -> integer id table with the same names and ids as the reference
(python/llm/src/ipex_llm/ggml/quantize.py:28-61), so that ``config.json`` files written by
``save_low_bit`` (key ``bigdl_transformers_low_bit``) stay interchangeable.
"""
from __future__ import annotations

ggml_tensor_qtype = {
    "sym_int4": 2,      # q4_0, block 64
    "asym_int4": 3,     # q4_1, block 64
    "sym_int5": 6,      # q5_0
    "asym_int5": 7,     # q5_1
    "sym_int8": 8,      # q8_0, block 64
    "nf4": 10,
    "nf3": 11,
    "fp16": 12,
    "fp8_e4m3": 15,
    "fp4": 16,
    "mixed_fp4": 17,    # picks sym_int4 or fp4 per tensor by MSE
    "mixed_fp8": 18,    # picks sym_int8 or fp8_e4m3 per tensor by MSE
    "fp8_e5m2": 19,
    "fp8": 19,          # alias of fp8_e5m2
    "bf16": 20,
    "gguf_iq2_xxs": 21,
    "gguf_iq2_xs": 22,
    "q2_k": 23,
    "gguf_iq1_s": 24,
    "gguf_iq1_m": 25,
    "q6_k": 26,
    "q4_k": 27,
    "q5_k": 28,
    "fp6": 29,
    "fp6_k": 30,
    "sym_int4_rtn": 31,
    "sym_int8_rtn": 32,
    "asym_int4_rtn": 33,
    "woq_int4": 34,
}

# mixed gguf presets (per-layer qtype policy, see quant/policy.py)
gguf_mixed_qtype = {"gguf_q4k_s": 101, "gguf_q4k_m": 102}

_id_to_name = {}
for _k, _v in ggml_tensor_qtype.items():
    _id_to_name.setdefault(_v, _k)

SYM_INT4 = ggml_tensor_qtype["sym_int4"]
ASYM_INT4 = ggml_tensor_qtype["asym_int4"]
SYM_INT5 = ggml_tensor_qtype["sym_int5"]
ASYM_INT5 = ggml_tensor_qtype["asym_int5"]
SYM_INT8 = ggml_tensor_qtype["sym_int8"]
NF4 = ggml_tensor_qtype["nf4"]
NF3 = ggml_tensor_qtype["nf3"]
FP16 = ggml_tensor_qtype["fp16"]
FP8E4 = ggml_tensor_qtype["fp8_e4m3"]
FP4 = ggml_tensor_qtype["fp4"]
MOFQ4 = ggml_tensor_qtype["mixed_fp4"]
MOFQ8 = ggml_tensor_qtype["mixed_fp8"]
FP8E5 = ggml_tensor_qtype["fp8_e5m2"]
BF16 = ggml_tensor_qtype["bf16"]
IQ2_XXS = ggml_tensor_qtype["gguf_iq2_xxs"]
IQ2_XS = ggml_tensor_qtype["gguf_iq2_xs"]
Q2_K = ggml_tensor_qtype["q2_k"]
IQ1_S = ggml_tensor_qtype["gguf_iq1_s"]
IQ1_M = ggml_tensor_qtype["gguf_iq1_m"]
Q6_K = ggml_tensor_qtype["q6_k"]
Q4_K = ggml_tensor_qtype["q4_k"]
Q5_K = ggml_tensor_qtype["q5_k"]
FP6 = ggml_tensor_qtype["fp6"]
FP6_K = ggml_tensor_qtype["fp6_k"]
SYM_INT4_RTN = ggml_tensor_qtype["sym_int4_rtn"]
SYM_INT8_RTN = ggml_tensor_qtype["sym_int8_rtn"]
ASYM_INT4_RTN = ggml_tensor_qtype["asym_int4_rtn"]
WOQ_INT4 = ggml_tensor_qtype["woq_int4"]

# qtypes whose block codec is implemented by the host library and the CUDA kernels
BLOCK_QTYPES = (SYM_INT4, ASYM_INT4, SYM_INT5, ASYM_INT5, SYM_INT8, NF4, NF3, FP4, FP6, FP6_K,
                FP8E4, FP8E5, Q2_K, Q4_K, Q5_K, Q6_K, WOQ_INT4)
# code-book super-blocks: codecs in quant/iq_codebooks.py, grids from the `gguf` package at run time
IQ_QTYPES = (IQ2_XXS, IQ2_XS, IQ1_S, IQ1_M)
UNSUPPORTED_QTYPES = ()
# qtypes whose device layout is the tensor-core tile layout (fast GEMV / GEMM kernels)
TILED_4BIT = (SYM_INT4, ASYM_INT4, NF4, FP4)
TILED_8BIT = (FP8E4, FP8E5, SYM_INT8)
FLOAT_QTYPES = (FP16, BF16)


def qtype_name(qtype: int) -> str:
    return _id_to_name[qtype]


def qtype_from_name(name: str) -> int:
    if name in ggml_tensor_qtype:
        return ggml_tensor_qtype[name]
    if name in gguf_mixed_qtype:
        return gguf_mixed_qtype[name]
    raise ValueError(
        f"Unknown load_in_low_bit value: {name}, expected one of "
        f"{sorted(list(ggml_tensor_qtype) + list(gguf_mixed_qtype))}")
