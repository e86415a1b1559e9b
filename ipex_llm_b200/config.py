"""One place for every environment flag the package honours.

The reference reads its switches ad hoc with ``os.environ`` all over the tree
(python/llm/src/ipex_llm/transformers/models/utils.py:77-99, 317-330; low_bit_linear.py:64, 613;
convert.py:73, 504).  The same names are honoured here, resolved lazily through one typed accessor so that
tests can monkeypatch the environment.
"""
from __future__ import annotations

import os


def _flag(name: str, default=None):
    v = os.environ.get(name)
    if v is None:
        return default
    return v


def env_bool(name: str, default=None):
    v = _flag(name)
    if v is None:
        return default
    return v.strip().lower() in ("1", "true", "yes", "on")


def env_int(name: str, default: int) -> int:
    v = _flag(name)
    return int(v) if v is not None else default


def quantize_kv_cache_flag():
    """IPEX_LLM_QUANTIZE_KV_CACHE (or deprecated BIGDL_QUANTIZE_KV_CACHE): True / False / None (=auto)."""
    v = env_bool("IPEX_LLM_QUANTIZE_KV_CACHE")
    if v is None:
        v = env_bool("BIGDL_QUANTIZE_KV_CACHE")
    return v


def kv_cache_format():
    """``"int4"`` when IPEX_LLM_QUANTIZE_KV_CACHE=int4 asks for the 4-bit cache (4.25 bits per element), else None
    (``"1"`` keeps meaning the e5m2 byte cache of the reference)."""
    v = _flag("IPEX_LLM_QUANTIZE_KV_CACHE")
    return "int4" if v is not None and v.strip().lower() == "int4" else None


def compress_kv_cache_flag():
    return env_bool("IPEX_LLM_COMPRESS_KV_CACHE")


def low_mem() -> bool:
    return bool(env_bool("IPEX_LLM_LOW_MEM", False))


def performance_mode() -> bool:
    return bool(env_bool("IPEX_LLM_PERFORMANCE_MODE", False))


def last_lm_head() -> bool:
    return _flag("IPEX_LLM_LAST_LM_HEAD", "1") != "0"


def fastapi_timeout() -> int:
    return env_int("IPEX_LLM_FASTAPI_TIMEOUT", 60)


def kv_alloc_block() -> int:
    return env_int("KV_CACHE_ALLOC_BLOCK_LENGTH", 256)


def linear_threshold() -> int:
    return env_int("BIGDL_LLM_LINEAR_THRESHOLD", 512)


def use_native_engine() -> bool:
    """IPEX_LLM_NATIVE_ENGINE=0 turns the CUDA-graph decode engine off (HF module path only)."""
    return _flag("IPEX_LLM_NATIVE_ENGINE", "1") != "0"


def nvtx_enabled() -> bool:
    return bool(env_bool("IPEX_LLM_NVTX", False))


ALL_FLAGS = [
    "IPEX_LLM_QUANTIZE_KV_CACHE", "BIGDL_QUANTIZE_KV_CACHE", "IPEX_LLM_LOW_MEM", "IPEX_LLM_COMPRESS_KV_CACHE",
    "IPEX_LLM_PERFORMANCE_MODE", "IPEX_LLM_LAST_LM_HEAD", "IPEX_LLM_CPU_LM_HEAD", "IPEX_LLM_NOT_USE_VLLM",
    "IPEX_LLM_NOT_CONVERT_LAST_MLP", "IPEX_LLM_FASTAPI_TIMEOUT", "KV_CACHE_ALLOC_BLOCK_LENGTH",
    "BIGDL_LLM_LINEAR_THRESHOLD", "BIGDL_OPT_IPEX", "BIGDL_IMPORT_IPEX", "BIGDL_USE_NPU", "BIGDL_COMPATIBLE_MODE",
    "BIGDL_CHECK_DUPLICATE_IMPORT", "BIGDL_GLIBC_CHECK", "IPEX_LLM_NATIVE_ENGINE", "IPEX_LLM_NVTX",
    "IPEX_LLM_REBUILD_NATIVE", "IPEX_LLM_TP_FUSED",
]
