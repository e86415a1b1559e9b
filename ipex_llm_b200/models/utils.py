"""Policy helpers used by the model forwards.

Counterparts of python/llm/src/ipex_llm/transformers/models/utils.py:34-353 of the reference
(``use_quantize_kv_cache``, ``should_use_compresskv``, ``mlp_fusion_check``, ``use_sdp*``, cache
allocators).  The Intel device-name heuristics are replaced by B200 ones: with 180 GB of HBM the fp8 KV
cache is a bandwidth optimisation, enabled by default on CUDA for batch <= 8 decode like the reference does
on its large GPUs, and always overridable by ``IPEX_LLM_QUANTIZE_KV_CACHE``.
"""
from __future__ import annotations

import torch

from .. import config as cfg
from ..ops.kv_cache import (DynamicCompressCache, DynamicCompressFp8Cache, DynamicFp8Cache, DynamicInt4Cache,
                            DynamicNormalCache)
from ..quant import qtypes as qt

FP8_KV_ALLOC_LENGTH = 512


def decoding_fast_path_qtype_check(proj) -> bool:
    qtype = getattr(proj, "qtype", None)
    return qtype in (qt.SYM_INT4, qt.FP8E5, qt.FP4, qt.WOQ_INT4)


def use_quantize_kv_cache(linear, x: torch.Tensor, num_heads: int = 1, num_kv_heads: int = 1) -> bool:
    """fp8 (e5m2) KV cache on/off.  Env flag wins; otherwise on for CUDA inference with batch <= 8."""
    flag = cfg.quantize_kv_cache_flag()
    if flag is not None:
        return flag
    if cfg.low_mem():
        return True
    if x.device.type != "cuda" or x.requires_grad:
        return False
    return 1 <= x.size(0) <= 8 and num_kv_heads * 2 >= 1


def should_use_compresskv(x: torch.Tensor, prompt_len: int) -> bool:
    """SnapKV only when asked for (IPEX_LLM_COMPRESS_KV_CACHE=1) and the prompt is in [1800, 4500] tokens when
    the flag is unset but performance mode is on (reference models/utils.py:317-330)."""
    flag = cfg.compress_kv_cache_flag()
    if flag is not None:
        return flag and x.size(0) == 1
    return False


def get_compresskv_attn_mask(key_states: torch.Tensor, attention_mask: torch.Tensor):
    if attention_mask is not None:
        return attention_mask[:, :, :, -key_states.size(2):]
    return attention_mask


def mlp_fusion_check(x: torch.Tensor, qtype: int, training: bool) -> bool:
    """Single-token decode with a qtype whose fused gate/up kernel exists (reference models/utils.py:246-259)."""
    if x.numel() // x.size(-1) != 1:
        return False
    if x.device.type != "cuda":
        return False
    if qtype not in (qt.SYM_INT4, qt.FP8E5, qt.FP4, qt.FP6, qt.WOQ_INT4, qt.FP8E4, qt.NF4, qt.ASYM_INT4):
        return False
    if training or x.requires_grad:
        return False
    return True


def use_sdp(q_len: int, kv_len: int, head_dim: int, query_states: torch.Tensor) -> bool:
    return query_states.device.type == "cuda" and head_dim in (64, 80, 96, 128, 192, 256) and q_len != kv_len \
        and q_len <= 32


def use_sdp_causal(q_len: int, kv_len: int, head_dim: int, query_states: torch.Tensor, training: bool) -> bool:
    return q_len == kv_len and head_dim in (-1, 64, 80, 96, 128) and query_states.device.type == "cuda" \
        and not query_states.requires_grad and not training


def select_cache(config, hidden_states: torch.Tensor, past_key_values, probe_linear=None, prompt_len=None):
    """Pick (or keep) the KV-cache class for this generation, mirroring llama_model_forward's choice
    (reference models/llama.py:69-95): compress > fp8 > normal."""
    n_heads = getattr(config, "num_attention_heads", 1)
    n_kv = getattr(config, "num_key_value_heads", None) or n_heads
    use_quantize = use_quantize_kv_cache(probe_linear, hidden_states, n_heads, n_kv)
    prompt_len = prompt_len if prompt_len is not None else hidden_states.shape[1]
    use_compress = should_use_compresskv(hidden_states, prompt_len)
    fresh = past_key_values is None or (past_key_values.get_seq_length() == 0
                                        and type(past_key_values).__name__ == "DynamicCache")
    if not fresh:
        return past_key_values
    if use_compress:
        return DynamicCompressFp8Cache(config) if use_quantize else DynamicCompressCache(config)
    if cfg.kv_cache_format() == "int4":
        return DynamicInt4Cache(config)
    if use_quantize:
        return DynamicFp8Cache(config)
    return DynamicNormalCache(config)
