"""``IPEXLLMClass`` / ``IPEXLLMAsyncLLMEngine`` / ``IPEXLLMLLMEngine``: vLLM's entry classes with a
``load_in_low_bit`` argument (reference: python/llm/src/ipex_llm/vllm/xpu/engine/engine.py:41-245)."""
from __future__ import annotations


def _convert(load_in_low_bit):
    from .model_convert import _ipex_llm_convert
    _ipex_llm_convert(load_in_low_bit)


def IPEXLLMClass(*args, load_in_low_bit: str = "sym_int4", **kwargs):
    """``vllm.LLM`` whose workers convert the model to ``load_in_low_bit`` after loading."""
    from vllm import LLM
    _convert(load_in_low_bit)
    return LLM(*args, **kwargs)


class IPEXLLMAsyncLLMEngine:
    @classmethod
    def from_engine_args(cls, engine_args, load_in_low_bit: str = "sym_int4", **kwargs):
        from vllm.engine.async_llm_engine import AsyncLLMEngine
        _convert(load_in_low_bit)
        return AsyncLLMEngine.from_engine_args(engine_args, **kwargs)


class IPEXLLMLLMEngine:
    @classmethod
    def from_engine_args(cls, engine_args, load_in_low_bit: str = "sym_int4", **kwargs):
        from vllm.engine.llm_engine import LLMEngine
        _convert(load_in_low_bit)
        return LLMEngine.from_engine_args(engine_args, **kwargs)
