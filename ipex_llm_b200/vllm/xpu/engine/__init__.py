"""Reference module path ``ipex_llm.vllm.xpu.engine`` (python/llm/src/ipex_llm/vllm/xpu/engine/__init__.py)."""
from ... import engine as _engine


def __getattr__(name):
    return getattr(_engine, name)
