"""Reference module path ``ipex_llm.vllm.cpu.engine`` (python/llm/src/ipex_llm/vllm/cpu/engine/engine.py): the same
engine classes serve every device here."""
from ... import engine as _engine


def __getattr__(name):
    return getattr(_engine, name)
