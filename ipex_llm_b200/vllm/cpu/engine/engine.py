"""Reference module path ``ipex_llm.vllm.cpu.engine.engine`` (python/llm/src/ipex_llm/vllm/cpu/engine/engine.py): the engine classes with ``load_in_low_bit``."""
from ... import engine as _engine
from ...engine import run_mp_engine  # noqa: F401


def __getattr__(name):
    return getattr(_engine, name)
