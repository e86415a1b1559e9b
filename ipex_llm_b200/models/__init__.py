"""Per-family forward replacements (``registry``, ``decoder``, ``common``, ``utils``).

The reference also uses the name ``ipex_llm.models`` as the short import path of its native model classes
(python/llm/src/ipex_llm/models.py:22-27: ``from ipex_llm.models import Llama, Bloom, Gptneox, Starcoder``); those
names resolve here too, lazily."""


def __getattr__(name):
    if name in ("Llama", "Bloom", "Gptneox", "Starcoder", "ChatGLM"):
        from ..ggml import model as _native
        return getattr(_native, name)
    raise AttributeError(name)
