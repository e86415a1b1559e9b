"""GGUF import (reference package python/llm/src/ipex_llm/transformers/gguf/__init__.py: ``load_gguf_model``)."""
from .api import load_gguf_model  # noqa: F401
