"""Reference module path ``ipex_llm.ggml.model.bloom`` (python/llm/src/ipex_llm/ggml/model/bloom/__init__.py): the
``Bloom`` class.  Every family runs on the one runtime of this package; see ``generic.py``."""
from .generic import Bloom  # noqa: F401
