"""Reference module path ``ipex_llm.ggml.model.llama`` (python/llm/src/ipex_llm/ggml/model/llama/__init__.py): the
``Llama`` class.  Every family runs on the one runtime of this package; see ``generic.py``."""
from .generic import Llama  # noqa: F401
