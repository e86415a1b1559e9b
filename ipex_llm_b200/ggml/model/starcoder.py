"""Reference module path ``ipex_llm.ggml.model.starcoder`` (python/llm/src/ipex_llm/ggml/model/starcoder/__init__.py): the
``Starcoder`` class.  Every family runs on the one runtime of this package; see ``generic.py``."""
from .generic import Starcoder  # noqa: F401
