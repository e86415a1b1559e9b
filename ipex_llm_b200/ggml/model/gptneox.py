"""Reference module path ``ipex_llm.ggml.model.gptneox`` (python/llm/src/ipex_llm/ggml/model/gptneox/__init__.py): the
``Gptneox`` class.  Every family runs on the one runtime of this package; see ``generic.py``."""
from .generic import Gptneox  # noqa: F401
