"""Reference module path ``ipex_llm.ggml.model.chatglm`` (python/llm/src/ipex_llm/ggml/model/chatglm/__init__.py): the
``ChatGLM`` class.  Every family runs on the one runtime of this package; see ``generic.py``."""
from .generic import ChatGLM  # noqa: F401
