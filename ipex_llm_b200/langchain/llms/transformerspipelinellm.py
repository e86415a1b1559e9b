"""Reference module path ``ipex_llm.langchain.llms.transformerspipelinellm``
(python/llm/src/ipex_llm/langchain/llms/transformerspipelinellm.py:63)."""
from .transformersllm import TransformersPipelineLLM  # noqa: F401
