"""Reference module path ``ipex_llm.llamaindex.llms.bigdlllm`` (python/llm/src/ipex_llm/llamaindex/llms/bigdlllm.py:90)."""
from .ipexllm import ChatMessage, ChatResponse, CompletionResponse, IpexLLM  # noqa: F401
