from .vllm import VLLM, VLLMOpenAI  # noqa: F401
