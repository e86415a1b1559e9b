"""LlamaIndex integration (reference: python/llm/src/ipex_llm/llamaindex/llms/bigdlllm.py, ``IpexLLM``)."""
