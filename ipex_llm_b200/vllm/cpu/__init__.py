"""Reference package path ``ipex_llm.vllm.cpu`` (the host flavour of the vLLM integration)."""
