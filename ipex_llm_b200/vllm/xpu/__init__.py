"""Reference package path ``ipex_llm.vllm.xpu`` (the accelerator flavour of the vLLM integration)."""
