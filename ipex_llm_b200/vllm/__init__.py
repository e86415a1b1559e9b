"""vLLM integration (reference: python/llm/src/ipex_llm/vllm/{xpu,cpu}/): load a model inside vLLM's workers with
this package's low-bit linears.  Imports of ``vllm`` are lazy so the rest of the package does not depend on it."""
