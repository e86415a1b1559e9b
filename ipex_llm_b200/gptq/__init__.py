"""Reference package path ``ipex_llm.gptq`` (GPTQ -> ggml converter of the legacy native flow)."""
