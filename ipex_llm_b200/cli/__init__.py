"""Command-line tools: ``llm-cli`` / ``llm-chat`` (reference: python/llm/src/ipex_llm/cli/llm-cli, llm-chat, which
wrap native llama.cpp-style binaries) and ``llm-convert`` (``ipex_llm_b200.convert_model``)."""
