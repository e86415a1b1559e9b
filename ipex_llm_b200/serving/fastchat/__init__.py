"""FastChat-protocol model worker (reference: python/llm/src/ipex_llm/serving/fastchat/)."""
