"""LangChain embeddings over the llama-cpp-python style classes.

Counterpart of python/llm/src/ipex_llm/langchain/embeddings/bigdlllm.py:58-385: ``BigdlNativeEmbeddings`` and the
per-family ``LlamaEmbeddings`` / ``BloomEmbeddings`` / ``GptneoxEmbeddings`` / ``StarcoderEmbeddings``; a text's
embedding is the mean of the last hidden states (``GenericModel.embed``)."""
from __future__ import annotations

from typing import List, Optional


class _BaseEmbeddings:
    ggml_family: Optional[str] = None

    def __init__(self, model_path: str = None, model_family: str = None, client=None, n_ctx: int = 512, seed: int = -1,
                 n_threads: Optional[int] = 2, n_batch: int = 512, low_bit: str = "sym_int4", device: str = "auto",
                 **kwargs):
        from ..llms.bigdlllm import _native_class
        self.model_family = model_family or type(self).ggml_family or "llama"
        self.model_path, self.n_ctx, self.n_threads, self.n_batch = model_path, n_ctx, n_threads, n_batch
        if client is None:
            if not model_path:
                raise ValueError("model_path is required")
            client = _native_class(self.model_family)(model_path, n_ctx=n_ctx, n_threads=n_threads, seed=seed,
                                                      n_batch=n_batch, embedding=True, low_bit=low_bit, device=device)
        self.client = client

    def embed_documents(self, texts: List[str]) -> List[List[float]]:
        return [list(map(float, self.client.embed(t))) for t in texts]

    def embed_query(self, text: str) -> List[float]:
        return list(map(float, self.client.embed(text)))


class BigdlNativeEmbeddings(_BaseEmbeddings):
    """``BigdlNativeEmbeddings(model_family="llama", model_path=...)``."""


class LlamaEmbeddings(_BaseEmbeddings):
    ggml_family = "llama"


class BloomEmbeddings(_BaseEmbeddings):
    ggml_family = "bloom"


class GptneoxEmbeddings(_BaseEmbeddings):
    ggml_family = "gptneox"


class StarcoderEmbeddings(_BaseEmbeddings):
    ggml_family = "starcoder"


__all__ = ["BigdlNativeEmbeddings", "LlamaEmbeddings", "BloomEmbeddings", "GptneoxEmbeddings", "StarcoderEmbeddings"]
