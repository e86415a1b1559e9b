"""Reference module path ``ipex_llm.transformers.embedding`` (``CPUEmbedding``, ``DiskEmbedding``,
``LowBitEmbedding``; python/llm/src/ipex_llm/transformers/embedding.py:29-241)."""
from ..ops import embedding as _e

globals().update({k: v for k, v in vars(_e).items() if not k.startswith("_")})
