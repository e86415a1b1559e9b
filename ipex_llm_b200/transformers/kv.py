"""Reference module path ``ipex_llm.transformers.kv`` (``DynamicNormalCache``, ``DynamicFp8Cache``,
``DynamicCompressCache``, ``DynamicCompressFp8Cache``; python/llm/src/ipex_llm/transformers/kv.py:32-449)."""
from ..ops import kv_cache as _kv

globals().update({k: v for k, v in vars(_kv).items() if not k.startswith("_")})
