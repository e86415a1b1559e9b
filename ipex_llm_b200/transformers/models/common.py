"""Reference module path ``ipex_llm.transformers.models.common`` (fused-op facade,
python/llm/src/ipex_llm/transformers/models/common.py:22-305)."""
from ...models import common as _c

globals().update({k: v for k, v in vars(_c).items() if not k.startswith("_")})
