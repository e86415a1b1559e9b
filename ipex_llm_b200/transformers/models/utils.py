"""Reference module path ``ipex_llm.transformers.models.utils`` (policy helpers,
python/llm/src/ipex_llm/transformers/models/utils.py:34-353)."""
from ...models import utils as _u

globals().update({k: v for k, v in vars(_u).items() if not k.startswith("_")})
