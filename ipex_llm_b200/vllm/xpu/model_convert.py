"""Reference module path ``ipex_llm.vllm.xpu.model_convert`` (python/llm/src/ipex_llm/vllm/xpu/model_convert.py:35-180)."""
from ..model_convert import *  # noqa: F401,F403
from ..model_convert import _ipex_llm_convert, convert_vllm_model  # noqa: F401
