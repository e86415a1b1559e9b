"""Reference module path ``ipex_llm.vllm.cpu.model_convert`` (CPU twin of the vLLM integration)."""
from ..model_convert import *  # noqa: F401,F403
from ..model_convert import _ipex_llm_convert, convert_vllm_model  # noqa: F401
