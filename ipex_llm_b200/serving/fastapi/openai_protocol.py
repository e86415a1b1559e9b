"""Reference module path ``ipex_llm.serving.fastapi.openai_protocol`` (python/llm/src/ipex_llm/serving/fastapi/openai_protocol.py): the OpenAI request and response schemas."""
from ..protocol import *  # noqa: F401,F403
