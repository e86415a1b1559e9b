"""Reference module path ``ipex_llm.serving.fastapi.api_server`` (python/llm/src/ipex_llm/serving/fastapi/api_server.py): ``FastApp``."""
from ..api_server import *  # noqa: F401,F403
from ..api_server import FastApp  # noqa: F401
