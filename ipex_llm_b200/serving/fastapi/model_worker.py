"""Reference module path ``ipex_llm.serving.fastapi.model_worker`` (python/llm/src/ipex_llm/serving/fastapi/model_worker.py): ``ModelWorker``."""
from ..model_worker import *  # noqa: F401,F403
from ..model_worker import ModelWorker  # noqa: F401
