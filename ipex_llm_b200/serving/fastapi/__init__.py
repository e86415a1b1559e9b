"""Import path of the reference (``ipex_llm.serving.fastapi``): ``FastApp``, ``ModelWorker``, ``PPModelWorker``."""
from ..api_server import FastApp  # noqa: F401
from ..model_worker import ModelWorker  # noqa: F401


def __getattr__(name):
    if name == "PPModelWorker":
        from ..pp_worker import PPModelWorker
        return PPModelWorker
    raise AttributeError(name)
