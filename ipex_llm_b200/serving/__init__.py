"""HTTP serving: ``FastApp`` over a ``ModelWorker`` (single GPU / tensor parallel) or ``PPModelWorker``
(pipeline parallel).  Reference: python/llm/src/ipex_llm/serving/fastapi/."""


def __getattr__(name):
    if name in ("ModelWorker", "SamplingParams", "ServingRequest"):
        from . import model_worker
        return getattr(model_worker, name)
    if name == "FastApp":
        from .api_server import FastApp
        return FastApp
    if name in ("PPModelWorker", "BatchTask"):
        from . import pp_worker
        return getattr(pp_worker, name)
    raise AttributeError(name)
