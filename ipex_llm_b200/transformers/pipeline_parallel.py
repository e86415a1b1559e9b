"""Import location kept from the reference (``ipex_llm.transformers.pipeline_parallel``); the implementation
lives in ``ipex_llm_b200.parallel.pp`` (partitioning, generate) and ``ipex_llm_b200.serving.pp_worker``
(``PPModelWorker``)."""
from ..parallel.pp import (Dummy_DecoderLayer, init_pipeline_parallel, pipeline_parallel,  # noqa: F401
                           pipeline_parallel_generate, stage_layer_range)


def __getattr__(name):
    if name == "PPModelWorker":
        from ..serving.pp_worker import PPModelWorker
        return PPModelWorker
    raise AttributeError(name)
