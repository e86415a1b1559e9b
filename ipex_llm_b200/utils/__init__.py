"""Utilities (reference: python/llm/src/ipex_llm/utils/)."""
from .common import invalidInputError, invalidOperationError  # noqa: F401


def __getattr__(name):
    if name == "BenchmarkWrapper":
        from .benchmark_util import BenchmarkWrapper
        return BenchmarkWrapper
    raise AttributeError(name)
