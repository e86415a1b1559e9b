"""Reference module path ``ipex_llm.utils.lazy_load_torch``: the pieces of ``low_memory_init``
(python/llm/src/ipex_llm/optimize.py:124-134).  ``LazyLoadTensors`` / ``DisableTorchAllocTensor`` here are the
same meta-device context the package's ``low_memory_init`` uses."""
from ..optimize import low_memory_init


class DisableTorchAllocTensor:
    """Context in which module constructors allocate nothing (parameters land on the meta device)."""

    def __init__(self):
        self._ctx = low_memory_init()

    def __enter__(self):
        return self._ctx.__enter__()

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)


LazyLoadTensors = DisableTorchAllocTensor
