"""Reference module path ``ipex_llm.transformers.convert_ipex`` (``BIGDL_OPT_IPEX=true``: Intel Extension for
PyTorch CPU optimisations + TorchScript tracing, python/llm/src/ipex_llm/transformers/convert_ipex.py:54-382).
That path is specific to Intel CPUs and has no counterpart on this hardware; the entry point says so."""
from ..utils.common import invalidInputError


def _ipex_optimize_model(model, *args, **kwargs):
    invalidInputError(False, "BIGDL_OPT_IPEX: the IPEX CPU path is not available in this build; "
                             "use optimize_model(model) instead")


def _ipex_jit(model):
    return _ipex_optimize_model(model)
