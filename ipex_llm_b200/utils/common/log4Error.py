"""Reference module path python/llm/src/ipex_llm/utils/common/log4Error.py:22-53."""
from ..common_impl import MuteHFLogger, invalidInputError, invalidOperationError  # noqa: F401
