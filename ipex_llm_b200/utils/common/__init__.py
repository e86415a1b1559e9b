"""``ipex_llm.utils.common``: error helpers (package form, as in the reference, with ``log4Error`` inside)."""
from ..common_impl import MuteHFLogger, invalidInputError, invalidOperationError, logger  # noqa: F401
from .lazyimport import LazyImport  # noqa: E402,F401
