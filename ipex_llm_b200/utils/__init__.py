from .common import invalidInputError, invalidOperationError  # noqa: F401
