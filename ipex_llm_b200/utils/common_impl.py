"""Error helpers with the reference's user-facing banner
(python/llm/src/ipex_llm/utils/common/log4Error.py:22-53)."""
from __future__ import annotations

import logging

logger = logging.getLogger("ipex_llm")


def _banner(err_msg, fix_msg):
    msg = "\n\n****************************Usage Error************************\n" + str(err_msg)
    if fix_msg is not None:
        msg += "\n\n\n****************************How to fix*************************\n" + str(fix_msg)
    msg += "\n\n****************************Call Stack*************************"
    return msg


def invalidInputError(condition, errMsg, fixMsg=None):
    if not condition:
        logger.error(_banner(errMsg, fixMsg))
        raise RuntimeError(errMsg)


def invalidOperationError(condition, errMsg, fixMsg=None, cause=None):
    if not condition:
        logger.error(_banner(errMsg, fixMsg))
        if cause is not None:
            raise cause
        raise RuntimeError(errMsg)


class MuteHFLogger:
    """Silence a Hugging Face logger inside a ``with`` block."""

    def __init__(self, logger, speak_level=logging.ERROR):
        self.logger = logger
        self.speak_level = speak_level
        self.old_level = logger.level

    def __enter__(self):
        self.logger.setLevel(self.speak_level)

    def __exit__(self, exc_type, exc_value, traceback):
        self.logger.setLevel(self.old_level)
