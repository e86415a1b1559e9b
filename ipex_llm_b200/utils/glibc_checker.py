"""glibc requirement of the native libraries (reference: python/llm/src/ipex_llm/utils/glibc_checker.py:25-63, env
``BIGDL_GLIBC_CHECK``).  The in-tree libraries are built on the machine that runs them, so the requirement that can
actually bite is the C++17 / OpenMP runtime baseline: glibc 2.28.  ``check_glibc_version()`` raises the usage error of
the reference when the running system is older; the package init calls it when ``BIGDL_GLIBC_CHECK`` is true."""
from __future__ import annotations

import os
import platform

from .common import invalidInputError


def _parse(v: str):
    return tuple(int(p) for p in v.split(".") if p.isdigit())


class GlibcChecker:
    def __init__(self, min_glibc_version: str):
        self.min_glibc_version = min_glibc_version

    @staticmethod
    def is_linux() -> bool:
        return platform.system() == "Linux"

    @staticmethod
    def get_glibc_version() -> str:
        try:
            return os.confstr("CS_GNU_LIBC_VERSION").split()[1]
        except (ValueError, OSError, AttributeError, IndexError):
            return platform.libc_ver()[1] or "0"

    def check_requirements(self):
        if not self.is_linux():
            return
        have = self.get_glibc_version()
        invalidInputError(_parse(have) >= _parse(self.min_glibc_version),
                          f"Detected glibc version: {have}. (required: >= {self.min_glibc_version}) "
                          "Please upgrade your operating system with a newer version of glibc.")


glibc_checker = GlibcChecker("2.28")


def check_glibc_version():
    glibc_checker.check_requirements()
