"""ipex_llm_b200 — a Blackwell (B200, sm_100a) native low-bit LLM library with the public API of ipex-llm.

``import ipex_llm`` resolves to this package (see the ``ipex_llm`` alias package at the repository root), so
code written against the reference (``from ipex_llm import optimize_model``,
``from ipex_llm.transformers import AutoModelForCausalLM``) runs unchanged.
"""
from __future__ import annotations

import logging as _logging

__version__ = "0.1.0"

_logging.getLogger("ipex_llm").addHandler(_logging.NullHandler())

import os as _os  # noqa: E402

if _os.environ.get("BIGDL_GLIBC_CHECK", "False").lower() in ("1", "true", "yes"):
    from .utils.glibc_checker import check_glibc_version as _check_glibc_version
    _check_glibc_version()

from .optimize import load_low_bit, low_memory_init, optimize_model  # noqa: E402,F401

_LAZY = {
    "llm_patch": ("ipex_llm_b200.llm_patching", "llm_patch"),
    "llm_unpatch": ("ipex_llm_b200.llm_patching", "llm_unpatch"),
    "llm_convert": ("ipex_llm_b200.convert_model", "llm_convert"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'ipex_llm_b200' has no attribute {name!r}")
