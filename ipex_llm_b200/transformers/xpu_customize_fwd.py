"""Autocast helpers for custom autograd functions (reference: python/llm/src/ipex_llm/transformers/
xpu_customize_fwd.py:137-192, a copy of ``torch.cuda.amp.custom_fwd / custom_bwd`` for the "xpu" device).  On CUDA the
stock decorators do the job; the names are kept so that code written against the reference imports unchanged."""
from __future__ import annotations

import functools

import torch


def custom_fwd(fwd=None, *, cast_inputs=None):
    if fwd is None:
        return functools.partial(custom_fwd, cast_inputs=cast_inputs)
    return torch.amp.custom_fwd(fwd, device_type="cuda", cast_inputs=cast_inputs)


def custom_bwd(bwd):
    return torch.amp.custom_bwd(bwd, device_type="cuda")
