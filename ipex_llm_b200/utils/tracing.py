"""Tracing hooks: NVTX ranges behind ``IPEX_LLM_NVTX=1`` and a ``torch.profiler`` wrapper for one ``generate``.

The reference has no tracer integration; its profiling is wall-clock around ``generate`` with a device
synchronise (python/llm/src/ipex_llm/utils/benchmark_util_4_47.py:3300, 3372-3381) and per-phase timers of the
speculative and pipeline loops.  Those timers exist here too (``first_token_time``, ``rest_cost_mean``,
``draft_time`` ...); this module adds named ranges that show up in Nsight timelines and a profiler table, both
off unless asked for so that the graph-replayed decode loop pays nothing.
"""
from __future__ import annotations

import contextlib

import torch

from .. import config as cfg


@contextlib.contextmanager
def nvtx_range(name: str):
    """``with nvtx_range("prefill"): ...`` — a named range when ``IPEX_LLM_NVTX=1`` on a CUDA machine, else free."""
    on = cfg.nvtx_enabled() and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def profile_generate(model, input_ids, sort_by: str = None, row_limit: int = 25, **generate_kwargs):
    """Run one ``model.generate`` under ``torch.profiler`` and return ``(output_ids, table_string)``.  The table
    lists device kernels by total time on CUDA models (host ops on CPU models)."""
    from torch.profiler import ProfilerActivity, profile
    acts = [ProfilerActivity.CPU]
    on_cuda = next(model.parameters()).is_cuda
    if on_cuda:
        acts.append(ProfilerActivity.CUDA)
    with profile(activities=acts) as prof:
        out = model.generate(input_ids, **generate_kwargs)
        if on_cuda:
            torch.cuda.synchronize()
    key = sort_by or ("cuda_time_total" if on_cuda else "cpu_time_total")
    return out, prof.key_averages().table(sort_by=key, row_limit=row_limit)
