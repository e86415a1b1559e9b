"""``BenchmarkWrapper``: wraps a model and reports first-token / next-token latency of every ``generate`` call.

The reference ships per-``transformers``-version copies of the whole HF ``generate`` loop with timers inside
(python/llm/src/ipex_llm/utils/benchmark_util_4_47.py and siblings).  Here timing is taken from outside the loop:
the native engine, the speculative / lookup loops and the pipeline loop publish ``first_token_time`` /
``rest_cost_mean`` themselves; for the stock HF loop a stopping criterion (called once per generated token, after
the forward and the sampling of that token) records device-synchronised timestamps.

Attributes after a call (same names as the reference): ``first_cost``, ``rest_cost_mean``, ``encoder_time``,
``peak_memory`` (GiB), and ``first_token_time`` as an alias.
"""
from __future__ import annotations

import time

import torch


class _StepTimer:
    """Callable with the ``StoppingCriteria`` signature; never stops anything."""

    def __init__(self, device):
        self.device = device
        self.stamps = []

    def __call__(self, input_ids, scores, **kwargs):
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.stamps.append(time.perf_counter())
        return torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)


class BenchmarkWrapper:
    def __init__(self, model, do_print: bool = False, verbose: bool = False):
        self.model = model
        self.do_print = do_print
        self.verbose = verbose
        self.encoder_time = 0.0
        self.first_cost = 0.0
        self.rest_cost_mean = 0.0
        self.peak_memory = 0.0
        print_fn = getattr(model, "__class__", type(model)).__name__
        self._name = print_fn

    def __getattr__(self, attr):
        return getattr(self.model, attr)

    def __call__(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    @property
    def first_token_time(self):
        return self.first_cost

    def generate(self, *args, **kwargs):
        model = self.model
        dev = next(model.parameters()).device
        for a in ("first_token_time", "rest_cost_mean"):
            if hasattr(model, a):
                try:
                    delattr(model, a)
                except AttributeError:
                    pass
        if dev.type == "cuda":
            torch.cuda.reset_peak_memory_stats(dev)
            torch.cuda.synchronize(dev)
        timer = _StepTimer(dev)
        t0 = time.perf_counter()
        out = model.generate(*args, **kwargs)
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        t_end = time.perf_counter()
        first = getattr(model, "first_token_time", None)
        rest = getattr(model, "rest_cost_mean", None)
        if first is None:
            # the loop published nothing: run once more with the per-token timer attached
            from transformers import StoppingCriteriaList
            sc = kwargs.pop("stopping_criteria", None)
            crit = StoppingCriteriaList(list(sc or []) + [timer])
            t0 = time.perf_counter()
            out = model.generate(*args, stopping_criteria=crit, **kwargs)
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            t_end = time.perf_counter()
            st = timer.stamps
            if st:
                first = st[0] - t0
                rest = (st[-1] - st[0]) / (len(st) - 1) if len(st) > 1 else 0.0
            else:
                first, rest = t_end - t0, 0.0
        self.first_cost = float(first)
        self.rest_cost_mean = float(rest or 0.0)
        if dev.type == "cuda":
            self.peak_memory = torch.cuda.max_memory_allocated(dev) / (1024 ** 3)
        if self.do_print:
            print(f"=========First token cost {self.first_cost:.4f} s and {self.peak_memory:.2f} GB=========")
            print(f"=========Rest tokens cost average {self.rest_cost_mean:.4f} s=========")
        return out
