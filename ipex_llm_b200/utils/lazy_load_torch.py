"""Lazy checkpoint tensors and the allocation-free construction context.

Counterpart of python/llm/src/ipex_llm/utils/lazy_load_torch.py:24-194 (``LazyStorage`` / ``LazyTensor`` /
``lazyload`` / ``LazyLoadTensors``) and of the pieces of ``low_memory_init`` (python/llm/src/ipex_llm/optimize.py:
124-134).  The reference re-implements the zip + pickle reader so that a tensor's bytes are read from the archive only
when ``LazyTensor.load()`` is called.  PyTorch's own loader can map the archive into memory (``torch.load(...,
mmap=True)``): storages then are file-backed pages that the kernel reads on first touch, which is the same laziness
with no second unpickler to maintain.  So here

* ``lazyload(path)`` returns ``{name: LazyTensor}`` over a memory-mapped checkpoint; nothing is read until
  ``load()``, and ``to(dtype)`` stacks a conversion that runs at load time;
* ``LazyLoadTensors`` is a context in which plain ``torch.load`` calls on zip checkpoints are memory-mapped;
* ``DisableTorchAllocTensor`` is the context in which module constructors allocate nothing.
"""
from __future__ import annotations

import os
import zipfile
from typing import Callable, Dict

import torch

from ..optimize import low_memory_init


class DisableTorchAllocTensor:
    """Context in which module constructors allocate nothing (parameters land on the meta device)."""

    def __init__(self):
        self._ctx = low_memory_init()

    def __enter__(self):
        return self._ctx.__enter__()

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)


class LazyTensor:
    """A tensor of a checkpoint that has not been read yet."""

    def __init__(self, load: Callable[[], torch.Tensor], shape, data_type: torch.dtype, description: str = ""):
        self._load, self.shape, self.data_type, self.description = load, list(shape), data_type, description

    def load(self) -> torch.Tensor:
        t = self._load()
        if t.dtype != self.data_type:
            raise RuntimeError(f"{self.description}: expected {self.data_type}, the checkpoint holds {t.dtype}")
        return t

    def to(self, data_type: torch.dtype) -> "LazyTensor":
        """The same tensor converted at load time."""
        return LazyTensor(lambda: self._load().to(data_type), self.shape, data_type,
                          f"{self.description} -> {data_type}")

    def __repr__(self):
        return f"LazyTensor({self.description or '?'}, shape={self.shape}, dtype={self.data_type})"


def _is_zip_checkpoint(f) -> bool:
    return isinstance(f, (str, os.PathLike)) and os.path.isfile(f) and zipfile.is_zipfile(f)


def _mapped_load(f, map_location=None, **kwargs):
    kwargs.setdefault("weights_only", True)
    return torch.load(f, map_location=map_location or "cpu", mmap=True, **kwargs)


def lazyload(f, *args, **kwargs) -> Dict[str, LazyTensor]:
    """``{name: LazyTensor}`` for a checkpoint written by ``torch.save`` (zip format).  Non-tensor entries are returned
    as they are."""
    if not _is_zip_checkpoint(f):
        raise ValueError(f"{f}: lazy loading needs a zip-format torch checkpoint on disk")
    mapped = _mapped_load(f, kwargs.get("map_location"))

    def wrap(name, value):
        if isinstance(value, torch.Tensor):
            return LazyTensor(lambda v=value: v.clone(), value.shape, value.dtype, f"{os.path.basename(str(f))}:{name}")
        if isinstance(value, dict):
            return {k: wrap(f"{name}.{k}", v) for k, v in value.items()}
        return value
    return {k: wrap(k, v) for k, v in mapped.items()}


class LazyLoadTensors:
    """Inside the context ``torch.load`` of a zip checkpoint maps the file instead of reading it: peak host memory is
    what the caller touches, not the checkpoint size."""

    def __init__(self):
        self._orig = None

    def __enter__(self):
        self._orig = torch.load
        orig = self._orig

        def load(f, *args, **kwargs):
            if _is_zip_checkpoint(f) and "mmap" not in kwargs:
                try:
                    return orig(f, *args, mmap=True, **kwargs)
                except (RuntimeError, ValueError):      # e.g. a map_location that cannot be combined with mmap
                    pass
            return orig(f, *args, **kwargs)
        torch.load = load
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        torch.load = self._orig
        self._orig = None
        return False
