"""``LazyImport('pkg.mod.attr')``: a stand-in that imports on first use (reference:
python/llm/src/ipex_llm/utils/common/lazyimport.py:23-76).  The dotted name may end in a module or in an attribute of
one; attribute access and calls are forwarded to whatever it resolves to."""
import importlib


class LazyImport:
    def __init__(self, module_name: str):
        self.module_name = module_name
        self._target = None

    def _resolve(self):
        if self._target is None:
            try:
                self._target = importlib.import_module(self.module_name)
            except ImportError:
                parent, _, child = self.module_name.rpartition(".")
                if not parent:
                    raise
                self._target = getattr(importlib.import_module(parent), child)
        return self._target

    def __getattr__(self, name):
        return getattr(self._resolve(), name)

    def __call__(self, *args, **kwargs):
        return self._resolve()(*args, **kwargs)
