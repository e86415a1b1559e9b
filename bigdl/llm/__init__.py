"""``bigdl.llm`` -> ``ipex_llm`` (-> ``ipex_llm_b200``), sub-modules included."""
import importlib
import importlib.abc
import importlib.util
import sys

import ipex_llm_b200 as _impl

_ALIAS, _TARGET = "bigdl.llm", "ipex_llm_b200"


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    _specs = {}

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        real = _TARGET + fullname[len(_ALIAS):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        mod = importlib.import_module(_TARGET + spec.name[len(_ALIAS):])
        self._specs[id(mod)] = mod.__spec__
        return mod

    def exec_module(self, module):
        real = self._specs.get(id(module))
        if real is not None:
            module.__spec__ = real


if not any(isinstance(f, _Finder) for f in sys.meta_path):
    sys.meta_path.insert(0, _Finder())

optimize_model = _impl.optimize_model


def __getattr__(name):
    return getattr(_impl, name)
