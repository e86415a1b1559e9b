"""``ipex_llm`` — import-name alias of ``ipex_llm_b200``.

Programs written for the reference library import ``ipex_llm`` and ``ipex_llm.transformers``; this package
makes those names resolve to the B200-native implementation, sub-modules included
(``ipex_llm.transformers.qlora``, ``ipex_llm.optimize``, ``ipex_llm.serving.fastapi`` ...).
"""
import importlib
import importlib.abc
import importlib.util
import sys

import ipex_llm_b200 as _impl

_ALIAS = "ipex_llm"
_TARGET = "ipex_llm_b200"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname == _ALIAS or not fullname.startswith(_ALIAS + "."):
            return None
        real = _TARGET + fullname[len(_ALIAS):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        real = _TARGET + spec.name[len(_ALIAS):]
        mod = importlib.import_module(real)
        self._orig_specs[spec.name] = (mod.__spec__, getattr(mod, "__loader__", None))
        return mod

    def exec_module(self, module):
        # the import system stamped the alias spec on the shared module object: put the real one back
        for name, (spec, loader) in list(self._orig_specs.items()):
            if sys.modules.get(spec.name) is module:
                module.__spec__ = spec
                if loader is not None:
                    module.__loader__ = loader
                self._orig_specs.pop(name, None)

    _orig_specs = {}


sys.meta_path.insert(0, _AliasFinder())
__version__ = _impl.__version__
from ipex_llm_b200 import *  # noqa: E402,F401,F403
from ipex_llm_b200 import load_low_bit, low_memory_init, optimize_model  # noqa: E402,F401


def __getattr__(name):
    return getattr(_impl, name)
