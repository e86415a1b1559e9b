"""vLLM's entry classes with a ``load_in_low_bit`` argument.

Counterpart of python/llm/src/ipex_llm/vllm/xpu/engine/engine.py:40-245: ``IPEXLLMClass`` (``vllm.LLM``),
``IPEXLLMAsyncLLMEngine`` / ``IPEXLLMLLMEngine`` (the engine classes) and their V1 forms ``IPEXLLMAsyncV1Engine`` /
``IPEXLLMLLMV1Engine``.  Each is a real subclass of the installed vLLM class, created on first use because importing
vLLM costs tens of seconds; constructing one first installs the loader patches of ``model_convert`` for the requested
format and then defers to vLLM with every other argument untouched.

The patches live on classes of this process.  vLLM's V1 engine core normally runs in a child process that would import
those classes afresh, so unless the caller decided otherwise the core is kept in-process
(``VLLM_ENABLE_V1_MULTIPROCESSING=0``); tensor-parallel workers are forked by default and inherit the patches.  The
multiprocessing front end of older releases (``MQLLMEngine``) does not exist in current vLLM: ``run_mp_engine`` serves
through it where the installed vLLM still has it and says so otherwise.
"""
from __future__ import annotations

import os

_CLASSES = {}
_SPECS = {
    # name -> (module, class, kind)
    "IPEXLLMClass": ("vllm", "LLM", "init"),
    "IPEXLLMAsyncLLMEngine": ("vllm.engine.async_llm_engine", "AsyncLLMEngine", "factory"),
    "IPEXLLMLLMEngine": ("vllm.engine.llm_engine", "LLMEngine", "factory"),
    "IPEXLLMAsyncV1Engine": ("vllm.v1.engine.async_llm", "AsyncLLM", "factory"),
    "IPEXLLMLLMV1Engine": ("vllm.v1.engine.llm_engine", "LLMEngine", "factory"),
}


def _convert(load_in_low_bit):
    from .model_convert import _ipex_llm_convert
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    _ipex_llm_convert(load_in_low_bit)


def _build(name):
    import importlib
    mod_name, cls_name, kind = _SPECS[name]
    base = getattr(importlib.import_module(mod_name), cls_name)
    if kind == "init":
        def __init__(self, *args, load_in_low_bit: str = "sym_int4", **kwargs):
            _convert(load_in_low_bit)
            base.__init__(self, *args, **kwargs)
        body = {"__init__": __init__}
    else:
        def from_engine_args(cls, engine_args, *args, load_in_low_bit: str = "sym_int4", **kwargs):
            _convert(load_in_low_bit)
            return super(new, cls).from_engine_args(engine_args, *args, **kwargs)

        def from_vllm_config(cls, vllm_config, *args, load_in_low_bit: str = "sym_int4", **kwargs):
            _convert(load_in_low_bit)
            return super(new, cls).from_vllm_config(vllm_config, *args, **kwargs)
        body = {"from_engine_args": classmethod(from_engine_args)}
        if hasattr(base, "from_vllm_config"):
            body["from_vllm_config"] = classmethod(from_vllm_config)
    body["__doc__"] = f"``{mod_name}.{cls_name}`` whose workers pack the model to ``load_in_low_bit`` after loading."
    body["__module__"] = __name__
    new = type(name, (base,), body)
    return new


def run_mp_engine(engine_args, usage_context, ipc_path: str, load_in_low_bit: str, engine_alive):
    """Body of the engine process of vLLM's ZeroMQ front end (reference engine.py:224-242): build the engine with the
    low-bit loader patches installed and serve until SIGTERM; ``engine_alive.value`` turns False on failure."""
    import importlib
    import signal
    from ..utils.common import invalidInputError
    try:
        base = importlib.import_module("vllm.engine.multiprocessing.engine").MQLLMEngine
    except (ImportError, AttributeError):
        invalidInputError(False, "the installed vLLM has no MQLLMEngine front end; use IPEXLLMAsyncV1Engine "
                                 "(ipex_llm.vllm.entrypoints.openai.api_server does)")

    def on_term(*_):
        raise KeyboardInterrupt("MQLLMEngine terminated")

    try:
        signal.signal(signal.SIGTERM, on_term)
        _convert(load_in_low_bit)
        engine = base.from_engine_args(engine_args=engine_args, usage_context=usage_context, ipc_path=ipc_path)
        engine.start()
    except BaseException:
        engine_alive.value = False
        raise


def __getattr__(name):
    if name in _SPECS:
        if name not in _CLASSES:
            _CLASSES[name] = _build(name)
        return _CLASSES[name]
    raise AttributeError(name)
