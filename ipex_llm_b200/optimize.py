"""``optimize_model`` for any ``nn.Module`` plus its ``save_low_bit`` / ``load_low_bit`` / ``low_memory_init``.

Counterpart of python/llm/src/ipex_llm/optimize.py:37-267 and utils/lazy_load_torch.py of the reference.
``accelerate`` is not a dependency: ``low_memory_init`` is a self-contained meta-device context, and
``load_low_bit`` assigns checkpoint tensors key by key.
"""
from __future__ import annotations

import json
import os
import types
import warnings
from contextlib import contextmanager

import torch

from .quant import qtypes as qt
from .transformers.convert import ggml_convert_low_bit
from .utils.common import invalidInputError

PYTORCH_MODEL_NAME = "pytorch_model.bin"
CONFIG_NAME = "bigdl_config.json"


def _save_low_bit(self, save_dir, *args, **kwargs):
    invalidInputError(self._bigdl_config.get("bigdl_transformers_low_bit", False),
                      "Detected this model is not a low-bit model, please use from_pretrained's"
                      " load_in_4bit or load_in_low_bit parameter to load a 4-bit model first.")
    os.makedirs(save_dir, exist_ok=True)
    from transformers import PreTrainedModel
    from .transformers.model import _plain_state_dict, save_low_bit
    if isinstance(self, PreTrainedModel):
        self.config.update({"bigdl_transformers_low_bit": self._bigdl_config["bigdl_transformers_low_bit"]})
        save_low_bit(self, save_dir, *args, **kwargs)
    else:
        torch.save(_plain_state_dict(self), os.path.join(save_dir, PYTORCH_MODEL_NAME))
    cfg = dict(self._bigdl_config)
    if cfg["bigdl_transformers_low_bit"] in ("mixed_fp4", "mixed_fp8"):
        # the per-layer choice between the integer and the float format (the bytes do not tell which)
        from .quant.params import FP4Params
        cfg["bigdl_layer_qtypes"] = {n: qt.qtype_name(m.weight.qtype) for n, m in self.named_modules()
                                     if isinstance(getattr(m, "weight", None), FP4Params) and m.weight.quantized}
    with open(os.path.join(save_dir, CONFIG_NAME), "w") as f:
        json.dump(cfg, f)


def low_bit_sanity_check(model_path):
    invalidInputError(os.path.isdir(model_path), "model_path should be a valid directory path.")
    invalidInputError(os.path.isfile(os.path.join(model_path, CONFIG_NAME)),
                      "bigdl_config.json should be under your model directory,"
                      "please check your input path.")
    with open(os.path.join(model_path, CONFIG_NAME), "r") as f:
        _config = json.load(f)
    low_bit = _config.get("bigdl_transformers_low_bit", None)
    if low_bit is None:
        warnings.warn("No low-bit optimization was applied to the saved model.")
    return low_bit


@contextmanager
def low_memory_init():
    """Create a model without allocating or initialising its weights (everything lands on ``meta``); pair it
    with ``load_low_bit(model, path)``.  Also neutralises ``load_state_dict`` so that a surrounding
    ``from_pretrained`` cannot pull the full-precision checkpoint into memory."""
    saved_load = torch.nn.Module.load_state_dict
    saved_to = torch.nn.Module.to

    def _noop_load(self, *a, **k):
        return torch.nn.modules.module._IncompatibleKeys([], [])

    def _noop_to(self, *a, **k):
        return self

    torch.nn.Module.load_state_dict = _noop_load
    torch.nn.Module.to = _noop_to
    try:
        with torch.device("meta"):
            yield
    finally:
        torch.nn.Module.load_state_dict = saved_load
        torch.nn.Module.to = saved_to


def _set_tensor(model, name, tensor):
    parts = name.split(".")
    mod = model
    for p in parts[:-1]:
        mod = getattr(mod, p)
    leaf = parts[-1]
    from .quant.params import FP4Params
    if leaf in mod._parameters:
        old = mod._parameters[leaf]
        if isinstance(old, FP4Params):
            mod._parameters[leaf] = FP4Params(tensor, requires_grad=False, quantized=True, _shape=old._shape,
                                              qtype=old.qtype)
        else:
            mod._parameters[leaf] = torch.nn.Parameter(tensor, requires_grad=False)
    elif leaf in mod._buffers:
        mod._buffers[leaf] = tensor
    else:
        setattr(mod, leaf, tensor)


def load_low_bit(model, model_path):
    """Load an optimized model saved by ``model.save_low_bit`` into ``model`` (an ``nn.Module`` instance on
    ``cpu`` or ``meta``, e.g. created under ``low_memory_init()``)."""
    low_bit = low_bit_sanity_check(model_path)
    invalidInputError(isinstance(model, torch.nn.Module),
                      f"model should be a instance of `torch.nn.Module`, but got {type(model)} at last.")
    if low_bit:
        if hasattr(model, "device"):
            invalidInputError(model.device.type in ("cpu", "meta"),
                              f"Expect model on device `cpu` or `meta`, but got device type {model.device.type}")
        qtype = qt.qtype_from_name(low_bit)
        on_meta = any(p.device.type == "meta" for p in model.parameters())
        model = ggml_convert_low_bit(model, qtype=qtype, convert_shape_only=True,
                                     device="meta" if on_meta else "cpu")
        with open(os.path.join(model_path, CONFIG_NAME)) as f:
            chosen = json.load(f).get("bigdl_layer_qtypes") or {}
        from .quant.params import FP4Params
        for mod_name, q_name in chosen.items():
            try:
                mod = model.get_submodule(mod_name)
            except AttributeError:
                continue
            if isinstance(getattr(mod, "weight", None), FP4Params):
                mod.weight.qtype = qt.qtype_from_name(q_name)
                if hasattr(mod, "qtype"):
                    mod.qtype = mod.weight.qtype
    from .transformers.model import _load_state_dict_from_dir, _rebuild_nonpersistent
    sd = _load_state_dict_from_dir(model_path)
    for name, tensor in sd.items():
        _set_tensor(model, name, tensor)
    _rebuild_nonpersistent(model, "cpu")
    model.eval()           # a shell built from a config is in training mode (dropout, router jitter); this is inference
    if low_bit:
        model._bigdl_config = {"bigdl_transformers_low_bit": low_bit}
        model.save_low_bit = types.MethodType(_save_low_bit, model)
    return model


def optimize_model(model, low_bit="sym_int4", optimize_llm=True, modules_to_not_convert=None,
                   cpu_embedding=False, **kwargs):
    """Apply low-bit optimisation to any PyTorch model (``nn.Module``).

    ``low_bit``: ``'sym_int4' | 'asym_int4' | 'sym_int5' | 'asym_int5' | 'sym_int8' | 'nf3' | 'nf4' | 'fp4' | 'fp6'
    | 'fp8' | 'fp8_e4m3' | 'fp8_e5m2' | 'fp16' | 'bf16'`` or ``None`` (only the forward optimisations).
    Returns the optimized model, which gains ``save_low_bit(dir)``.
    """
    invalidInputError(low_bit is None or low_bit in qt.ggml_tensor_qtype,
                      f"Unknown load_in_low_bit value: {low_bit}, expected:"
                      f" sym_int4, asym_int4, sym_int5, asym_int5 or sym_int8.")
    from .models.sd import is_diffusion_pipeline, optimize_pipeline
    if is_diffusion_pipeline(model):
        # a diffusers pipeline (reference convert.py:1253-1265): UNet attention on the package's SDPA; with a low_bit
        # the UNet's linears are packed as well
        if optimize_llm:
            optimize_pipeline(model)
        if low_bit is not None:
            model.unet = ggml_convert_low_bit(model.unet, qtype=qt.qtype_from_name(low_bit), optimize_model=False,
                                              modules_to_not_convert=modules_to_not_convert,
                                              device=kwargs.pop("device", None) or "cpu")
        return model
    invalidInputError(isinstance(model, torch.nn.Module),
                      f"model should be an instance of `torch.nn.Module`, but got {type(model)} at last.")
    if hasattr(model, "device") and isinstance(getattr(model, "device"), torch.device):
        invalidInputError(model.device.type in ("cpu", "meta", "cuda"),
                          f"Expect model on device `cpu`, `meta` or `cuda`, but got device type {model.device.type}")
    if kwargs.pop("replace_embedding", False):
        warnings.warn("replace_embedding is deprecated and will be removed in a future version,"
                      " please use cpu_embedding instead.", FutureWarning)
        cpu_embedding = True
    if low_bit == "fp16":
        torch_dtype = kwargs.get("torch_dtype", None)
        invalidInputError(torch_dtype is None or torch_dtype == torch.float16,
                          "Please use torch_dtype=torch.float16 when setting low_bit='fp16'.")
        torch_dtype = torch.float16
    else:
        torch_dtype = kwargs.get("torch_dtype", "auto")
    device = kwargs.pop("device", None)
    if device is None:
        p = next(model.parameters(), None)
        device = "cuda" if (p is not None and p.is_cuda) else "cpu"
    if low_bit is None:
        from .transformers.convert import _optimize_post, _optimize_pre
        if optimize_llm:
            model = _optimize_post(_optimize_pre(model))
        return model
    qtype = qt.qtype_from_name(low_bit)
    model = ggml_convert_low_bit(model, qtype=qtype, torch_dtype=torch_dtype, optimize_model=optimize_llm,
                                 modules_to_not_convert=modules_to_not_convert, cpu_embedding=cpu_embedding,
                                 disable_optimize_pre=kwargs.pop("disable_optimize_pre", False), device=device)
    model._bigdl_config = {"bigdl_transformers_low_bit": low_bit}
    model.save_low_bit = types.MethodType(_save_low_bit, model)
    if hasattr(model, "config") and hasattr(model.config, "update"):
        try:
            model.config.update({"bigdl_transformers_low_bit": low_bit})
        except Exception:  # noqa: BLE001
            pass
    if hasattr(model, "generate"):
        from .transformers.model import _attach_api
        save = model.save_low_bit
        _attach_api(model)
        model.save_low_bit = save
    return model
