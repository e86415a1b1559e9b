"""Loading of pre-quantized AWQ / GPTQ checkpoints.

Counterpart of python/llm/src/ipex_llm/transformers/awq/awq.py (``_replace_with_awq_layers`` :187-226,
``get_blocks`` / ``get_named_linears`` / ``get_layer_type`` :62-120, ``_load_config`` :123-184) and of the GPTQ branch
of ``from_pretrained`` (transformers/model.py:253-291), which in the reference leans on auto-gptq's ``QuantLinear``.
Neither auto-awq nor auto-gptq is needed here: the model skeleton is built on the ``meta`` device, its linears are
swapped for small containers that own ``qweight / qzeros / scales`` buffers with the checkpoint's shapes, the
checkpoint tensors are copied in file by file, and the caller (``from_pretrained``) then repacks every container into
``asym_int4`` blocks (``convert.convert_gptq``) without a round trip through floating point.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterator, Tuple

import torch
from torch import nn

from ...utils.common import invalidInputError
from .linear import AwqBackendPackingMethod, WQLinear_GEMM

layer_type_dict = {
    "mpt": "MPTBlock", "llama": "LlamaDecoderLayer", "opt": "OPTDecoderLayer", "RefinedWeb": "FalconDecoderLayer",
    "RefinedWebModel": "FalconDecoderLayer", "falcon": "FalconDecoderLayer", "bloom": "BloomBlock",
    "gptj": "GPTJBlock", "gpt_bigcode": "GPTBigCodeBlock", "mistral": "MistralDecoderLayer",
    "gpt_neox": "GPTNeoXDecoderLayer", "aquila": "AquilaDecoderLayer", "Yi": "YiDecoderLayer",
    "mixtral": "MixtralDecoderLayer", "qwen2": "Qwen2DecoderLayer", "gemma": "GemmaDecoderLayer",
    "qwen3": "Qwen3DecoderLayer", "phi3": "Phi3DecoderLayer",
}


class QuantLinear(nn.Module):
    """Container with the AutoGPTQ (v1) tensor layout: ``qweight [in/8, out]``, ``qzeros [in/g, out/8]`` (stored
    minus one), ``scales [in/g, out]``, ``g_idx [in]``."""

    def __init__(self, bits, group_size, infeatures, outfeatures, bias, device="meta"):
        super().__init__()
        invalidInputError(bits == 4, "Only 4-bit gptq is supported.")
        self.bits, self.infeatures, self.outfeatures = bits, infeatures, outfeatures
        self.in_features, self.out_features = infeatures, outfeatures
        self.group_size = group_size if group_size != -1 else infeatures
        g = infeatures // self.group_size
        self.register_buffer("qweight", torch.zeros((infeatures // 8, outfeatures), dtype=torch.int32, device=device))
        self.register_buffer("qzeros", torch.zeros((g, outfeatures // 8), dtype=torch.int32, device=device))
        self.register_buffer("scales", torch.zeros((g, outfeatures), dtype=torch.float16, device=device))
        self.register_buffer("g_idx", torch.zeros(infeatures, dtype=torch.int32, device=device))
        if bias:
            self.register_buffer("bias", torch.zeros(outfeatures, dtype=torch.float16, device=device))
        else:
            self.bias = None

    def forward(self, x):
        raise RuntimeError("QuantLinear is a checkpoint container; load the model through "
                           "AutoModelForCausalLM.from_pretrained(..., load_in_4bit=True)")


def get_layer_type(config) -> str:
    return layer_type_dict.get(config.model_type, "")


def get_blocks(model) -> nn.ModuleList:
    """The decoder stack: the longest ModuleList of the model."""
    best = None
    for m in model.modules():
        if isinstance(m, nn.ModuleList) and len(m) and (best is None or len(m) > len(best)):
            best = m
    invalidInputError(best is not None, f"cannot find the decoder blocks of {type(model).__name__}")
    return best


def get_named_linears(module) -> Dict[str, nn.Linear]:
    return {name: m for name, m in module.named_modules() if isinstance(m, nn.Linear)}


def set_op_by_name(layer, name, new_module):
    parent = layer
    parts = name.split(".")
    for p in parts[:-1]:
        parent = parent[int(p)] if p.isdigit() else getattr(parent, p)
    if parts[-1].isdigit():
        parent[int(parts[-1])] = new_module
    else:
        setattr(parent, parts[-1], new_module)


def _replace_with_awq_layers(model, awq_config, backend=AwqBackendPackingMethod.AUTOAWQ):
    skip = set(awq_config.get("modules_to_not_convert") or [])
    for layer in get_blocks(model):
        for name, lin in get_named_linears(layer).items():
            if any(s in name for s in skip):
                continue
            q = WQLinear_GEMM(awq_config["bits"], awq_config["group_size"], lin.in_features, lin.out_features,
                              lin.bias is not None, "meta", backend)
            set_op_by_name(layer, name, q)
    return model


def _replace_with_gptq_layers(model, gptq_config):
    for layer in get_blocks(model):
        for name, lin in get_named_linears(layer).items():
            set_op_by_name(layer, name, QuantLinear(gptq_config["bits"], gptq_config["group_size"], lin.in_features,
                                                    lin.out_features, lin.bias is not None))
    return model


def iter_checkpoint_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """Every tensor of a Hugging Face checkpoint directory (safetensors or .bin, sharded or not)."""
    files = []
    for idx in ("model.safetensors.index.json", "pytorch_model.bin.index.json"):
        p = os.path.join(path, idx)
        if os.path.exists(p):
            with open(p) as f:
                files = sorted(set(json.load(f)["weight_map"].values()))
            break
    if not files:
        files = [f for f in ("model.safetensors", "pytorch_model.bin", "gptq_model-4bit-128g.safetensors")
                 if os.path.exists(os.path.join(path, f))]
    if not files:
        files = sorted(f for f in os.listdir(path) if f.endswith((".safetensors", ".bin", ".pt")))
    invalidInputError(len(files) > 0, f"no weight files under {path}")
    for fn in files:
        full = os.path.join(path, fn)
        if fn.endswith(".safetensors"):
            from safetensors import safe_open
            with safe_open(full, framework="pt", device="cpu") as f:
                for k in f.keys():
                    yield k, f.get_tensor(k)
        else:
            sd = torch.load(full, map_location="cpu", weights_only=True)
            yield from sd.items()


def _materialize_and_load(model, path: str, dtype):
    model.to_empty(device="cpu")
    targets = dict(model.named_parameters())
    targets.update(dict(model.named_buffers()))
    seen = set()
    with torch.no_grad():
        for k, v in iter_checkpoint_tensors(path):
            if k not in targets:
                continue
            t = targets[k]
            invalidInputError(tuple(t.shape) == tuple(v.shape),
                              f"checkpoint tensor {k} has shape {tuple(v.shape)}, the model expects {tuple(t.shape)}")
            t.copy_(v.to(t.dtype))
            seen.add(k)
    missing = [k for k, _ in model.named_parameters() if k not in seen]
    if getattr(model.config, "tie_word_embeddings", False):
        model.tie_weights()
        missing = [k for k in missing if "lm_head" not in k]
    invalidInputError(not missing, f"checkpoint lacks tensors for {missing[:5]}")
    from ..model import _rebuild_nonpersistent
    _rebuild_nonpersistent(model)
    for m in model.modules():   # floating-point leftovers (norms, embeddings) follow the requested dtype
        for n, p in list(m._parameters.items()):
            if p is not None and p.is_floating_point() and p.dtype != dtype:
                p.data = p.data.to(dtype)
    return model.eval()


def _skeleton(hf_cls, path, trust_remote_code, dtype):
    import transformers
    config = transformers.AutoConfig.from_pretrained(path, trust_remote_code=trust_remote_code)
    try:
        from transformers.initialization import no_init_weights
    except ImportError:
        from transformers.modeling_utils import no_init_weights
    with no_init_weights(), torch.device("meta"):
        model = hf_cls.from_config(config, trust_remote_code=trust_remote_code, dtype=dtype)
    return model


def load_awq_checkpoint(hf_cls, awq_config, pretrained_model_name_or_path, *args, **kwargs):
    dtype = kwargs.get("dtype") or kwargs.get("torch_dtype") or torch.float16
    if isinstance(dtype, str):
        dtype = torch.float16
    model = _skeleton(hf_cls, pretrained_model_name_or_path, kwargs.get("trust_remote_code", False), dtype)
    backend = AwqBackendPackingMethod.LLMAWQ if awq_config.get("backend") == "llm-awq" else \
        AwqBackendPackingMethod.AUTOAWQ
    model = _replace_with_awq_layers(model, awq_config, backend)
    return _materialize_and_load(model, pretrained_model_name_or_path, dtype)


def load_gptq_checkpoint(hf_cls, gptq_config, pretrained_model_name_or_path, *args, **kwargs):
    dtype = kwargs.get("dtype") or kwargs.get("torch_dtype") or torch.float16
    if isinstance(dtype, str):
        dtype = torch.float16
    model = _skeleton(hf_cls, pretrained_model_name_or_path, kwargs.get("trust_remote_code", False), dtype)
    model = _replace_with_gptq_layers(model, gptq_config)
    return _materialize_and_load(model, pretrained_model_name_or_path, dtype)
