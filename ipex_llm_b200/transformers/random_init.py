"""Build a random-initialised low-bit model layer by layer on the GPU (no checkpoint, no host copy).

Used by ``AutoModelForCausalLM.from_config``.  The model skeleton lives on ``meta``; each linear (or fused expert
bank) is given real N(0, std) weights on the device only for the instant it takes the GPU quantizer to pack
them, so the half-precision model never exists as a whole.  The reference has no counterpart: its benchmarks
load real checkpoints through ``from_pretrained`` (python/llm/dev/benchmark/all-in-one/run.py:552-584).
"""
from __future__ import annotations

import zlib

import torch
from torch import nn

from ..quant.params import FP4Params
from .convert import ggml_convert_low_bit


def _seed_for(name: str, seed: int) -> int:
    return (zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF


def convert_random_init(model, qtype, optimize_model, device, dtype, seed, std, modules_to_not_convert,
                        tp_group=None):
    from .model import _rebuild_nonpersistent
    device = torch.device(device)
    if tp_group is not None:
        from ..parallel.tp import auto_tp
        model = auto_tp(model, tp_group)
        seed = seed + 7919 * tp_group.rank
    gen = torch.Generator(device=device)

    def materialize(module, full_name):
        for pname, p in list(module._parameters.items()):
            if p is None or p.device.type != "meta" or isinstance(p, FP4Params):
                continue
            gen.manual_seed(_seed_for(f"{full_name}.{pname}", seed))
            if p.dim() >= 2:
                t = torch.empty(tuple(p.shape), dtype=dtype, device=device).normal_(0.0, std, generator=gen)
            elif pname == "weight" and "norm" in type(module).__name__.lower():
                t = torch.ones(tuple(p.shape), dtype=dtype, device=device)
            else:
                t = torch.zeros(tuple(p.shape), dtype=dtype, device=device)
            module._parameters[pname] = nn.Parameter(t, requires_grad=False)
        for bname, b in list(module._buffers.items()):
            if b is not None and b.device.type == "meta":
                module._buffers[bname] = torch.zeros(b.shape, dtype=b.dtype, device=device)

    model = ggml_convert_low_bit(model, qtype, optimize_model, device=device,
                                 modules_to_not_convert=modules_to_not_convert, torch_dtype=dtype,
                                 materialize=materialize)
    # whatever is still on meta (norm scales, embeddings of skipped modules, buffers)
    for name, mod in model.named_modules():
        materialize(mod, name)
        for bname, b in list(mod._buffers.items()):
            if b is not None and b.device.type == "meta":
                mod._buffers[bname] = torch.zeros(b.shape, dtype=b.dtype, device=device)
    _rebuild_nonpersistent(model, device)
    model.eval()
    return model
