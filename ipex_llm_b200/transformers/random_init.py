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
                        tp_group=None, consistent_shards=False):
    """``consistent_shards``: under tensor parallelism, draw every sharded matrix whole (with the seed an unsharded
    model would use) and keep this rank's slice, so that the sharded model IS the unsharded one; off by default
    because every rank then generates the full model (the default draws each shard independently).  Replicated
    parameters (embeddings, norms) always use the same seed on every rank."""
    from .model import _rebuild_nonpersistent
    device = torch.device(device)
    shard_seed = seed
    col_cls = row_cls = ()
    world = rank = 1
    if tp_group is not None:
        from ..parallel.tp import ColumnParallelLinear, RowParallelLinear, auto_tp
        model = auto_tp(model, tp_group)
        shard_seed = seed + 7919 * tp_group.rank
        col_cls, row_cls = ColumnParallelLinear, RowParallelLinear
        world, rank = tp_group.world_size, tp_group.rank
    gen = torch.Generator(device=device)

    cfg = model.config
    n_heads = getattr(cfg, "num_attention_heads", 1)
    n_kv = getattr(cfg, "num_key_value_heads", None) or n_heads
    head_dim = getattr(cfg, "head_dim", None) or getattr(cfg, "hidden_size", n_heads) // n_heads

    def materialize(module, full_name):
        is_col, is_row = isinstance(module, col_cls), isinstance(module, row_cls)
        # q / k / v of a sharded model were merged into one matrix before this point: [q_shard; k_shard; v_shard]
        merged_qkv = world > 1 and full_name.endswith("qkv_proj") and not is_col and not is_row
        for pname, p in list(module._parameters.items()):
            if p is None or p.device.type != "meta" or isinstance(p, FP4Params):
                continue
            sharded = (is_col or merged_qkv or (is_row and p.dim() >= 2)) and world > 1
            whole = sharded and consistent_shards
            gen.manual_seed(_seed_for(f"{full_name}.{pname}", shard_seed if sharded and not whole else seed))
            if whole and merged_qkv:
                # the unsharded model's merged matrix (or bias) holds all q heads, then all k heads, then all v
                # heads; this rank keeps its contiguous block of each
                full_shape = (p.shape[0] * world,) + tuple(p.shape[1:])
                full = torch.empty(full_shape, dtype=dtype, device=device)
                full = full.normal_(0.0, std, generator=gen) if p.dim() >= 2 else full.zero_()
                q_l, kv_l = n_heads // world * head_dim, n_kv // world * head_dim
                q0, k0, v0 = rank * q_l, n_heads * head_dim + rank * kv_l, (n_heads + n_kv) * head_dim + rank * kv_l
                t = torch.cat([full[q0:q0 + q_l], full[k0:k0 + kv_l], full[v0:v0 + kv_l]], dim=0).contiguous()
                del full
            elif whole and p.dim() >= 2:
                # the matrix an unsharded model holds under this name; this rank keeps its rows (column-parallel)
                # or columns (row-parallel)
                n, k = p.shape
                if is_col:
                    full = torch.empty((n * world, k), dtype=dtype, device=device).normal_(0.0, std, generator=gen)
                    t = full[rank * n:(rank + 1) * n].contiguous()
                else:
                    full = torch.empty((n, k * world), dtype=dtype, device=device).normal_(0.0, std, generator=gen)
                    t = full[:, rank * k:(rank + 1) * k].contiguous()
                del full
            elif p.dim() >= 2:
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
