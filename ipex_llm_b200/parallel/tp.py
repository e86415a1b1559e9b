"""Tensor parallelism: module injection (AutoTP) and the process-group wrapper.

The reference delegates sharding to ``deepspeed.init_inference(mp_size=W, replace_method="auto")`` and only
keeps the ``mp_group`` on the row-parallel linears to all-reduce their outputs
(python/llm/example/GPU/Deepspeed-AutoTP/deepspeed_autotp.py:74-106,
python/llm/src/ipex_llm/transformers/convert.py:215-226, low_bit_linear.py:675-682).  DeepSpeed is not a
dependency here: ``auto_tp`` does the injection itself —

* column-parallel (output rows split): q/k/v (by heads, GQA aware), gate/up;
* row-parallel (input columns split, output all-reduced): ``o_proj``, ``down_proj``;
* ``lm_head`` vocabulary-parallel (rows split, logits gathered; the reference does the same under vLLM,
  python/llm/src/ipex_llm/vllm/xpu/model_convert.py:52-54) unless ``IPEX_LLM_TP_VOCAB_PARALLEL=0`` or the vocabulary
  does not split into multiples of 16 rows;
* everything else (norms, embeddings) replicated.  Models that keep q/k/v or gate/up fused in one ``nn.Linear``
  (phi3-style ``qkv_proj`` / ``gate_up_proj``) are refused: their rows interleave heads and would need a re-layout.

``TPGroup.all_reduce`` uses the fused NVLink kernels of ``parallel.symm_mem`` on CUDA and falls back to the
process group's all-reduce elsewhere (gloo ranks in the CPU tests).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import nn


class TPGroup:
    """A tensor-parallel group: rank / size plus the collectives the model needs."""

    def __init__(self, group=None, rank=None, world_size=None):
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank(group) if rank is None else rank
            self.world_size = dist.get_world_size(group) if world_size is None else world_size
        else:
            self.rank = 0 if rank is None else rank
            self.world_size = 1 if world_size is None else world_size
        self._symm = None

    def size(self):
        return self.world_size

    def symm(self):
        """Lazily created symmetric-memory communicator (CUDA only)."""
        if self._symm is None and self.world_size > 1 and torch.cuda.is_available():
            from .symm_mem import SymmComm
            self._symm = SymmComm.get(self.group)
        return self._symm

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return t
        if t.is_cuda:
            comm = self.symm()
            if comm is not None and comm.can_all_reduce(t):
                return comm.all_reduce(t)
        dist.all_reduce(t, group=self.group)
        return t

    def all_gather_last_dim(self, t: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.group)


class ColumnParallelLinear(nn.Linear):
    """Holds rows ``[rank*N/W, (rank+1)*N/W)`` of the full weight; no communication."""

    def __init__(self, in_features, out_features, bias=False, mp_group=None, device=None, dtype=None):
        super().__init__(in_features, out_features, bias, device=device, dtype=dtype)
        self.mp_group = mp_group


class RowParallelLinear(nn.Linear):
    """Holds columns ``[rank*K/W, (rank+1)*K/W)``; the partial outputs are summed over ``mp_group``."""

    def __init__(self, in_features, out_features, bias=False, mp_group=None, device=None, dtype=None):
        super().__init__(in_features, out_features, bias, device=device, dtype=dtype)
        self.mp_group = mp_group

    def forward(self, x):
        y = nn.functional.linear(x, self.weight)
        if self.mp_group is not None:
            y = self.mp_group.all_reduce(y)
        if self.bias is not None:
            y = y + self.bias
        return y


COLUMN_NAMES = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "w1", "w3")
ROW_NAMES = ("o_proj", "down_proj", "w2", "dense_4h_to_h")


def _shard_rows(w, rank, world, unit=1):
    n = w.shape[0]
    if (n // unit) % world != 0:
        raise ValueError(f"cannot split {n // unit} units over {world} ranks")
    per = n // world
    return w[rank * per:(rank + 1) * per].contiguous()


def _shard_cols(w, rank, world):
    k = w.shape[1]
    if k % world != 0:
        raise ValueError(f"cannot split {k} columns over {world} ranks")
    per = k // world
    return w[:, rank * per:(rank + 1) * per].contiguous()


def _column(lin: nn.Linear, rank, world, group, unit=1):
    w = _shard_rows(lin.weight.data, rank, world, unit)
    # no mp_group on column-parallel layers: the converter all-reduces whatever carries one
    new = ColumnParallelLinear(lin.in_features, w.shape[0], lin.bias is not None, mp_group=None,
                               device="meta", dtype=w.dtype)
    new.tp_group = group
    new.weight = nn.Parameter(w, requires_grad=False)
    if lin.bias is not None:
        new.bias = nn.Parameter(_shard_rows(lin.bias.data, rank, world, unit), requires_grad=False)
    return new


def _row(lin: nn.Linear, rank, world, group):
    w = _shard_cols(lin.weight.data, rank, world)
    new = RowParallelLinear(w.shape[1], lin.out_features, lin.bias is not None, mp_group=group,
                            device="meta", dtype=w.dtype)
    new.weight = nn.Parameter(w, requires_grad=False)
    if lin.bias is not None:
        new.bias = nn.Parameter(lin.bias.data.clone(), requires_grad=False)
    return new


def auto_tp(model: nn.Module, group: TPGroup = None, rank=None, world_size=None):
    """Shard a (not yet quantized) Hugging Face decoder in place for this rank.

    Must run before ``optimize_model`` / ``ggml_convert_low_bit``: the converter then turns the parallel
    linears into ``LowBitLinear`` (keeping ``mp_group`` on the row-parallel ones), as the reference does with
    DeepSpeed's ``LinearLayer`` / ``LinearAllreduce``.
    """
    group = group or TPGroup(rank=rank, world_size=world_size)
    rank, world = group.rank, group.world_size
    if world == 1:
        return model
    cfg = model.config
    n_heads = cfg.num_attention_heads
    n_kv = getattr(cfg, "num_key_value_heads", None) or n_heads
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // n_heads
    if n_heads % world != 0:
        raise ValueError(f"num_attention_heads={n_heads} is not divisible by tensor-parallel size {world}")
    if n_kv % world != 0:
        raise ValueError(f"num_key_value_heads={n_kv} is not divisible by tensor-parallel size {world}")

    for mod in model.modules():
        for name, child in list(mod.named_children()):
            if not isinstance(child, nn.Linear) or isinstance(child, (ColumnParallelLinear, RowParallelLinear)):
                continue
            if name in ("qkv_proj", "gate_up_proj", "query_key_value", "dense_h_to_4h"):
                raise NotImplementedError(
                    f"auto_tp: '{name}' holds several projections in one matrix; tensor parallelism needs them "
                    "split (q/k/v, gate/up) before sharding")
            if name in COLUMN_NAMES:
                unit = head_dim if name in ("q_proj", "k_proj", "v_proj") else 1
                mod._modules[name] = _column(child, rank, world, group, unit)
            elif name in ROW_NAMES:
                mod._modules[name] = _row(child, rank, world, group)
    # fused 3-D experts: split the intermediate dimension
    for mod in model.modules():
        gu = getattr(mod, "gate_up_proj", None)
        dn = getattr(mod, "down_proj", None)
        if isinstance(gu, nn.Parameter) and gu.dim() == 3 and isinstance(dn, nn.Parameter):
            E, two_i, H = gu.shape
            inter = two_i // 2
            per = inter // world
            g = gu.data[:, rank * per:(rank + 1) * per]
            u = gu.data[:, inter + rank * per: inter + (rank + 1) * per]
            mod.gate_up_proj = nn.Parameter(torch.cat([g, u], dim=1).contiguous(), requires_grad=False)
            mod.down_proj = nn.Parameter(dn.data[:, :, rank * per:(rank + 1) * per].contiguous(), requires_grad=False)
            mod.intermediate_dim = per
            mod._tp_group = group
    head = getattr(model, "lm_head", None)
    if isinstance(head, nn.Linear) and not isinstance(head, ColumnParallelLinear) and \
            os.environ.get("IPEX_LLM_TP_VOCAB_PARALLEL", "1") != "0" and \
            not getattr(cfg, "tie_word_embeddings", False) and head.out_features % (16 * world) == 0:
        new = _column(head, rank, world, group)
        new.gather_output = True          # the converted module gathers its logits over the group
        model.lm_head = new
    model._tp_group = group
    model.config.tp_size = world
    return model
