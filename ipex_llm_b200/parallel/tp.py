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
  (phi3-style ``qkv_proj`` / ``gate_up_proj``) are split part by part; attention modules that cannot take fewer heads
  (latent attention, head-interleaved ``query_key_value``, forwards that reshape with the configured head count) stay
  replicated while their MLP / expert banks are split.

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


COLUMN_NAMES = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "w1", "w3", "dense_h_to_4h", "fc1", "c_fc")
ROW_NAMES = ("o_proj", "down_proj", "w2", "dense_4h_to_h", "fc2", "c_proj")


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


def _column_fused(lin: nn.Linear, parts, rank, world, group, unit=1):
    """Column-parallel split of a matrix that stacks several projections (``[q; k; v]``, ``[gate; up]``): every part
    is split on its own and the rank's slices are stacked again, so the module that owns the matrix still finds the
    parts where it expects them."""
    bounds, start = [], 0
    for n in parts:
        bounds.append((start, start + n))
        start += n
    if start != lin.weight.shape[0]:
        raise ValueError(f"fused matrix has {lin.weight.shape[0]} rows, its parts add up to {start}")
    w = torch.cat([_shard_rows(lin.weight.data[a:b], rank, world, unit) for a, b in bounds], dim=0)
    new = ColumnParallelLinear(lin.in_features, w.shape[0], lin.bias is not None, mp_group=None,
                               device="meta", dtype=w.dtype)
    new.tp_group = group
    new.weight = nn.Parameter(w, requires_grad=False)
    if lin.bias is not None:
        new.bias = nn.Parameter(torch.cat([_shard_rows(lin.bias.data[a:b], rank, world, unit) for a, b in bounds]),
                                requires_grad=False)
    return new


def _row(lin: nn.Linear, rank, world, group):
    w = _shard_cols(lin.weight.data, rank, world)
    new = RowParallelLinear(w.shape[1], lin.out_features, lin.bias is not None, mp_group=group,
                            device="meta", dtype=w.dtype)
    new.weight = nn.Parameter(w, requires_grad=False)
    if lin.bias is not None:
        new.bias = nn.Parameter(lin.bias.data.clone(), requires_grad=False)
    return new


_ATTN_CHILDREN = ("q_proj", "k_proj", "v_proj", "o_proj", "qkv_proj", "q_a_proj", "q_b_proj", "kv_a_proj_with_mqa",
                  "kv_b_proj", "query_key_value", "c_attn", "Wqkv", "out_proj")


def _is_attention(mod: nn.Module) -> bool:
    return any(name in _ATTN_CHILDREN for name, _ in mod.named_children())


def _attention_shard_safe(model, attn: nn.Module) -> bool:
    """Can q / k / v be split by heads and o_proj by columns under this attention module?  Yes when the package's own
    attention forward will replace it (it reads the head counts off the weights), or when the module's own forward
    views its projections as ``(-1, head_dim)`` and has no norm over a whole q / k vector; no for latent attention
    and for forwards that reshape with the configured head count."""
    children = dict(attn.named_children())
    if ("q_proj" not in children and "qkv_proj" not in children) or "o_proj" not in children:
        return False                             # latent attention (q_a / q_b, kv_a / kv_b), head-interleaved qkv
    from ..models import decoder as D
    from ..models.registry import family_for
    fam = family_for(model)
    if fam is not None and any(fwd is D.decoder_attention_forward and target == type(attn).__name__
                               for target, fwd in fam.post):
        return True
    q_out = children["q_proj"].out_features if "q_proj" in children else -1
    for norm_name in ("q_norm", "k_norm", "q_layernorm", "k_layernorm"):
        w = getattr(children.get(norm_name), "weight", None)
        if w is not None and w.numel() == q_out:
            return False
    import inspect
    try:
        src = inspect.getsource(type(attn).forward)
    except (OSError, TypeError):
        return False
    return "-1, self.head_dim" in src and "self.num_heads" not in src and "self.num_attention_heads" not in src


def install_expert_allreduce(experts: nn.Module, group):
    """An expert bank split along its intermediate dimension returns partial sums: sum them over ``group`` right at
    the bank's output, whatever MoE block (the package's or the modeling file's own) called it."""
    experts._tp_group = group
    if getattr(experts, "_tp_hooked", False):
        return experts
    experts._tp_hooked = True
    experts.register_forward_hook(lambda mod, args, out: mod._tp_group.all_reduce(out))
    return experts


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

    replicated = []
    for mod_name, mod in model.named_modules():
        if _is_attention(mod) and not _attention_shard_safe(model, mod):
            # this attention module computes its head count from the config (or normalises whole q / k vectors, or
            # is latent attention): it stays whole on every rank, the MLP / expert shards still divide the bulk
            replicated.append(mod_name)
            continue
        for name, child in list(mod.named_children()):
            if not isinstance(child, nn.Linear) or isinstance(child, (ColumnParallelLinear, RowParallelLinear)):
                continue
            if name == "qkv_proj":
                # [all q heads; all k heads; all v heads] (Phi-3): every part split by heads
                mod._modules[name] = _column_fused(child, [n_heads * head_dim, n_kv * head_dim, n_kv * head_dim],
                                                   rank, world, group, head_dim)
            elif name == "gate_up_proj":
                half = child.out_features // 2                     # [gate; up] (Phi-3, GLM)
                mod._modules[name] = _column_fused(child, [half, half], rank, world, group)
            elif name in COLUMN_NAMES:
                unit = head_dim if name in ("q_proj", "k_proj", "v_proj") else 1
                mod._modules[name] = _column(child, rank, world, group, unit)
            elif name in ROW_NAMES:
                mod._modules[name] = _row(child, rank, world, group)
    if replicated:
        import logging
        logging.getLogger(__name__).info("auto_tp: %d attention modules of class %s stay replicated", len(replicated),
                                         type(model.get_submodule(replicated[0])).__name__)
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
            install_expert_allreduce(mod, group)
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
