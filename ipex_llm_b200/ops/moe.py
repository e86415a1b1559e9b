"""Mixture-of-experts building blocks: quantized expert banks and routers.

transformers 5 stores MoE experts as fused 3-D parameters (``gate_up_proj [E, 2I, H]``,
``down_proj [E, H, I]``); the reference's ``nn.Linear`` walk (convert.py:485-499) would leave them in
half precision.  ``LowBitExperts`` holds every expert as packed blocks (``experts.{e}.w1|w3|w2`` =
gate|up|down, the transformers-4 Mixtral names) and evaluates
``sum_k weight_k * down_e(act(gate_e x) * up_e x)``:

* decode (few tokens)  -> per-token expert GEMVs through a device pointer table (the reference's
  ``xe_linear.moe_forward_vec``, models/deepseek.py:293-315);
* prefill / large batch -> tokens sorted by expert, one low-bit GEMM per hit expert.

Routers: softmax top-k (Mixtral / Qwen2-MoE) and grouped top-k with bias (DeepSeek-V3 ``moe_group_topk``,
models/deepseek.py:283-287).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ..quant.params import FP4Params, get_block_size
from .linear import LowBitLinear


def is_fused_experts(module: nn.Module) -> bool:
    gu = getattr(module, "gate_up_proj", None)
    dn = getattr(module, "down_proj", None)
    return isinstance(gu, nn.Parameter) and isinstance(dn, nn.Parameter) and gu.dim() == 3 and dn.dim() == 3


class _Expert(nn.Module):
    def __init__(self, hidden, inter, qtype, enable_scale_search=False):
        super().__init__()
        self.w1 = LowBitLinear(hidden, inter, qtype, bias=False, enable_scale_search=enable_scale_search)  # gate
        self.w3 = LowBitLinear(hidden, inter, qtype, bias=False, enable_scale_search=enable_scale_search)  # up
        self.w2 = LowBitLinear(inter, hidden, qtype, bias=False, enable_scale_search=enable_scale_search)  # down


class LowBitExperts(nn.ModuleList):
    """Bank of ``num_experts`` SwiGLU experts with packed low-bit weights."""

    def __init__(self, num_experts, hidden_dim, intermediate_dim, qtype, act_fn=None, enable_scale_search=False):
        super().__init__([_Expert(hidden_dim, intermediate_dim, qtype, enable_scale_search)
                          for _ in range(num_experts)])
        self.num_experts = num_experts
        self.hidden_dim = hidden_dim
        self.intermediate_dim = intermediate_dim
        self.qtype = qtype
        self.act_fn = act_fn or F.silu

    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor):
        from ..models.common import SILU, _act_mul
        if hidden_states.is_cuda and not hidden_states.requires_grad:
            from . import cuda_ops
            if cuda_ops.moe_supported(self):
                return cuda_ops.moe_forward(self, hidden_states, top_k_index, top_k_weights)
        final = torch.zeros_like(hidden_states)
        with torch.no_grad():
            mask = F.one_hot(top_k_index, num_classes=self.num_experts).permute(2, 1, 0)
            hit = torch.greater(mask.sum(dim=(-1, -2)), 0).nonzero()
        for e in hit:
            e = int(e[0])
            pos, tok = torch.where(mask[e])
            x = hidden_states[tok]
            exp = self[e]
            h = _act_mul(exp.w1(x), exp.w3(x), SILU) if self.act_fn is F.silu else self.act_fn(exp.w1(x)) * exp.w3(x)
            y = exp.w2(h) * top_k_weights[tok, pos, None].to(h.dtype)
            final.index_add_(0, tok, y.to(final.dtype))
        return final


def convert_fused_experts(module, qtype, device="cpu", convert_shape_only=False, enable_scale_search=False):
    """``MixtralExperts``-style fused parameters -> ``LowBitExperts``."""
    gu = module.gate_up_proj.data          # [E, 2I, H]
    dn = module.down_proj.data             # [E, H, I]
    E, two_i, H = gu.shape
    inter = two_i // 2
    block = get_block_size(qtype)
    if H % block != 0 or inter % block != 0 or H % 64 != 0 or inter % 64 != 0:
        return module
    bank = LowBitExperts(E, H, inter, qtype, getattr(module, "act_fn", None), enable_scale_search)
    for e in range(E):
        for name, w in (("w1", gu[e, :inter]), ("w3", gu[e, inter:]), ("w2", dn[e])):
            lin = getattr(bank[e], name)
            p = FP4Params(w, requires_grad=False, quantized=False, qtype=qtype,
                          convert_shape_only=convert_shape_only, in_features=w.shape[-1],
                          enable_scale_search=enable_scale_search)
            lin._parameters["weight"] = p.to(device)
    # a bank that auto_tp split along the intermediate dimension yields partial sums: they are summed over the group
    # at the bank's output
    if getattr(module, "_tp_group", None) is not None:
        from ..parallel.tp import install_expert_allreduce
        install_expert_allreduce(bank, module._tp_group)
    return bank


# ------------------------------------------------------------------------------------------------
# routers
# ------------------------------------------------------------------------------------------------
def softmax_topk_router(router_logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """Mixtral / Qwen2-MoE routing: softmax over experts in fp32, top-k, optional renormalisation.
    Returns ``(probs [T,E], weights [T,k], indices [T,k])``."""
    if router_logits.is_cuda and not router_logits.requires_grad:
        from . import cuda_ops
        return cuda_ops.moe_softmax_topk(router_logits, top_k, renormalize)
    probs = torch.softmax(router_logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return probs, w, idx


def moe_group_topk(scores: torch.Tensor, bias: torch.Tensor, n_group: int, topk_group: int, top_k: int,
                   norm_topk_prob: bool, routed_scaling_factor: float):
    """DeepSeek-V3 routing: sigmoid scores + per-expert bias choose ``topk_group`` of ``n_group`` expert groups
    (group score = sum of its two best biased scores), then ``top_k`` experts inside them; weights are the
    unbiased scores, renormalised and scaled.  On the GPU this is one kernel (``ipex_moe_group_topk``, a warp per
    token; the reference's ``xe_addons.moe_group_topk``, models/deepseek.py:283-287)."""
    if scores.is_cuda and not scores.requires_grad:
        from . import cuda_ops
        return cuda_ops.moe_group_topk(scores, bias, n_group, topk_group, top_k, norm_topk_prob,
                                       routed_scaling_factor)
    return _group_topk_impl(scores, bias, n_group, topk_group, top_k, norm_topk_prob, routed_scaling_factor)


def _group_topk_impl(scores, bias, n_group, topk_group, top_k, norm_topk_prob, routed_scaling_factor):
    T, E = scores.shape
    s = torch.sigmoid(scores.float())
    sb = s + bias.float().unsqueeze(0)
    g = sb.view(T, n_group, E // n_group)
    group_scores = g.topk(2, dim=-1).values.sum(dim=-1)
    gidx = group_scores.topk(topk_group, dim=-1).indices
    gmask = torch.zeros_like(group_scores).scatter_(1, gidx, 1.0)
    emask = gmask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E)
    masked = sb.masked_fill(emask == 0, float("-inf"))
    idx = masked.topk(top_k, dim=-1).indices
    w = s.gather(1, idx)
    if norm_topk_prob:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return idx, w * routed_scaling_factor


def get_moe_indexes(selected_experts: torch.Tensor, num_experts: int):
    """Token lists per expert: returns ``(sorted_token_ids, expert_offsets[E+1], sorted_slot)`` on the input's
    device (the reference builds the same on the CPU with ``xe_linear.get_moe_indexes``,
    models/qwen2_moe.py:404)."""
    flat = selected_experts.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    offsets[1:] = torch.cumsum(counts, 0)
    k = selected_experts.shape[-1]
    return order // k, offsets, order % k
