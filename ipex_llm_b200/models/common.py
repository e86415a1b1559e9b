"""Fused-op façade shared by every model forward replacement.

Counterpart of python/llm/src/ipex_llm/transformers/models/common.py:22-305 of the reference
(``merge_qkv_base``, ``fuse_mlp_base`` / ``mlp_silu_forward`` / ``mlp_gelu_forward``, ``rms_norm_forward``,
``layer_norm_forward``, ``attention_softmax``, ``scaled_dot_product_attention``, head-dim padding helpers).
On a CUDA tensor every function calls the package's own sm_100a kernel; on the CPU it is plain PyTorch in fp32.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..ops.kv_cache import fp8_e5m2_dequantize

SILU = 0
GELU = 1


# ------------------------------------------------------------------------------------------------
# weight surgery helpers
# ------------------------------------------------------------------------------------------------
def merge_linear(linears):
    """Concatenate several ``nn.Linear`` along the output dimension into one."""
    if hasattr(linears[0], "weight"):
        new_weight = torch.cat([lin.weight.data for lin in linears], dim=0)
        if linears[0].bias is not None:
            new_linear = nn.Linear(0, 0, bias=True)
            new_linear.bias = nn.Parameter(torch.cat([lin.bias.data for lin in linears], dim=0), requires_grad=False)
        else:
            new_linear = nn.Linear(0, 0, bias=False)
        new_linear.weight = nn.Parameter(new_weight, requires_grad=False)
        new_linear.in_features = new_weight.size(1)
        new_linear.out_features = new_weight.size(0)
        return new_linear
    raise TypeError("merge_linear expects nn.Linear-like modules")


def merge_qkv_base(module: nn.Module, attention_class):
    """Replace q_proj/k_proj/v_proj of ``attention_class`` modules by one ``qkv_proj``
    (reference models/common.py:40-52).  ``attention_class`` may be a class or a class name."""
    hit = (module.__class__.__name__ == attention_class) if isinstance(attention_class, str) \
        else isinstance(module, attention_class)
    if hit and hasattr(module, "q_proj") and hasattr(module, "k_proj") and hasattr(module, "v_proj"):
        module.qkv_proj = merge_linear([module.q_proj, module.k_proj, module.v_proj])
        del module.q_proj, module.k_proj, module.v_proj


def padding_linear_hd(linear: nn.Linear, old_hd: int, new_hd: int) -> nn.Linear:
    in_features, out_features = linear.in_features, linear.out_features
    weight = linear.weight.data.view(-1, old_hd, in_features)
    new_weight = torch.zeros(weight.shape[0], new_hd, in_features, dtype=weight.dtype, device=weight.device)
    new_weight[:, :old_hd] = weight
    new_linear = nn.Linear(0, 0, bias=linear.bias is not None)
    new_linear.weight = nn.Parameter(new_weight.view(-1, in_features), requires_grad=False)
    if linear.bias is not None:
        bias = linear.bias.data.view(-1, old_hd)
        nb = torch.zeros(bias.shape[0], new_hd, dtype=bias.dtype, device=bias.device)
        nb[:, :old_hd] = bias
        new_linear.bias = nn.Parameter(nb.flatten(), requires_grad=False)
    new_linear.in_features = in_features
    new_linear.out_features = out_features // old_hd * new_hd
    return new_linear


def padding_states_hd(states: torch.Tensor, old_hd: int, new_hd: int):
    return F.pad(states, (0, new_hd - old_hd))


# ------------------------------------------------------------------------------------------------
# norms
# ------------------------------------------------------------------------------------------------
def rms_norm_forward(self, hidden_states: torch.Tensor, residual: torch.Tensor = None):
    weight = self.weight
    eps = getattr(self, "variance_epsilon", None)
    if eps is None:
        eps = getattr(self, "eps", None)
    if eps is None:
        eps = getattr(self, "epsilon", 1e-6)
    offset = getattr(self, "_ipex_weight_offset", 0.0)  # Gemma: weight + 1
    if hidden_states.is_cuda and not hidden_states.requires_grad and \
            hidden_states.dtype in (torch.float16, torch.bfloat16):
        from ..ops import cuda_ops
        return cuda_ops.rms_norm(hidden_states, weight, eps, offset)
    input_dtype = hidden_states.dtype
    h = hidden_states.to(torch.float32)
    variance = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(variance + eps)
    return ((weight.float() + offset) * h).to(input_dtype)


def gemma_rms_norm_forward(self, hidden_states):
    self._ipex_weight_offset = 1.0
    return rms_norm_forward(self, hidden_states)


def layer_norm_forward(self, hidden_states: torch.Tensor):
    if hidden_states.is_cuda and not hidden_states.requires_grad and self.weight is not None and \
            hidden_states.dtype in (torch.float16, torch.bfloat16):
        from ..ops import cuda_ops
        return cuda_ops.layer_norm(hidden_states, self.weight, self.bias, self.eps)
    return F.layer_norm(hidden_states, self.normalized_shape, self.weight, self.bias, self.eps)


# ------------------------------------------------------------------------------------------------
# MLP
# ------------------------------------------------------------------------------------------------
def _act_mul(gate: torch.Tensor, up: torch.Tensor, act: int):
    if gate.is_cuda and not gate.requires_grad and gate.dtype in (torch.float16, torch.bfloat16):
        from ..ops import cuda_ops
        return cuda_ops.act_mul(gate, up, act)
    if act == SILU:
        return F.silu(gate) * up
    return F.gelu(gate, approximate="tanh") * up


def fuse_mlp_base(module: nn.Module, act: int, x: torch.Tensor):
    """down(act(gate(x)) * up(x)); a merged ``gate_up_proj`` (if the converter built one) is used as one GEMM."""
    if hasattr(module, "gate_up_proj") and isinstance(module.gate_up_proj, nn.Module):
        gu = module.gate_up_proj(x)
        gate, up = gu.chunk(2, dim=-1)
        return module.down_proj(_act_mul(gate.contiguous(), up.contiguous(), act))
    return module.down_proj(_act_mul(module.gate_proj(x), module.up_proj(x), act))


def mlp_silu_forward(self, x: torch.Tensor, *args, **kwargs):
    return fuse_mlp_base(self, SILU, x)


def mlp_gelu_forward(self, x: torch.Tensor, *args, **kwargs):
    return fuse_mlp_base(self, GELU, x)


# ------------------------------------------------------------------------------------------------
# rotary embedding
# ------------------------------------------------------------------------------------------------
def rotate_half(x):
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1, interleaved=False):
    """RoPE on q and k (``[B, H, S, D]``); ``cos``/``sin`` are ``[B, S, R]`` with R <= D (partial rotary).
    ``interleaved`` selects the GPT-J "two" pairing instead of the NeoX "half" pairing."""
    if q.is_cuda and not q.requires_grad and q.dtype in (torch.float16, torch.bfloat16) and cos.dim() == 3:
        from ..ops import cuda_ops
        return cuda_ops.rotary_inplace(q, k, cos, sin, interleaved)
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    rot = cos.shape[-1]

    def _apply(x):
        xr, xp = x[..., :rot], x[..., rot:]
        if interleaved:
            x1 = xr[..., 0::2]
            x2 = xr[..., 1::2]
            # GPT-J tables repeat every frequency twice (f0, f0, f1, f1, ...): take one of each pair
            c = cos[..., 0::2]
            s = sin[..., 0::2]
            o = torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).flatten(-2)
        else:
            o = xr * cos + rotate_half(xr) * sin
        return torch.cat((o.to(x.dtype), xp), dim=-1) if xp.shape[-1] else o.to(x.dtype)

    return _apply(q), _apply(k)


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
def attention_softmax(attn_weights: torch.Tensor):
    if attn_weights.is_cuda and attn_weights.is_contiguous() and not attn_weights.requires_grad and \
            attn_weights.dtype in (torch.float16, torch.bfloat16, torch.float32):
        from ..ops import cuda_ops
        return cuda_ops.softmax_inplace(attn_weights)
    return F.softmax(attn_weights, dim=-1, dtype=torch.float32).to(attn_weights.dtype)


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    if n_rep == 1:
        return hidden_states
    b, h, s, d = hidden_states.shape
    return hidden_states[:, :, None, :, :].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)


def scaled_dot_product_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                 mask: torch.Tensor = None, is_causal: bool = False, scale: float = None,
                                 softcap: float = None, sliding_window: int = None,
                                 infer_causal: bool = True) -> torch.Tensor:
    """softmax(q k^T * scale + mask) v with GQA handled inside.

    ``query`` is ``[B, Hq, Sq, D]``; ``key``/``value`` are ``[B, Hkv, Skv, D]`` in the activation dtype or packed
    e5m2 bytes (uint8).  Routing (reference models/common.py:249-305): short queries against a long cache
    (decode, speculative verification, lookup: Sq <= 32) go to the split-KV decode kernel, which reads fp8 KV
    directly; everything else goes to the prefill path.  With ``infer_causal`` (the decoder forwards of this
    package) a missing mask on a multi-token query means causal; encoders and cross-attention pass False and get
    exactly ``is_causal``."""
    bsz, n_heads, q_len, head_dim = query.shape
    kv_len = key.shape[2]
    n_kv = key.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    fp8 = key.dtype == torch.uint8
    causal = bool(is_causal) or (infer_causal and mask is None and q_len > 1)

    if query.is_cuda and not query.requires_grad and query.dtype in (torch.float16, torch.bfloat16):
        from ..ops import cuda_ops
        if q_len <= 32 and cuda_ops.sdpa_decode_supported(head_dim, value.shape[-1]):
            return cuda_ops.sdpa_decode(query, key, value, mask, scale, softcap, sliding_window, causal=causal)
        if fp8:
            key = fp8_e5m2_dequantize(key, query.dtype)
            value = fp8_e5m2_dequantize(value, query.dtype)
        return cuda_ops.sdpa_prefill(query, key, value, mask, scale, softcap, sliding_window, causal=causal)

    if fp8:
        key = fp8_e5m2_dequantize(key, query.dtype)
        value = fp8_e5m2_dequantize(value, query.dtype)
    key = repeat_kv(key, n_heads // n_kv)
    value = repeat_kv(value, n_heads // n_kv)
    if softcap is None and sliding_window is None:
        if mask is not None:
            mask = mask[..., :kv_len]
            if mask.dtype != torch.bool and mask.dtype != query.dtype:
                mask = mask.to(query.dtype)
        if mask is None and causal and q_len != kv_len:
            # a causal query block at the end of a longer cache (chunked prompt, verification of several tokens)
            qi = torch.arange(kv_len - q_len, kv_len, device=query.device).view(-1, 1)
            mask = torch.arange(kv_len, device=query.device).view(1, -1) <= qi
        return F.scaled_dot_product_attention(query, key, value, attn_mask=mask, scale=scale,
                                              is_causal=(mask is None and causal))
    # eager path (soft-capped logits, sliding window)
    w = torch.matmul(query.float(), key.float().transpose(2, 3)) * scale
    if softcap is not None:
        w = torch.tanh(w / softcap) * softcap
    if mask is not None:
        m = mask[..., :kv_len]
        w = w.masked_fill(~m, float("-inf")) if m.dtype == torch.bool else w + m.float()
    elif causal or sliding_window is not None:
        qi = torch.arange(kv_len - q_len, kv_len, device=w.device).view(-1, 1)
        ki = torch.arange(kv_len, device=w.device).view(1, -1)
        allowed = ki <= qi if causal else torch.ones(q_len, kv_len, dtype=torch.bool, device=w.device)
        if sliding_window is not None:
            allowed = allowed & (ki > qi - sliding_window)
        w = w.masked_fill(~allowed, float("-inf"))
    # a query row that may see no key at all (the rows of left padding under a sliding window) softmaxes to NaN,
    # which would then leak into real rows through the next layer's keys: such rows attend to nothing instead
    w = torch.nan_to_num(torch.softmax(w, dim=-1), nan=0.0)
    return torch.matmul(w, value.float()).to(query.dtype)


def t5_dense_forward(self, hidden_states):
    """``T5DenseActDense`` / ``T5DenseGatedActDense`` without the cast of the activations to ``wo.weight.dtype``: a
    packed weight is a byte tensor, and the original forward would turn the hidden states into bytes."""
    if hasattr(self, "wi_0"):
        hidden_states = self.act(self.wi_0(hidden_states)) * self.wi_1(hidden_states)
    else:
        hidden_states = self.act(self.wi(hidden_states))
    return self.wo(self.dropout(hidden_states))


# ------------------------------------------------------------------------------------------------
# attention interface of transformers 5: every model whose attention goes through ALL_ATTENTION_FUNCTIONS
# ------------------------------------------------------------------------------------------------
ATTN_INTERFACE_NAME = "ipex_llm"


def attention_interface(module, query, key, value, attention_mask=None, dropout: float = 0.0, scaling=None,
                        is_causal=None, softcap=None, sliding_window=None, **kwargs):
    """The package's SDPA behind the transformers attention-interface contract: ``query [B, Hq, Sq, D]``,
    ``key`` / ``value [B, Hkv, Skv, D]`` (already read back from the cache), returns ``([B, Sq, Hq, Dv], None)``.

    This is how the families that the reference patches file by file (whisper, bert, mllama, qwen2_vl, deepseek,
    starcoder2, stablelm, gpt_neox, bloom, ... python/llm/src/ipex_llm/transformers/convert.py:1303-2040) reach the
    native attention kernels here without a forward of their own."""
    if is_causal is None:
        is_causal = query.shape[2] > 1 and attention_mask is None and getattr(module, "is_causal", True)
    mask = attention_mask
    if mask is not None and mask.dim() == 4 and mask.shape[-1] > key.shape[2]:
        mask = mask[..., : key.shape[2]]
    if dropout and module.training:
        # training with attention dropout keeps the library path
        import torch.nn.functional as F_
        k2, v2 = repeat_kv(key, query.shape[1] // key.shape[1]), repeat_kv(value, query.shape[1] // key.shape[1])
        out = F_.scaled_dot_product_attention(query, k2, v2, attn_mask=mask, dropout_p=dropout, scale=scaling,
                                              is_causal=bool(is_causal) and mask is None)
        return out.transpose(1, 2).contiguous(), None
    out = scaled_dot_product_attention(query, key, value, mask, is_causal=bool(is_causal), scale=scaling,
                                       softcap=softcap, sliding_window=sliding_window, infer_causal=False)
    return out.transpose(1, 2).contiguous(), None


def register_attention_interface() -> bool:
    """Register ``attention_interface`` under the name ``ipex_llm``; False when transformers has no such registry."""
    try:
        from transformers import AttentionInterface
    except ImportError:
        return False
    try:
        AttentionInterface.register(ATTN_INTERFACE_NAME, attention_interface)
        try:   # masks are built as for the sdpa path
            from transformers import AttentionMaskInterface
            from transformers.masking_utils import sdpa_mask
            AttentionMaskInterface.register(ATTN_INTERFACE_NAME, sdpa_mask)
        except Exception:  # noqa: BLE001
            pass
        return True
    except Exception:  # noqa: BLE001
        return False


def _uses_attention_registry(mod) -> bool:
    """Does the modeling file of this module dispatch its attention through the interface registry?  Files that do
    import ``ALL_ATTENTION_FUNCTIONS``; the others (GPT-J, CodeGen, ...) run their own eager attention and only
    read ``_attn_implementation`` to build the mask, which must then stay in the additive form they expect."""
    import sys
    pymod = sys.modules.get(type(mod).__module__)
    return pymod is not None and hasattr(pymod, "ALL_ATTENTION_FUNCTIONS")


def use_attention_interface(model) -> bool:
    """Point every sub-model whose attention goes through the registry at the registered interface; the rest keep
    their own attention path and mask format."""
    if not register_attention_interface():
        return False
    done = False
    seen = set()
    for mod in model.modules():
        cfg = getattr(mod, "config", None)
        if cfg is None or id(cfg) in seen or not hasattr(cfg, "to_dict"):
            continue
        if not _uses_attention_registry(mod):
            continue
        seen.add(id(cfg))
        try:
            cfg._attn_implementation = ATTN_INTERFACE_NAME
            done = True
        except Exception:  # noqa: BLE001
            pass
    return done
