"""Generic forwards for rotary decoder-only transformers on the transformers-5 module interfaces.

Most families the reference patches one by one (llama, mistral, qwen2, gemma, glm, phi3, starcoder2,
stablelm, ... — python/llm/src/ipex_llm/transformers/models/*.py) share one attention contract in
transformers 5: ``forward(hidden_states, position_embeddings, attention_mask, past_key_values, **kw)
-> (attn_output, attn_weights)``.  One implementation therefore serves them all; per-family differences
are data on the module (``_ipex_attn``): optional q/k norms, soft-capped logits, sliding window, rotary
pairing, partial rotary, scaling override.

``decoder_attention_forward`` consumes the fused ``qkv_proj`` built by ``merge_qkv`` (one low-bit GEMM
instead of three), applies RoPE with the fused kernel, appends to the block-grown / fp8 KV cache and calls
the package's SDPA.  ``decoder_model_forward`` wraps the HF ``*Model.forward`` to pick the cache class, as
``llama_model_forward`` does in the reference (models/llama.py:56-116).
"""
from __future__ import annotations

import math

import torch

from ..ops.kv_cache import CompressLayer, is_ipex_cache
from .common import apply_rotary_pos_emb, scaled_dot_product_attention
from .utils import select_cache


class AttnSpec:
    """Per-family attention details."""

    def __init__(self, interleaved_rope=False, softcap_attr=None, sliding=False, qk_norm=False,
                 scaling_attr="scaling", query_pre_attn_scalar=False):
        self.interleaved_rope = interleaved_rope
        self.softcap_attr = softcap_attr
        self.sliding = sliding
        self.qk_norm = qk_norm
        self.scaling_attr = scaling_attr


DEFAULT_SPEC = AttnSpec()


def _split_heads(self, hidden_states):
    bsz, q_len, _ = hidden_states.shape
    hd = self.head_dim
    if hasattr(self, "qkv_proj"):
        qkv = self.qkv_proj(hidden_states)
        total = qkv.shape[-1] // hd
        groups = getattr(self, "num_key_value_groups", 1)
        n_kv = total // (groups + 2)
        n_q = total - 2 * n_kv
        qkv = qkv.view(bsz, q_len, total, hd).transpose(1, 2)
        q, k, v = qkv.split([n_q, n_kv, n_kv], dim=1)
    else:
        q = self.q_proj(hidden_states).view(bsz, q_len, -1, hd).transpose(1, 2)
        k = self.k_proj(hidden_states).view(bsz, q_len, -1, hd).transpose(1, 2)
        v = self.v_proj(hidden_states).view(bsz, q_len, -1, hd).transpose(1, 2)
    return q, k, v


def alibi_slopes(n_heads: int) -> torch.Tensor:
    """Per-head slopes of "attention with linear biases": a geometric series for a power-of-two head count, and for
    other counts the series of the next lower power of two followed by every other slope of the next higher one
    (Baichuan-13B has 40 heads; reference models/baichuan.py:403-447 builds the same mask)."""
    def series(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]
    if math.log2(n_heads).is_integer():
        vals = series(n_heads)
    else:
        low = 2 ** math.floor(math.log2(n_heads))
        vals = series(low) + series(2 * low)[0::2][: n_heads - low]
    return torch.tensor(vals, dtype=torch.float32)


def alibi_mask(n_heads, q_len, kv_len, mask, dtype, device):
    """Additive ``[B or 1, H, q_len, kv_len]`` mask: slope_h * (key position - last position) plus the causal /
    padding mask.  Soft-max is invariant to a shift per row, so the distance to the query reduces to the key position;
    counting from the last key keeps the magnitudes small near the diagonal of a decode step."""
    slopes = alibi_slopes(n_heads).to(device)
    kj = torch.arange(kv_len, device=device, dtype=torch.float32)
    bias = slopes.view(1, n_heads, 1, 1) * (kj - (kv_len - 1)).view(1, 1, 1, kv_len)
    if mask is None:
        qi = torch.arange(kv_len - q_len, kv_len, device=device).view(q_len, 1)
        allowed = (kj.view(1, kv_len) <= qi).view(1, 1, q_len, kv_len)
        bias = bias.expand(1, n_heads, q_len, kv_len).masked_fill(~allowed, float("-inf"))
    elif mask.dtype == torch.bool:
        bias = bias.expand(mask.shape[0], n_heads, q_len, kv_len).masked_fill(~mask, float("-inf"))
    else:
        bias = bias + mask.float()
    return bias.to(dtype)


def decoder_attention_forward(self, hidden_states, position_embeddings=None, attention_mask=None,
                              past_key_values=None, **kwargs):
    spec: AttnSpec = getattr(self, "_ipex_attn", DEFAULT_SPEC)
    bsz, q_len, _ = hidden_states.shape
    q, k, v = _split_heads(self, hidden_states)

    if spec.qk_norm and hasattr(self, "q_norm"):
        q = self.q_norm(q)
        k = self.k_norm(k)

    alibi = bool(getattr(self.config, "ipex_alibi", False))
    if position_embeddings is not None and not alibi:
        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin, interleaved=spec.interleaved_rope)

    if past_key_values is not None:
        layer_idx = self.layer_idx
        extra = {}
        if is_ipex_cache(past_key_values):
            while len(past_key_values.layers) <= layer_idx:
                past_key_values.layers.append(past_key_values.layer_class_to_replicate())
            if isinstance(past_key_values.layers[layer_idx], CompressLayer):
                extra = dict(query_states=q, attention_mask=attention_mask,
                             num_key_value_groups=q.shape[1] // k.shape[1])
        k, v = past_key_values.update(k, v, layer_idx, **extra)

    softcap = getattr(self, spec.softcap_attr, None) if spec.softcap_attr else None
    if softcap is None and spec.softcap_attr:
        softcap = getattr(self.config, spec.softcap_attr, None)
    sliding_window = getattr(self, "sliding_window", None) if spec.sliding else None
    scaling = getattr(self, spec.scaling_attr, None)
    kv_len = k.shape[2]
    mask = attention_mask
    if mask is not None and mask.dim() == 4 and mask.shape[-1] != kv_len:
        mask = mask[..., :kv_len] if mask.shape[-1] > kv_len else None
    if alibi:
        mask = alibi_mask(q.shape[1], q_len, kv_len, mask, q.dtype, q.device)
    attn_output = scaled_dot_product_attention(q, k, v, mask, is_causal=(mask is None and q_len > 1),
                                               scale=scaling, softcap=softcap, sliding_window=sliding_window)
    attn_output = attn_output.transpose(1, 2).reshape(bsz, q_len, -1).contiguous()
    attn_output = self.o_proj(attn_output)
    return attn_output, None


def decoder_model_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                          inputs_embeds=None, use_cache=None, **kwargs):
    """Instance-bound replacement of ``*Model.forward``: choose the cache class, then run the HF forward."""
    use_cache = use_cache if use_cache is not None else getattr(self.config, "use_cache", True)
    ref = inputs_embeds if inputs_embeds is not None else input_ids
    if use_cache and ref is not None and not self.training:
        probe = torch.empty((ref.shape[0], ref.shape[1], 0), device=ref.device)
        past_key_values = select_cache(self.config, probe, past_key_values)
    return type(self).forward(self, input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                              past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache,
                              **kwargs)
