"""Stable-Diffusion pipelines: the attention processor that puts UNet self- and cross-attention on the package's
SDPA, and the VAE precision fix for SDXL.

Counterpart of python/llm/src/ipex_llm/transformers/models/sd.py:45-160 and the pipeline branch of
python/llm/src/ipex_llm/transformers/convert.py:1253-1265.  The processor follows the diffusers attention-processor
protocol by duck typing (``attn.to_q / to_k / to_v / to_out / heads / group_norm / spatial_norm / norm_cross /
residual_connection / rescale_output_factor``), so diffusers itself is only needed by the caller that owns the
pipeline.  UNet attention is never causal and its mask, when there is one, is an additive bias over the text tokens.

On a B200 the VAE fix is simply bfloat16 for the whole VAE: the fp16 overflow of the SDXL decoder is a range problem,
bf16 has the fp32 exponent, and the tensor cores run it at the fp16 rate.
"""
from __future__ import annotations

import torch

from .common import scaled_dot_product_attention


class AttnProcessor2_0:
    """Drop-in for ``diffusers.models.attention_processor.AttnProcessor2_0``."""

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: torch.Tensor = None,
                 attention_mask: torch.Tensor = None, temb: torch.Tensor = None, *args, **kwargs) -> torch.Tensor:
        residual = hidden_states
        if getattr(attn, "spatial_norm", None) is not None:
            hidden_states = attn.spatial_norm(hidden_states, temb)
        spatial = hidden_states.dim() == 4
        if spatial:
            b, c, h, w = hidden_states.shape
            hidden_states = hidden_states.view(b, c, h * w).transpose(1, 2)
        context = hidden_states if encoder_hidden_states is None else encoder_hidden_states
        bsz, kv_len = context.shape[0], context.shape[1]
        if attention_mask is not None:
            # [B * heads, 1 or Sq, Skv] from the pipeline -> [B, heads, Sq, Skv]
            attention_mask = attn.prepare_attention_mask(attention_mask, kv_len, bsz)
            attention_mask = attention_mask.view(bsz, attn.heads, -1, attention_mask.shape[-1])
        if getattr(attn, "group_norm", None) is not None:
            hidden_states = attn.group_norm(hidden_states.transpose(1, 2)).transpose(1, 2)
            if encoder_hidden_states is None:
                context = hidden_states
        if encoder_hidden_states is not None and getattr(attn, "norm_cross", None):
            context = attn.norm_encoder_hidden_states(encoder_hidden_states)

        q = attn.to_q(hidden_states)
        k = attn.to_k(context)
        v = attn.to_v(context)
        head_dim = k.shape[-1] // attn.heads
        q = q.view(bsz, -1, attn.heads, head_dim).transpose(1, 2)
        k = k.view(bsz, -1, attn.heads, head_dim).transpose(1, 2)
        v = v.view(bsz, -1, attn.heads, head_dim).transpose(1, 2)
        if getattr(attn, "norm_q", None) is not None:
            q = attn.norm_q(q)
        if getattr(attn, "norm_k", None) is not None:
            k = attn.norm_k(k)
        scale = getattr(attn, "scale", None)
        out = scaled_dot_product_attention(q, k, v, attention_mask, is_causal=False, scale=scale, infer_causal=False)
        out = out.transpose(1, 2).reshape(bsz, -1, attn.heads * head_dim).to(q.dtype)

        out = attn.to_out[0](out)
        out = attn.to_out[1](out)                                   # dropout
        if spatial:
            out = out.transpose(-1, -2).reshape(b, c, h, w)
        if getattr(attn, "residual_connection", False):
            out = out + residual
        factor = getattr(attn, "rescale_output_factor", 1.0)
        return out / factor if factor != 1.0 else out


def upcast_vae(self):
    """Bound as ``pipeline.upcast_vae``: the SDXL VAE decodes in bfloat16 instead of overflowing in float16."""
    self.vae.to(torch.bfloat16)


def is_diffusion_pipeline(model) -> bool:
    """A diffusers pipeline by shape: not an ``nn.Module``, owns a ``unet`` that accepts attention processors."""
    unet = getattr(model, "unet", None)
    return not isinstance(model, torch.nn.Module) and unet is not None and hasattr(unet, "set_attn_processor")


def optimize_pipeline(pipe):
    """What ``optimize_model`` / ``_optimize_post`` do to a pipeline: UNet attention through the package's SDPA, and
    for SDXL (two text encoders) the VAE precision fix."""
    from types import MethodType
    pipe.unet.set_attn_processor(AttnProcessor2_0())
    if getattr(pipe, "text_encoder_2", None) is not None and getattr(pipe, "vae", None) is not None:
        pipe.upcast_vae = MethodType(upcast_vae, pipe)
    return pipe
