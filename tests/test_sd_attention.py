"""Stable-Diffusion attention processor: a UNet-style attention block (duck-typed like diffusers' ``Attention``) run
through ``AttnProcessor2_0`` equals the plain softmax(QK^T)V formulation; ``optimize_model`` installs it on a pipeline."""
import math

import torch
from torch import nn


class _Attention(nn.Module):
    """The attributes of ``diffusers.models.attention_processor.Attention`` that a processor reads."""

    def __init__(self, dim, heads, cross_dim=None, group_norm=False, residual=False, rescale=1.0):
        super().__init__()
        self.heads, self.scale = heads, 1.0 / math.sqrt(dim // heads)
        self.to_q = nn.Linear(dim, dim, bias=False)
        self.to_k = nn.Linear(cross_dim or dim, dim, bias=False)
        self.to_v = nn.Linear(cross_dim or dim, dim, bias=False)
        self.to_out = nn.ModuleList([nn.Linear(dim, dim), nn.Dropout(0.0)])
        self.group_norm = nn.GroupNorm(4, dim) if group_norm else None
        self.spatial_norm, self.norm_cross, self.norm_q, self.norm_k = None, None, None, None
        self.residual_connection, self.rescale_output_factor = residual, rescale
        self.processor = None

    def prepare_attention_mask(self, mask, target_length, batch_size):
        return mask.repeat_interleave(self.heads, dim=0)

    def forward(self, x, encoder_hidden_states=None, attention_mask=None):
        return self.processor(self, x, encoder_hidden_states=encoder_hidden_states, attention_mask=attention_mask)


def _plain(attn, x, ctx=None, mask=None):
    residual = x
    spatial = x.dim() == 4
    if spatial:
        b, c, h, w = x.shape
        x = x.view(b, c, h * w).transpose(1, 2)
    if attn.group_norm is not None:
        x = attn.group_norm(x.transpose(1, 2)).transpose(1, 2)
    ctx = x if ctx is None else ctx
    B, H = x.shape[0], attn.heads
    q = attn.to_q(x).view(B, -1, H, x.shape[-1] // H).transpose(1, 2)
    k = attn.to_k(ctx).view(B, -1, H, x.shape[-1] // H).transpose(1, 2)
    v = attn.to_v(ctx).view(B, -1, H, x.shape[-1] // H).transpose(1, 2)
    w_ = (q @ k.transpose(-1, -2)) * attn.scale
    if mask is not None:
        w_ = w_ + mask[:, None]
    o = (torch.softmax(w_, -1) @ v).transpose(1, 2).reshape(B, -1, x.shape[-1])
    o = attn.to_out[0](o)
    if spatial:
        o = o.transpose(-1, -2).reshape(b, c, h, w)
    if attn.residual_connection:
        o = o + residual
    return o / attn.rescale_output_factor


def test_processor_matches_plain_attention():
    from ipex_llm_b200.models.sd import AttnProcessor2_0
    torch.manual_seed(0)
    proc = AttnProcessor2_0()
    # self-attention over a feature map (head dim 40 as in the SD 1.5 UNet), with group norm, residual and rescale
    a = _Attention(160, 4, group_norm=True, residual=True, rescale=2.0).eval()
    a.processor = proc
    x = torch.randn(2, 160, 6, 6)
    with torch.no_grad():
        assert torch.allclose(a(x), _plain(a, x), atol=1e-5)
    # cross-attention to 77 text tokens with an additive mask over the padding
    c = _Attention(128, 8, cross_dim=96).eval()
    c.processor = proc
    h, ctx = torch.randn(2, 36, 128), torch.randn(2, 77, 96)
    mask = torch.zeros(2, 1, 77)
    mask[1, :, 50:] = -10000.0
    with torch.no_grad():
        assert torch.allclose(c(h, ctx, mask), _plain(c, h, ctx, mask), atol=1e-5)


def test_optimize_model_installs_the_processor_on_a_pipeline():
    from ipex_llm import optimize_model
    from ipex_llm_b200.models.sd import AttnProcessor2_0
    from ipex_llm_b200.ops.linear import LowBitLinear

    class UNet(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn = _Attention(128, 4)

        def set_attn_processor(self, p):
            self.attn.processor = p

    class StableDiffusionXLPipeline:                    # a pipeline is not an nn.Module
        def __init__(self):
            self.unet, self.vae = UNet(), nn.Conv2d(4, 4, 1).half()
            self.text_encoder_2 = nn.Identity()

    pipe = optimize_model(StableDiffusionXLPipeline(), low_bit=None)
    assert isinstance(pipe.unet.attn.processor, AttnProcessor2_0)
    pipe.upcast_vae()
    assert pipe.vae.weight.dtype == torch.bfloat16
    pipe = optimize_model(StableDiffusionXLPipeline(), low_bit="sym_int8")
    assert isinstance(pipe.unet.attn.to_q, LowBitLinear) and isinstance(pipe.unet.attn.processor, AttnProcessor2_0)
    x = torch.randn(1, 9, 128)
    with torch.no_grad():
        assert torch.isfinite(pipe.unet.attn(x)).all()
