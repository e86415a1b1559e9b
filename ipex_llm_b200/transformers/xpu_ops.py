"""Reference module path ``ipex_llm.transformers.xpu_ops`` (python/llm/src/ipex_llm/transformers/xpu_ops.py:23-162):
the reference registers fake tensors for the ops of its closed ``xe_linear`` / ``xe_addons`` extensions.  Importing
this module registers the same op names as ``torch.ops.ipex_llm.*`` custom ops with fake-tensor kernels
(``ops/library.py``), so graphs traced by ``torch.compile`` can carry them; the functions below are the eager
conveniences for code that called the extensions directly."""
import torch

from ..ops import library as _library

_library.register()

from ..ops import cuda_ops as _ops
from ..ops.rwkv import rwkv_linear_attention_v4, rwkv_linear_attention_v5, rwkv_time_shift  # noqa: F401


def forward_new(x: torch.Tensor, weight, qtype: int = None, output_size: int = None) -> torch.Tensor:
    """``x [M, K] @ dequant(weight).T``; ``weight`` is the layer's ``FP4Params``."""
    return _ops.lowbit_linear(x.reshape(-1, x.shape[-1]), weight)


def batch_forward(x: torch.Tensor, weight, qtype: int = None) -> torch.Tensor:
    return forward_new(x, weight, qtype)


def dequant(x: torch.Tensor, weight, qtype: int = None) -> torch.Tensor:
    return _ops.dequantize_device(weight.data, tuple(int(v) for v in weight._shape), weight.qtype, x.dtype)


def dequantize_rows(ids: torch.Tensor, weight, qtype: int, state_size: int, output_size: int) -> torch.Tensor:
    return _ops.dequantize_rows(ids, weight, state_size, output_size, torch.float32)


def rms_norm(weight: torch.Tensor, x: torch.Tensor, eps: float) -> torch.Tensor:
    return _ops.rms_norm(x, weight, eps)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    return _ops.layer_norm(x, weight, bias, eps)


def mlp_silu_mul_inplaced(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    gate.copy_(_ops.act_mul(gate, up, 1))
    return gate


def rotary_half_inplaced(inv_freq: torch.Tensor, position_ids: torch.Tensor, query: torch.Tensor,
                         key: torch.Tensor):
    """NeoX-layout RoPE on ``query`` / ``key`` ``[B, H, S, D]`` in place, angles from ``inv_freq`` x positions."""
    ang = position_ids[..., None].float() * inv_freq.float()
    cos, sin = torch.cat([ang.cos(), ang.cos()], dim=-1), torch.cat([ang.sin(), ang.sin()], dim=-1)
    _ops.rotary_inplace(query, key, cos, sin)


def attn_softmax_inplaced(attn_weights: torch.Tensor) -> torch.Tensor:
    from ..models.common import attention_softmax
    out = attention_softmax(attn_weights)
    if out.data_ptr() != attn_weights.data_ptr():
        attn_weights.copy_(out)
    return attn_weights


def sdp(query, key, value, mask=None, scale=None):
    from ..models.common import scaled_dot_product_attention
    return scaled_dot_product_attention(query, key, value, mask, False, scale)


def sdp_causal(query, key, value, mask=None, scale=None):
    from ..models.common import scaled_dot_product_attention
    return scaled_dot_product_attention(query, key, value, mask, True, scale)
