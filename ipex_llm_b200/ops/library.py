"""``torch.library`` registrations: the package's kernels as ``torch.ops.ipex_llm.*`` with fake-tensor kernels.

The reference registers fake tensors for the ops of its closed extensions so that a converted model can go through
``torch.compile`` graph capture (python/llm/src/ipex_llm/transformers/xpu_ops.py:23-162; example
python/llm/example/GPU/GraphMode/gpt2-graph-mode-benchmark.py:87-103).  Here each op is a ``torch.library.custom_op``
over the CUDA launchers of ``ops.cuda_ops`` (with a PyTorch restatement on CPU tensors), plus a ``register_fake``
shape function with the reference's op names and argument order.  Packed weights are passed as the raw byte tensor
in the device layout together with their qtype id and shape, which is what a traced graph can carry.
"""
from __future__ import annotations

import torch

_LIB = "ipex_llm"
_registered = False


def _weight_view(weight: torch.Tensor, qtype: int, n: int, k: int):
    from ..quant.params import FP4Params
    return FP4Params(weight, requires_grad=False, quantized=True, _shape=torch.Size((n, k)), qtype=int(qtype),
                     layout="device" if weight.is_cuda else "canonical")


def register() -> bool:
    """Idempotent; returns False on a torch without ``torch.library.custom_op``."""
    global _registered
    if _registered:
        return True
    if not hasattr(torch.library, "custom_op"):
        return False
    from . import cuda_ops

    @torch.library.custom_op(f"{_LIB}::forward_new", mutates_args=())
    def forward_new(x: torch.Tensor, weight: torch.Tensor, qtype: int, output_size: int) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        w = _weight_view(weight, qtype, output_size, x2.shape[-1])
        if x2.is_cuda:
            return cuda_ops.lowbit_linear(x2.contiguous(), w)
        return torch.nn.functional.linear(x2.float(), w.dequantize(torch.float32)).to(x.dtype)

    @forward_new.register_fake
    def _(x, weight, qtype, output_size):
        return torch.empty([x.reshape(-1, x.shape[-1]).size(0), output_size], dtype=x.dtype, device=x.device)

    @torch.library.custom_op(f"{_LIB}::batch_forward", mutates_args=())
    def batch_forward(x: torch.Tensor, weight: torch.Tensor, qtype: int, output_size: int) -> torch.Tensor:
        return forward_new(x, weight, qtype, output_size)

    @batch_forward.register_fake
    def _(x, weight, qtype, output_size):
        return torch.empty([x.reshape(-1, x.shape[-1]).size(0), output_size], dtype=x.dtype, device=x.device)

    @torch.library.custom_op(f"{_LIB}::dequant", mutates_args=())
    def dequant(x: torch.Tensor, weight: torch.Tensor, qtype: int, rows: int, cols: int) -> torch.Tensor:
        w = _weight_view(weight, qtype, rows, cols)
        if weight.is_cuda:
            return cuda_ops.dequantize_device(weight, (rows, cols), qtype, x.dtype)
        return w.dequantize(x.dtype)

    @dequant.register_fake
    def _(x, weight, qtype, rows, cols):
        return torch.empty([rows, cols], dtype=x.dtype, device=weight.device)

    @torch.library.custom_op(f"{_LIB}::mlp_forward_xpu", mutates_args=())
    def mlp_forward_xpu(x: torch.Tensor, weight1: torch.Tensor, weight2: torch.Tensor, batch_size: int,
                        state_size: int, output_size: int, act_type: int, qtype: int) -> torch.Tensor:
        g = forward_new(x, weight1, qtype, output_size)
        u = forward_new(x, weight2, qtype, output_size)
        if g.is_cuda:
            return cuda_ops.act_mul(g, u, 1 if act_type == 0 else 2)
        a = torch.nn.functional.silu(g.float()) if act_type == 0 else torch.nn.functional.gelu(g.float())
        return (a * u.float()).to(x.dtype)

    @mlp_forward_xpu.register_fake
    def _(x, weight1, weight2, batch_size, state_size, output_size, act_type, qtype):
        return torch.empty([batch_size, output_size], dtype=x.dtype, device=x.device)

    @torch.library.custom_op(f"{_LIB}::rms_norm", mutates_args=())
    def rms_norm(weight: torch.Tensor, x: torch.Tensor, eps: float) -> torch.Tensor:
        if x.is_cuda:
            return cuda_ops.rms_norm(x.contiguous(), weight, eps)
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)

    @rms_norm.register_fake
    def _(weight, x, eps):
        return torch.empty_like(x)

    @torch.library.custom_op(f"{_LIB}::layer_norm", mutates_args=())
    def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
        if x.is_cuda:
            return cuda_ops.layer_norm(x.contiguous(), weight, bias, eps)
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)

    @layer_norm.register_fake
    def _(x, weight, bias, eps):
        return torch.empty_like(x)

    @torch.library.custom_op(f"{_LIB}::mlp_silu_mul_inplaced", mutates_args=("gate",))
    def mlp_silu_mul_inplaced(gate: torch.Tensor, up: torch.Tensor) -> None:
        if gate.is_cuda:
            gate.copy_(cuda_ops.act_mul(gate, up, 1))
        else:
            gate.copy_((torch.nn.functional.silu(gate.float()) * up.float()).to(gate.dtype))

    @mlp_silu_mul_inplaced.register_fake
    def _(gate, up):
        return None

    @torch.library.custom_op(f"{_LIB}::sdp", mutates_args=())
    def sdp(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, mask: torch.Tensor | None = None,
            scale: float | None = None) -> torch.Tensor:
        from ..models.common import scaled_dot_product_attention
        return scaled_dot_product_attention(query, key, value, mask, False, scale, infer_causal=False)

    @sdp.register_fake
    def _(query, key, value, mask=None, scale=None):
        return torch.empty(query.shape[:-1] + (value.shape[-1],), dtype=query.dtype, device=query.device)

    @torch.library.custom_op(f"{_LIB}::sdp_causal", mutates_args=())
    def sdp_causal(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, mask: torch.Tensor | None = None,
                   scale: float | None = None) -> torch.Tensor:
        from ..models.common import scaled_dot_product_attention
        return scaled_dot_product_attention(query, key, value, mask, True, scale)

    @sdp_causal.register_fake
    def _(query, key, value, mask=None, scale=None):
        return torch.empty(query.shape[:-1] + (value.shape[-1],), dtype=query.dtype, device=query.device)

    @torch.library.custom_op(f"{_LIB}::quantize_key_value", mutates_args=())
    def quantize_key_value(x: torch.Tensor) -> torch.Tensor:
        from .kv_cache import fp8_e5m2_quantize
        return fp8_e5m2_quantize(x)

    @quantize_key_value.register_fake
    def _(x):
        return torch.empty(x.shape, dtype=torch.uint8, device=x.device)

    @torch.library.custom_op(f"{_LIB}::attn_softmax_inplaced", mutates_args=("attn_weights",))
    def attn_softmax_inplaced(attn_weights: torch.Tensor) -> None:
        from ..models.common import attention_softmax
        out = attention_softmax(attn_weights)
        if out.data_ptr() != attn_weights.data_ptr():
            attn_weights.copy_(out)

    @attn_softmax_inplaced.register_fake
    def _(attn_weights):
        return None

    _registered = True
    return True
