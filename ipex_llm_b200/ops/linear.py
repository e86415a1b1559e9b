"""Low-bit / half-precision linear modules.

Counterparts of the reference's ``LowBitLinear``, ``MatMulLowBit``, ``MatMulLowBitCPU``, ``FP16Linear``,
``BF16Linear`` and their vLLM variants (python/llm/src/ipex_llm/transformers/low_bit_linear.py:500-908).

Dispatch on a CUDA tensor (always the package's own sm_100a kernels, never a silent eager fallback):
  M <= 8 rows   -> tensor-core-fragment GEMV reading the tile layout (bandwidth bound)
  M  > 8 rows   -> tcgen05/TMEM GEMM with in-kernel dequantization
On the CPU the packed canonical blocks go through the host library's low-bit matmul.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F
from torch import nn

from ..quant import qtypes as qt
from ..quant.params import FP4Params, ggml_matmul_src1_x_src0_t

TORCH_LINEAR_THRESHOLD = int(os.getenv("BIGDL_LLM_LINEAR_THRESHOLD", "512"))


def reshape_lm_head_input(x: torch.Tensor) -> torch.Tensor:
    """Only the last position goes through lm_head (reference low_bit_linear.py:262-269)."""
    if x.dim() < 3:
        return x            # [tokens, hidden] from a serving engine that already selected the positions it wants
    if x.dim() > 3:
        x = x.reshape([-1, x.shape[-2], x.shape[-1]])
    shape = list(x.size())
    if shape[1] > 10:
        shape[1] = 1
        x = x[:, -1, :].view(shape)
    return x


def _gather_last_dim(t: torch.Tensor, module):
    """Vocabulary-parallel layers (``tp_gather`` set by the converter) return their slice of the output features;
    the full tensor is the concatenation over the group."""
    grp = getattr(module, "tp_gather", None)
    if grp is None or getattr(grp, "world_size", 1) <= 1:
        return t
    return grp.all_gather_last_dim(t)


def _all_reduce(t: torch.Tensor, mp_group):
    """Row-parallel output reduction.  ``mp_group`` may be a torch ProcessGroup, an object with an
    ``all_reduce`` method (vLLM GroupCoordinator style) or a ``TPGroup`` of this package."""
    if mp_group is None:
        return t
    if hasattr(mp_group, "all_reduce") and not isinstance(mp_group, torch.distributed.ProcessGroup):
        return mp_group.all_reduce(t)
    torch.distributed.all_reduce(t, group=mp_group)
    return t


class MatMulLowBit(torch.autograd.Function):
    """``y = x @ dequant(W).T`` with gradient for x only (frozen base weight, QLoRA)."""

    @staticmethod
    def forward(ctx, A, weight, output_size):
        ctx.is_empty = False
        from . import cuda_ops
        result = cuda_ops.lowbit_linear(A, weight)
        if any(ctx.needs_input_grad[:2]):
            ctx.weight = weight
        else:
            ctx.weight = None
        return result

    @staticmethod
    def backward(ctx, grad_output):
        req_gradA = ctx.needs_input_grad[0]
        grad_A = None
        if req_gradA:
            from . import cuda_ops
            grad_A = cuda_ops.lowbit_linear_backward(grad_output, ctx.weight)
        return grad_A, None, None


class MatMulLowBitCPU(torch.autograd.Function):

    @staticmethod
    def forward(ctx, A, weight):
        raw = weight.data if weight.data.dtype == torch.uint8 else weight.data.view(torch.uint8)
        result = ggml_matmul_src1_x_src0_t(raw, A.detach(), weight._shape, weight.qtype).to(A.dtype)
        if any(ctx.needs_input_grad[:2]):
            ctx.weight = weight
        else:
            ctx.weight = None
        return result

    @staticmethod
    def backward(ctx, grad_output):
        grad_A = None
        if ctx.needs_input_grad[0]:
            w = ctx.weight.dequantize(grad_output.dtype)
            grad_A = torch.matmul(grad_output, w)
        return grad_A, None


class LowBitLinear(nn.Linear):
    """``nn.Linear`` whose weight is an ``FP4Params`` of any block qtype."""

    def __init__(self, input_features, output_features, qtype, bias=True, conver_to_half=True, mp_group=None,
                 optimize_lm_head=False, act_order=False, enable_scale_search=False):
        super().__init__(input_features, output_features, bias, device="meta")
        self.weight = FP4Params(torch.empty(0), requires_grad=False, quantized=False, _shape=None, qtype=qtype,
                                enable_scale_search=enable_scale_search)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_features), requires_grad=False)
        self.in_len = input_features
        self.out_len = output_features
        self.weight_shape = (self.out_len, self.in_len)
        self.weight_length = self.out_len * self.in_len
        self.qtype = qtype
        self.conver_to_half = conver_to_half
        self.mp_group = mp_group
        self.compute_dtype = None  # only for training
        self.optimize_lm_head = optimize_lm_head
        self.device = None  # detected only once in the first forward
        self.act_order = act_order
        self.is_lm_head = optimize_lm_head
        self.disable_fp16_opt = False
        if act_order:
            self.register_buffer("g_idx_map", torch.arange(self.in_len, dtype=torch.int64), persistent=False)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        key = prefix + "weight"
        found = key in state_dict
        if found and isinstance(self.weight, FP4Params):
            data = state_dict[key]
            w = self.weight
            shape = w._shape if w._shape is not None else torch.Size(self.weight_shape)
            from ..quant.params import packed_nbytes
            want = packed_nbytes(int(shape[0]) * int(shape[1]), w.qtype)
            got = data.numel() * data.element_size()
            if got != want:   # a truncated or foreign tensor must fail at load time, not at the first forward
                error_msgs.append(f"size mismatch for {key}: packed {qt.qtype_name(w.qtype)} weight of shape "
                                  f"{tuple(shape)} needs {want} bytes, the checkpoint holds {got}")
                return
            self._parameters["weight"] = FP4Params(data.detach(), requires_grad=False, quantized=True,
                                                   _shape=torch.Size(shape), qtype=w.qtype, layout="canonical")
            state_dict = {k: v for k, v in state_dict.items() if k != key}
        # `strict` is forwarded as given: Module.load_state_dict passes True at this level even for a non-strict
        # load, and that is what fills missing_keys, so a packed weight or bias that is absent from the checkpoint
        # is reported instead of leaving an empty parameter behind.
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)
        if found and key in missing_keys:     # the packed weight was installed above from the original dict
            missing_keys.remove(key)

    def forward(self, x: torch.Tensor):
        # empty tensor support (MoE experts that receive no token)
        if self.training and x.requires_grad and self.compute_dtype is not None:
            x = x.to(self.compute_dtype)
        if self.bias is not None and self.bias.dtype != x.dtype:
            self.bias.data = self.bias.data.to(x.dtype)
        if self.optimize_lm_head and os.environ.get("IPEX_LLM_LAST_LM_HEAD", "1") != "0":
            x = reshape_lm_head_input(x)
        x_shape = x.shape
        new_shape = x_shape[:-1] + (self.out_len,)
        x_2d = x.contiguous().view(-1, x_shape[-1])
        if self.act_order:
            x_2d = x_2d[:, self.g_idx_map]
        w = self.weight
        if x_2d.shape[0] == 0:
            return torch.empty(new_shape, dtype=x.dtype, device=x.device)
        if x_2d.is_cuda:
            if not (w.quantized and w.data.is_cuda):
                raise RuntimeError("LowBitLinear: input is on cuda but the packed weight is not; call model.to('cuda')")
            if x_2d.requires_grad:
                result = MatMulLowBit.apply(x_2d, w, self.out_len)
            else:
                from . import cuda_ops
                # IPEX_LLM_LOW_MEM=1: give cached blocks back around the large products of a long prompt
                # (reference low_bit_linear.py:648-671)
                low_mem = x_2d.shape[0] >= 1024 and os.environ.get("IPEX_LLM_LOW_MEM", "0") == "1"
                if low_mem:
                    torch.cuda.empty_cache()
                result = cuda_ops.lowbit_linear(x_2d, w)
                if low_mem:
                    torch.cuda.empty_cache()
            result = result.view(new_shape)
            result = _all_reduce(result, self.mp_group)
            if self.bias is not None:
                result = result + self.bias
            return _gather_last_dim(result, self)
        # CPU
        if not w.quantized:
            w = w.quantize("cpu")
            self._parameters["weight"] = w
        if x_2d.requires_grad:
            result = MatMulLowBitCPU.apply(x_2d, w)
        elif x_2d.shape[0] >= TORCH_LINEAR_THRESHOLD:
            result = F.linear(x_2d.float(), w.dequantize(torch.float32)).to(x.dtype)
        else:
            result = ggml_matmul_src1_x_src0_t(w.data.view(torch.uint8) if w.data.dtype != torch.uint8 else w.data,
                                               x_2d, self.weight_shape, w.qtype).to(x.dtype)
        result = result.view(new_shape)
        result = _all_reduce(result, self.mp_group)
        if self.bias is not None:
            result = result + self.bias
        return _gather_last_dim(result, self)

    def extra_repr(self):
        return (f"in_features={self.in_len}, out_features={self.out_len}, qtype={qt.qtype_name(self.qtype)}, "
                f"bias={self.bias is not None}")


class FP16Linear(nn.Linear):
    """fp16 "low_bit" mode (reference low_bit_linear.py:718-835).  On CUDA it runs the package's own
    half-precision GEMV (M <= 8) or tcgen05 GEMM."""

    compute_dtype = torch.float16

    def __init__(self, input_features, output_features, bias=True, mp_group=None, weight_type=1, optimize_lm_head=False):
        super().__init__(input_features, output_features, bias)
        self.in_len = input_features
        self.out_len = output_features
        self.weight_shape = (self.out_len, self.in_len)
        self.weight_length = self.out_len * self.in_len
        self.qtype = qt.FP16 if self.compute_dtype == torch.float16 else qt.BF16
        self.mp_group = mp_group
        self.weight_type = weight_type  # 1: [out, in] as stored by nn.Linear
        self.optimize_lm_head = optimize_lm_head
        self.disable_fp16_opt = False

    def forward(self, x: torch.Tensor):
        if self.optimize_lm_head and os.environ.get("IPEX_LLM_LAST_LM_HEAD", "1") != "0":
            x = reshape_lm_head_input(x)
        dt = self.compute_dtype
        x_in = x.to(dt)
        if self.weight.dtype != dt:
            self.weight.data = self.weight.data.to(dt)
        if self.bias is not None and self.bias.dtype != dt:
            self.bias.data = self.bias.data.to(dt)
        if x_in.is_cuda and not x_in.requires_grad and not self.weight.requires_grad:
            from . import cuda_ops
            x_2d = x_in.contiguous().view(-1, x_in.shape[-1])
            result = cuda_ops.dense_linear(x_2d, self.weight).view(*x_in.shape[:-1], self.out_len)
        else:
            result = F.linear(x_in, self.weight)
        result = _all_reduce(result, self.mp_group)
        if self.bias is not None:
            result = result + self.bias
        return _gather_last_dim(result, self).to(x.dtype)


class BF16Linear(FP16Linear):
    compute_dtype = torch.bfloat16


class vLLMLowBitLinear(LowBitLinear):
    def forward(self, x):
        return super().forward(x.to(torch.bfloat16) if x.dtype == torch.float32 else x), None


class vLLMFP16Linear(FP16Linear):
    def forward(self, x):
        return super().forward(x), None


class vLLMBF16Linear(BF16Linear):
    def forward(self, x):
        return super().forward(x), None
