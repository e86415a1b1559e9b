"""AWQ / GPTQ checkpoint containers and unpackers.

``WQLinear_GEMM`` mirrors the buffer names and shapes AutoAWQ (and llm-awq) checkpoints carry so that their
state dicts load unchanged (reference python/llm/src/ipex_llm/transformers/awq/linear.py:70-130); the
unpackers turn the int32-packed 4-bit tensors of AWQ and GPTQ into plain code matrices which
``convert_gptq`` repacks into asym_int4 blocks (reference convert.py:379-453).
"""
from __future__ import annotations

import torch
from torch import nn

AWQ_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)   # nibble i of an AutoAWQ int32 holds column AWQ_ORDER^-1 ...
LLM_AWQ_ORDER = (0, 1, 2, 3, 4, 5, 6, 7)


class AwqBackendPackingMethod:
    AUTOAWQ = "autoawq"
    LLMAWQ = "llm-awq"


def _shifts(order, bits, device):
    return (torch.tensor(order, dtype=torch.int32, device=device) * bits)


def _zeros_width_llm_awq(in_features, group_size, pack_num=8):
    mult = {128: 1, 64: 2, 32: 4}.get(group_size)
    if mult is None:
        raise NotImplementedError(f"Not implemented group size {group_size}.")
    base = -(-(in_features // group_size) // pack_num)
    return -(-base // mult) * mult


class WQLinear_GEMM(nn.Module):
    def __init__(self, bits, group_size, in_features, out_features, bias, dev, backend=AwqBackendPackingMethod.AUTOAWQ):
        super().__init__()
        if bits != 4:
            raise NotImplementedError("Only 4-bit AWQ is supported.")
        self.in_features = in_features
        self.out_features = out_features
        self.w_bit = bits
        self.bits = bits
        self.group_size = group_size if group_size != -1 else in_features
        self.backend = backend
        if self.in_features % self.group_size != 0:
            raise ValueError(f"Invalid in_features number {in_features}.")
        pack = 32 // bits
        if out_features % pack != 0:
            raise ValueError(f"Invalid out_features number {out_features}.")
        if backend == AwqBackendPackingMethod.LLMAWQ:
            zw = _zeros_width_llm_awq(in_features, self.group_size)
            self.register_buffer("qweight", torch.zeros((out_features, in_features // pack), dtype=torch.int32, device=dev))
            self.register_buffer("qzeros", torch.zeros((out_features, zw), dtype=torch.int32, device=dev))
            self.register_buffer("scales", torch.zeros((out_features, zw * pack), dtype=torch.float16, device=dev))
        else:
            self.register_buffer("qweight", torch.zeros((in_features, out_features // pack), dtype=torch.int32, device=dev))
            self.register_buffer("qzeros", torch.zeros((in_features // self.group_size, out_features // pack),
                                                       dtype=torch.int32, device=dev))
            self.register_buffer("scales", torch.zeros((in_features // self.group_size, out_features),
                                                       dtype=torch.float16, device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16, device=dev))
        else:
            self.bias = None

    @classmethod
    def from_linear(cls, linear, bits, group_size, backend=AwqBackendPackingMethod.AUTOAWQ, init_only=False,
                    scales=None, zeros=None):
        """Build from an fp linear.  With ``scales``/``zeros`` ([in/group, out]) the weights are really packed
        (round((w + zero*scale)/scale)); ``init_only`` just allocates the buffers for ``load_state_dict``."""
        obj = cls(bits, group_size, linear.in_features, linear.out_features, linear.bias is not None,
                  linear.weight.device, backend)
        if init_only:
            return obj
        if scales is None or zeros is None:
            raise ValueError("Scales and zeros should not be None.")
        if backend != AwqBackendPackingMethod.AUTOAWQ:
            raise NotImplementedError("from_linear packs the AutoAWQ layout only")
        g = obj.group_size
        w = linear.weight.data.float().t()                      # [in, out]
        s = scales.float().repeat_interleave(g, dim=0)          # [in, out]
        z = zeros.float().repeat_interleave(g, dim=0)
        codes = torch.clamp(torch.round(w / s + z), 0, 15).to(torch.int32)
        obj.scales = scales.clone().half()
        if linear.bias is not None:
            obj.bias = linear.bias.clone().half()
        pack = 8
        qweight = torch.zeros((codes.shape[0], codes.shape[1] // pack), dtype=torch.int32, device=codes.device)
        qzeros = torch.zeros((zeros.shape[0], zeros.shape[1] // pack), dtype=torch.int32, device=codes.device)
        zi = zeros.to(torch.int32)
        for j, pos in enumerate(AWQ_ORDER):
            # column j of every group of 8 lives at nibble position AWQ_ORDER[j]
            qweight |= codes[:, j::pack] << (4 * pos)
            qzeros |= zi[:, j::pack] << (4 * pos)
        obj.qweight = qweight
        obj.qzeros = qzeros
        return obj

    def forward(self, x):
        raise RuntimeError("WQLinear_GEMM is a checkpoint container; convert the model with optimize_model / "
                           "from_pretrained(load_in_4bit=True) before running it")


def _unpack_int32(packed: torch.Tensor, order, bits=4):
    """[R, C] int32 -> [R, C*8] codes, column j of each group of 8 taken from nibble position ``order[j]``."""
    shifts = _shifts(order, bits, packed.device)
    out = (packed.unsqueeze(-1) >> shifts.view(1, 1, -1)) & ((1 << bits) - 1)
    return out.reshape(packed.shape[0], -1)


def unpack_awq(qweight, qzeros, bits=4, llm_awq=False):
    """Returns ``(weight [out, in] uint8 codes, zeros [in/group, out] int)``."""
    if llm_awq:
        weight = _unpack_int32(qweight, LLM_AWQ_ORDER, bits)            # [out, in]
        zeros = _unpack_int32(qzeros, LLM_AWQ_ORDER, bits).t()          # -> [groups(padded), out]
        groups = weight.shape[1] // (weight.shape[1] // max(1, zeros.shape[0])) if zeros.shape[0] else 0
        return weight.to(torch.uint8), zeros[:groups] if groups else zeros
    w = _unpack_int32(qweight, AWQ_ORDER, bits)                          # [in, out]
    z = _unpack_int32(qzeros, AWQ_ORDER, bits)                           # [in/group, out]
    return w.t().contiguous().to(torch.uint8), z


def unpack_gptq(qweight, qzeros, bits=4):
    """GPTQ (AutoGPTQ v1): qweight [in/8, out] packs 8 input rows per int32; stored zero points are ``z - 1``.
    Returns ``(weight [out, in] uint8 codes, zeros [in/group, out] int)``."""
    pack = 32 // bits
    shifts = torch.arange(pack, dtype=torch.int32, device=qweight.device) * bits
    w = (qweight.unsqueeze(1) >> shifts.view(1, -1, 1)) & ((1 << bits) - 1)   # [in/8, 8, out]
    w = w.reshape(-1, qweight.shape[1])                                       # [in, out]
    z = (qzeros.unsqueeze(-1) >> shifts.view(1, 1, -1)) & ((1 << bits) - 1)   # [groups, out/8, 8]
    z = z.reshape(qzeros.shape[0], -1) + 1
    return w.t().contiguous().to(torch.uint8), z
