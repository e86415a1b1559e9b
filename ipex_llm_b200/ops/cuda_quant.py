"""GPU-side quantization straight into the device tile layout.

The reference quantizes on the host (OpenMP, ``ggml_quantize_tensor``) and re-lays the bytes out when the
parameter moves to the accelerator (python/llm/src/ipex_llm/transformers/low_bit_linear.py:348-459).  On a
B200 the weights are quantized where they will live: one kernel reads the half/float matrix and writes codes and
scales in tile order, bit-identical to the host quantizer for the integer formats.
"""
from __future__ import annotations

import torch

from ..native import cuda_api as api
from ..native.lib import cuda_lib, current_stream, ptr
from ..quant import qtypes as qt
from ..quant.params import device_nbytes

_GPU_QTYPES = {
    qt.SYM_INT4: (api.WF_SYM_INT4, 0), qt.ASYM_INT4: (api.WF_ASYM_INT4, 0), qt.NF4: (api.WF_LUT4, 0),
    qt.FP4: (api.WF_LUT4, 1), qt.FP8E4: (api.WF_FP8_E4M3, 0), qt.FP8E5: (api.WF_FP8_E5M2, 0),
    qt.SYM_INT8: (api.WF_INT8, 0),
}


def can_quantize_on_gpu(qtype: int) -> bool:
    return qtype in _GPU_QTYPES and torch.cuda.is_available()


def quantize_to_device_layout(w: torch.Tensor, qtype: int, out: torch.Tensor = None) -> torch.Tensor:
    """``w [N, K]`` (cuda, fp16/bf16/fp32) -> uint8 tensor in the device layout of ``qtype``."""
    assert w.is_cuda and w.dim() >= 2
    lib = cuda_lib()
    w2 = w.reshape(-1, w.shape[-1])
    if w2.stride(-1) != 1:
        w2 = w2.contiguous()
    rows, cols = w2.shape
    block = 128 if qtype in (qt.FP8E4, qt.FP8E5) else 64
    if cols % block != 0:
        raise ValueError(f"in_features {cols} is not a multiple of the {block}-wide block")
    nbytes = device_nbytes(rows, cols, qtype)
    if out is None:
        out = torch.zeros(nbytes, dtype=torch.uint8, device=w.device)
    else:
        out.zero_()
    wf, lut_kind = _GPU_QTYPES[qtype]
    rc = lib.ipex_quantize_to_tiles(ptr(w2), ptr(out), rows, cols, w2.stride(0), wf, lut_kind,
                                    api.dtype_code(w2.dtype), current_stream())
    api.check(rc, "quantize_to_tiles")
    return out


def dequantize_device(data: torch.Tensor, shape, qtype: int, dtype=torch.float16) -> torch.Tensor:
    from .cuda_ops import dequantize_device as _dq
    return _dq(data, shape, qtype, dtype)
