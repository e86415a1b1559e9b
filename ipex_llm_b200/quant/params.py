"""Packed low-bit weights: quantize / dequantize wrappers and the ``FP4Params`` parameter class.

Covers the reference's ``ggml_convert_qtype``, ``ggml_q_format_convet_cpu2xpu/xpu2cpu``,
``ggml_convert_fp32`` and ``FP4Params`` (python/llm/src/ipex_llm/transformers/low_bit_linear.py:104-259,
312-459).

Two layouts exist for every packed tensor:

* **canonical** — interleaved blocks ``[scale | (min) | codes]`` exactly as serialized by ``save_low_bit``;
  this is what lives on the CPU (``nf4`` is viewed as bfloat16, as in the reference, so that every
  parameter of a QLoRA model has one dtype).
* **device** — what the sm_100a kernels read: tensor-core tile order for the 4-bit and 8-bit families
  (see ``native/host/quant_core.cpp``), canonical bytes for the rest.

``FP4Params.to("cuda")`` quantizes if needed (on the GPU when the source weight is already there) and
converts canonical -> device; ``.to("cpu")`` converts back, so a state dict saved from either place is
byte-identical.
"""
from __future__ import annotations

import ctypes

import torch

from ..native import lib as _nl
from . import iq_codebooks as iq
from . import qtypes as qt

RTN_DTYPE = {qt.SYM_INT4_RTN: torch.uint8, qt.ASYM_INT4_RTN: torch.uint8, qt.SYM_INT8_RTN: torch.int8}


def get_block_size(qtype) -> int:
    if isinstance(qtype, str):
        qtype = qt.qtype_from_name(qtype)
    if qtype == qt.MOFQ4:
        return 64          # picks sym_int4 or fp4 per layer: both 64 values per block
    if qtype == qt.MOFQ8:
        return 128         # picks sym_int8 (64) or fp8_e4m3 (128): a layer must suit both
    return _nl.host_lib().ggml_qk_size(qtype)


get_qk_size = get_block_size


def get_type_size(qtype: int) -> int:
    return _nl.host_lib().ggml_type_size(qtype)


def packed_nbytes(numel: int, qtype: int) -> int:
    return numel // get_block_size(qtype) * get_type_size(qtype)


def device_nbytes(rows: int, cols: int, qtype: int) -> int:
    return int(_nl.host_lib().ipex_device_bytes(rows, cols, qtype))


def _check_supported(qtype: int):
    if iq.is_iq(qtype):
        iq.grid(qtype, "cpu")          # raises NotImplementedError when the grids cannot be had
        return
    if not _nl.host_lib().ipex_qtype_supported(qtype) and qtype not in RTN_DTYPE:
        raise NotImplementedError(f"qtype id {qtype} has no block codec")


def ggml_convert_qtype(tensor: torch.Tensor, qtype: int, device=None, convert_shape_only=False,
                       imatrix: torch.Tensor = None, in_features: int = None,
                       enable_scale_search: bool = False):
    """fp32 tensor ``[..., K]`` -> canonical packed tensor (CPU).  RTN qtypes return ``(codes, scale)``."""
    _check_supported(qtype)
    lib = _nl.host_lib()
    QK = lib.ggml_qk_size(qtype)
    ts = lib.ggml_type_size(qtype)
    if tensor.dtype != torch.float32:
        raise TypeError("Input tensor must be float32")
    n = tensor.numel()
    k = tensor.shape[-1]
    if qtype in RTN_DTYPE:
        rows = n // k
        bits4 = qtype != qt.SYM_INT8_RTN
        dst = torch.empty((rows, k // 2 if bits4 else k), dtype=RTN_DTYPE[qtype], device=device)
        scale = torch.empty(rows * (2 if qtype == qt.ASYM_INT4_RTN else 1), dtype=torch.float32, device=device)
        if not convert_shape_only and device != "meta":
            src = tensor.contiguous()
            lib.ggml_quantize_tensor_rtn(src.data_ptr(), dst.data_ptr(), scale.data_ptr(), qtype, n, k, None,
                                         int(enable_scale_search))
        return dst, scale.to(torch.float16)
    if k % QK != 0:
        raise ValueError(f"Last dim of input tensor must be multiple of {QK}")
    dst_size = (n // QK) * ts
    if iq.is_iq(qtype):
        if convert_shape_only or device == "meta":
            return torch.empty(dst_size, dtype=torch.uint8, device=device)
        src = tensor.view(-1, in_features) if in_features and in_features != k else tensor
        return iq.quantize(src, qtype, imatrix)
    if qtype == qt.NF4:
        dst = torch.empty(dst_size // 2, dtype=torch.bfloat16, device=device)
    else:
        dst = torch.empty(dst_size, dtype=torch.uint8, device=device)
    if not convert_shape_only and device != "meta":
        src = tensor.contiguous()
        if imatrix is not None:
            im = imatrix.to(torch.float32).contiguous()
            nrow = n // (in_features or k)
            lib.ggml_quantize_tensor_with_weights(src.data_ptr(), dst.data_ptr(), qtype, nrow, in_features or k,
                                                  None, im.data_ptr())
        else:
            hist = (ctypes.c_int64 * 16)()
            lib.ggml_quantize_tensor(src.data_ptr(), dst.data_ptr(), qtype, n, k, None, int(enable_scale_search))
            del hist
    return dst


def ggml_convert_fp32(tensor: torch.Tensor, weight_shape, k: int, qtype: int) -> torch.Tensor:
    """canonical packed CPU tensor -> fp32 tensor of ``weight_shape``."""
    lib = _nl.host_lib()
    if iq.is_iq(qtype):
        return iq.dequantize(tensor, tuple(weight_shape), qtype, torch.float32)
    src = tensor.contiguous()
    dst = torch.empty(tuple(weight_shape), dtype=torch.float32)
    lib.ggml_dequantize(src.data_ptr(), dst.data_ptr(), k, qtype)
    return dst


def ggml_q_format_convet_cpu2xpu(tensor: torch.Tensor, shape, qtype: int, device=None) -> torch.Tensor:
    """canonical CPU bytes -> device-layout bytes, placed on ``device``."""
    lib = _nl.host_lib()
    rows = int(torch.Size(shape[:-1]).numel()) if len(shape) > 1 else 1
    cols = int(shape[-1])
    src = tensor.contiguous().view(torch.uint8) if tensor.dtype != torch.uint8 else tensor.contiguous()
    dst = torch.empty(device_nbytes(rows, cols, qtype), dtype=torch.uint8)
    rc = lib.ggml_q_format_convet_cpu2xpu(src.data_ptr(), dst.data_ptr(), rows, cols, qtype)
    if rc != 0:
        raise RuntimeError("canonical -> device layout conversion failed")
    return dst.to(device) if device is not None else dst


def ggml_q_format_convet_xpu2cpu(tensor: torch.Tensor, shape, qtype: int) -> torch.Tensor:
    """device-layout bytes (any device) -> canonical CPU tensor (bf16 view for nf4)."""
    lib = _nl.host_lib()
    rows = int(torch.Size(shape[:-1]).numel()) if len(shape) > 1 else 1
    cols = int(shape[-1])
    src = tensor.detach().to("cpu").contiguous().view(torch.uint8)
    dst = torch.empty(packed_nbytes(rows * cols, qtype), dtype=torch.uint8)
    rc = lib.ggml_q_format_convet_xpu2cpu(src.data_ptr(), dst.data_ptr(), rows, cols, qtype)
    if rc != 0:
        raise RuntimeError("device -> canonical layout conversion failed")
    return dst.view(torch.bfloat16) if qtype == qt.NF4 else dst


def ggml_int4_convert_fp32(tensor, weight_shape, k):
    return ggml_convert_fp32(tensor, weight_shape, k, qt.SYM_INT4)


def ggml_matmul_src1_x_src0_t(src0: torch.Tensor, src1: torch.Tensor, src0_shape, src0_qtype: int) -> torch.Tensor:
    """CPU oracle: ``src1[M,K] @ dequant(src0[N,K]).T`` in fp32 (reference low_bit_linear.py:462-497)."""
    lib = _nl.host_lib()
    if src1.dtype != torch.float32:
        src1 = src1.float()
    src1 = src1.contiguous()
    N, K = int(src0_shape[0]), int(src0_shape[1])
    lead = src1.shape[:-1]
    M = int(src1.numel() // K)
    out = torch.empty((M, N), dtype=torch.float32)
    ne0 = (ctypes.c_int64 * 4)(K, N, 1, 1)
    ne1 = (ctypes.c_int64 * 4)(K, M, 1, 1)
    w = src0.contiguous()
    need = N * K // get_block_size(src0_qtype) * get_type_size(src0_qtype)
    have = w.numel() * w.element_size()
    if have < need or w.device.type != "cpu":
        raise RuntimeError(f"packed weight holds {have} bytes on {w.device}, a [{N}, {K}] "
                           f"{qt.qtype_name(src0_qtype)} matrix needs {need} on cpu: the checkpoint does not match "
                           "the module layout (was it saved with another `optimize_model` setting?)")
    if iq.is_iq(src0_qtype):
        torch.matmul(src1.view(M, K), iq.dequantize(w, (N, K), src0_qtype).t(), out=out)
        return out.view(*lead, N)
    lib.ggml_compute_forward_mul_mat_q_fp32(ne0, w.data_ptr(), src0_qtype, ne1, src1.data_ptr(), out.data_ptr())
    return out.view(*lead, N)


def quantize_mse(w: torch.Tensor, qtype: int) -> float:
    w = w.float().contiguous()
    return float(_nl.host_lib().ipex_quantize_mse(w.data_ptr(), qtype, w.numel(), w.shape[-1]))


class FP4Params(torch.nn.Parameter):
    """Parameter holding a packed low-bit weight (any qtype, the name is historical).

    State: ``quantized`` (is ``data`` packed?), ``_shape`` (logical weight shape), ``qtype``,
    ``layout`` ("canonical" | "device"), plus the quantization options.
    """

    def __new__(cls, data=None, requires_grad=False, quantized=False, _shape=None, convert_shape_only=False,
                qtype=None, imatrix=None, in_features=None, enable_scale_search=False, layout="canonical"):
        if data is None:
            data = torch.empty(0)
        self = torch.Tensor._make_subclass(cls, data, requires_grad)
        self.data = data
        self.quantized = quantized
        self._shape = _shape
        self.qtype = qtype
        self.convert_shape_only = convert_shape_only
        self.imatrix = imatrix
        self.in_features = in_features
        self.enable_scale_search = enable_scale_search
        return self

    @property
    def layout(self) -> str:
        """"device" when the packed bytes are in the GPU tile layout, else "canonical".  Derived from where
        the bytes live so that ``nn.Module._apply`` (which swaps ``.data`` in place) cannot desynchronise it."""
        if getattr(self, "keep_canonical", False):
            return "canonical"   # row-addressed tables (quantized embeddings) stay in block order on the GPU
        return "device" if (self.quantized and self.data.is_cuda) else "canonical"

    @layout.setter
    def layout(self, value):  # kept for call sites that state the layout explicitly
        pass

    def half(self, *a, **k):
        return self if self.quantized else super().half(*a, **k)

    def float(self, *a, **k):
        return self if self.quantized else super().float(*a, **k)

    def bfloat16(self, *a, **k):
        return self if self.quantized else super().bfloat16(*a, **k)

    # -- helpers --------------------------------------------------------------------------------
    def _like(self, data, **over):
        kw = dict(requires_grad=self.requires_grad, quantized=self.quantized, _shape=self._shape, qtype=self.qtype,
                  imatrix=self.imatrix, in_features=self.in_features, enable_scale_search=self.enable_scale_search,
                  convert_shape_only=self.convert_shape_only)
        kw.update(over)
        new = FP4Params(data, **kw)
        if getattr(self, "keep_canonical", False):
            new.keep_canonical = True
        return new

    def ggml_mse(self, w, ggml_qtype, device):
        if device == "meta":
            return 0.0
        return quantize_mse(w, ggml_qtype)

    def quantize(self, device=None):
        """Pack ``data`` (a float weight) into canonical blocks on the CPU (or shapes only on meta)."""
        if self.quantized:
            return self
        w = self.data.contiguous().float()
        qtype = self.qtype
        if qtype == qt.MOFQ4:
            qtype = qt.SYM_INT4 if self.ggml_mse(w, qt.SYM_INT4, device) <= self.ggml_mse(w, qt.FP4, device) \
                else qt.FP4
        elif qtype == qt.MOFQ8:
            qtype = qt.SYM_INT8 if self.ggml_mse(w, qt.SYM_INT8, device) <= self.ggml_mse(w, qt.FP8E4, device) \
                else qt.FP8E4
        self.qtype = qtype
        self._shape = w.shape
        meta = device is not None and str(device) == "meta"
        if not meta and w.is_cuda and iq.is_iq(qtype):
            # the code-book search is tensor code: it runs where the weight is, and block order is also what the
            # device keeps for these formats
            src = w.view(-1, self.in_features) if self.in_features and self.in_features != w.shape[-1] else w
            self.data = iq.quantize(src, qtype, self.imatrix)
            self.quantized = True
            return self
        if not meta and w.is_cuda:
            from ..ops import cuda_quant
            if cuda_quant.can_quantize_on_gpu(qtype) and self.imatrix is None:
                packed = cuda_quant.quantize_to_device_layout(w, qtype)
                self.data = packed
                self.quantized = True
                self.layout = "device"
                return self
            w = w.cpu()
        packed = ggml_convert_qtype(w, qtype, device="meta" if meta else None,
                                    convert_shape_only=self.convert_shape_only or meta,
                                    imatrix=self.imatrix, in_features=self.in_features,
                                    enable_scale_search=self.enable_scale_search)
        self.data = packed
        self.quantized = True
        self.layout = "canonical"
        return self

    def get_shape(self):
        return self._shape

    # -- device moves -----------------------------------------------------------------------------
    def to(self, *args, **kwargs):
        device, dtype, non_blocking, _ = torch._C._nn._parse_to(*args, **kwargs)
        if device is None:
            return self
        dev_type = device.type
        if dev_type == "meta":
            if not self.quantized:
                return self.quantize("meta")
            return self._like(self.data.to("meta"))
        if dev_type == "cpu":
            if not self.quantized:
                if self.data.is_cuda:
                    self.data = self.data.cpu()
                return self.quantize("cpu")
            if self.layout == "device":
                data = ggml_q_format_convet_xpu2cpu(self.data, self._shape, self.qtype)
                return self._like(data, layout="canonical")
            return self._like(self.data.to("cpu"))
        if dev_type == "cuda":
            if not self.quantized:
                if not self.data.is_cuda:
                    from ..ops import cuda_quant
                    if iq.is_iq(self.qtype) or (cuda_quant.can_quantize_on_gpu(self.qtype) and self.imatrix is None
                                                and self.qtype not in (qt.MOFQ4, qt.MOFQ8)):
                        self.data = self.data.to(device, non_blocking=non_blocking)
                self.quantize(device)
            if self.layout == "canonical":
                if self.data.device.type == "meta":
                    raise RuntimeError("cannot move a meta FP4Params to cuda; load weights first")
                data = ggml_q_format_convet_cpu2xpu(self.data.cpu(), self._shape, self.qtype, device)
                return self._like(data, layout="device")
            return self._like(self.data.to(device, non_blocking=non_blocking))
        # other accelerators: keep canonical bytes
        return self._like(self.data.to(device))

    def cuda(self, device=None):
        return self.to(torch.device("cuda", device) if isinstance(device, int) else (device or "cuda"))

    def cpu(self):
        return self.to("cpu")

    # -- views ------------------------------------------------------------------------------------
    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        """Full logical weight, on the parameter's device."""
        assert self.quantized
        if self.data.is_cuda:
            from ..ops import cuda_quant
            return cuda_quant.dequantize_device(self.data, tuple(self._shape), self.qtype, dtype)
        raw = self.data
        w = ggml_convert_fp32(raw.view(torch.uint8) if raw.dtype != torch.uint8 else raw,
                              self._shape, int(torch.Size(self._shape).numel()), self.qtype)
        return w.to(dtype)

    def __deepcopy__(self, memo):
        new = self._like(self.data.clone())
        memo[id(self)] = new
        return new

    def __reduce_ex__(self, proto):
        # serialize as the raw packed tensor (what save_low_bit writes)
        return (torch._utils._rebuild_tensor_v2,
                (self.data.untyped_storage(), self.data.storage_offset(), tuple(self.data.size()),
                 self.data.stride(), False, {}))
