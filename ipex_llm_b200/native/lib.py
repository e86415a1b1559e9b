"""ctypes loaders for the two in-tree native libraries.

``host_lib()`` is the stand-in for the reference's ``libllama-api.so`` binding
(python/llm/src/ipex_llm/ggml/model/llama/llama_cpp.py:946-1185): same C entry-point names
(``ggml_quantize_tensor``, ``ggml_dequantize``, ``ggml_qk_size``, ``ggml_type_size``,
``ggml_q_format_convet_cpu2xpu``, ``ggml_compute_forward_mul_mat_q_fp32``).

``cuda_lib()`` exposes the sm_100a kernels.  On a machine with a GPU a missing CUDA library is a hard
error: the GPU path never silently falls back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

_lock = threading.Lock()
_host = None
_cuda = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_int64 = ctypes.c_int64
c_float = ctypes.c_float
c_size_t = ctypes.c_size_t


def host_lib() -> ctypes.CDLL:
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                path = _build.HOST_LIB
                if not os.path.exists(path) or os.environ.get("IPEX_LLM_REBUILD_NATIVE") == "1":
                    path = _build.build_host()
                lib = ctypes.CDLL(path)
                lib.ggml_qk_size.argtypes = [c_int]
                lib.ggml_qk_size.restype = c_int
                lib.ggml_type_size.argtypes = [c_int]
                lib.ggml_type_size.restype = c_int
                lib.ipex_qtype_supported.argtypes = [c_int]
                lib.ipex_qtype_supported.restype = c_int
                lib.ggml_quantize_tensor.argtypes = [c_void_p, c_void_p, c_int, c_size_t, c_int, c_void_p, c_int]
                lib.ggml_quantize_tensor.restype = c_size_t
                lib.ggml_quantize_tensor_with_weights.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int,
                                                                  c_void_p, c_void_p]
                lib.ggml_quantize_tensor_with_weights.restype = c_size_t
                lib.ggml_quantize_tensor_rtn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int,
                                                         c_void_p, c_int]
                lib.ggml_quantize_tensor_rtn.restype = c_size_t
                lib.ggml_dequantize.argtypes = [c_void_p, c_void_p, c_size_t, c_int]
                lib.ggml_dequantize.restype = None
                lib.ipex_device_bytes.argtypes = [c_int64, c_int64, c_int]
                lib.ipex_device_bytes.restype = c_size_t
                lib.ggml_q_format_convet_cpu2xpu.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int]
                lib.ggml_q_format_convet_cpu2xpu.restype = c_int
                lib.ggml_q_format_convet_xpu2cpu.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int]
                lib.ggml_q_format_convet_xpu2cpu.restype = c_int
                lib.ggml_compute_forward_mul_mat_q_fp32.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                                    c_void_p]
                lib.ggml_compute_forward_mul_mat_q_fp32.restype = None
                lib.ipex_quantize_mse.argtypes = [c_void_p, c_int, c_size_t, c_int]
                lib.ipex_quantize_mse.restype = ctypes.c_double
                _host = lib
    return _host


def cuda_available() -> bool:
    import torch
    return torch.cuda.is_available()


def cuda_lib() -> ctypes.CDLL:
    """Load the CUDA kernel library (builds it when absent and nvcc is present)."""
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                path = os.environ.get("IPEX_LLM_CUDA_LIB") or _build.CUDA_LIB
                if not os.path.exists(path):
                    try:
                        path = _build.build_cuda()
                    except Exception as e:  # noqa: BLE001
                        raise RuntimeError(
                            "ipex_llm_b200: the sm_100a kernel library is missing and could not be built "
                            f"({e}). Run `python -m ipex_llm_b200.native.build`.") from e
                lib = ctypes.CDLL(path)
                from . import cuda_api
                cuda_api.declare(lib)
                _cuda = lib
    return _cuda


def ptr(t) -> ctypes.c_void_p:
    """Device/host pointer of a tensor (None -> NULL)."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def current_stream() -> ctypes.c_void_p:
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
