"""Embedding variants: host-resident, disk-resident and low-bit tables.

Counterparts of ``CPUEmbedding``, ``DiskEmbedding`` and ``LowBitEmbedding`` of the reference
(python/llm/src/ipex_llm/transformers/embedding.py:29-241).
"""
from __future__ import annotations


import numpy as np
import torch
from torch import Tensor, nn

from ..quant import qtypes as qt
from ..quant.params import FP4Params, get_block_size, get_type_size


def _scaled(module, out: Tensor) -> Tensor:
    """Scaled word embeddings (Gemma family: rows times sqrt(hidden)) keep their factor when the table is replaced;
    the converter stores it as ``embed_scale_value``."""
    scale = getattr(module, "embed_scale_value", None)
    return out if scale is None or scale == 1.0 else out * torch.tensor(scale, dtype=out.dtype, device=out.device)


class CPUEmbedding(nn.Embedding):
    """Table pinned to host memory whatever ``.to(device)`` says; lookups return on the ids' device."""

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, max_norm=None, norm_type=2.0,
                 scale_grad_by_freq=False, sparse=True, _weight=None, _freeze=False, device=None, dtype=None):
        super().__init__(num_embeddings, embedding_dim, padding_idx, max_norm, norm_type, scale_grad_by_freq,
                         sparse, _weight, True, device, dtype)
        self.weight.requires_grad_(False)

    def _apply(self, fn, recurse=True):
        # never leave the host
        return self

    def forward(self, x: Tensor):
        return _scaled(self, super().forward(x.to("cpu")).to(x.device))

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding):
        return cls(embedding.num_embeddings, embedding.embedding_dim, embedding.padding_idx, embedding.max_norm,
                   embedding.norm_type, embedding.scale_grad_by_freq, True, embedding.weight.data, True,
                   embedding.weight.device, embedding.weight.dtype)


class DiskEmbedding(nn.Embedding):
    """Rows are read on demand from an fp16 file (``embeddings.bin``): only the looked-up rows touch memory."""

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, max_norm=None, norm_type=2.0,
                 scale_grad_by_freq=False, sparse=False, _weight=None, _freeze=False, device=None, dtype=None):
        super().__init__(num_embeddings, embedding_dim, padding_idx, max_norm, norm_type, scale_grad_by_freq,
                         sparse, _weight, True, device, dtype)
        self.filename = "embeddings.bin"
        self.weight.data.flatten().to(torch.float16).numpy().tofile(self.filename)
        self.weight = nn.Parameter(torch.empty(0, dtype=torch.float16), requires_grad=False)

    def forward(self, input_ids: Tensor):
        ids = input_ids.cpu().flatten()
        out = torch.empty(ids.numel(), self.embedding_dim, dtype=torch.float16)
        row_bytes = self.embedding_dim * 2
        with open(self.filename, "rb") as f:
            for i, idx in enumerate(ids.tolist()):
                f.seek(idx * row_bytes)
                out[i] = torch.from_numpy(np.frombuffer(f.read(row_bytes), dtype=np.float16).copy())
        return out.view(*input_ids.shape, self.embedding_dim).to(input_ids.device)

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding):
        return cls(embedding.num_embeddings, embedding.embedding_dim, embedding.padding_idx, embedding.max_norm,
                   embedding.norm_type, embedding.scale_grad_by_freq, embedding.sparse, embedding.weight.data, True,
                   embedding.weight.device, embedding.weight.dtype)

    def to_embedding(self):
        with open(self.filename, "rb") as f:
            w = torch.from_numpy(np.frombuffer(f.read(), dtype=np.float16).copy()).view(
                self.num_embeddings, self.embedding_dim)
        return nn.Embedding(self.num_embeddings, self.embedding_dim, self.padding_idx, self.max_norm, self.norm_type,
                            self.scale_grad_by_freq, self.sparse, w, True)

    @staticmethod
    def replace_normal_embedding(m: nn.Module):
        for name, module in m.named_children():
            if type(module) is nn.Embedding:
                setattr(m, name, DiskEmbedding.from_embedding(module))

    @staticmethod
    def restore_normal_embedding(m: nn.Module):
        for name, module in m.named_children():
            if isinstance(module, DiskEmbedding):
                setattr(m, name, module.to_embedding())


class LowBitEmbedding(nn.Embedding):
    """Embedding whose table is packed blocks; looked-up rows are dequantized on the device
    (the reference's ``xe_linear.dequantize_rows``)."""

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, max_norm=None, norm_type=2.0,
                 scale_grad_by_freq=False, sparse=False, _weight=None, _freeze=False, device=None, dtype=None,
                 convert_shape_only=None, qtype=None):
        super().__init__(num_embeddings, embedding_dim, padding_idx, max_norm, norm_type, scale_grad_by_freq,
                         sparse, _weight, True, device, dtype)
        self.qtype = qtype
        self.torch_dtype = dtype or torch.float32
        self.weight = FP4Params(self.weight.data, requires_grad=False, quantized=False, _shape=None,
                                convert_shape_only=bool(convert_shape_only), qtype=qtype, in_features=embedding_dim)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        """A packed table from a low-bit checkpoint is installed as ``FP4Params`` (``assign=True`` would otherwise
        leave a plain parameter behind, without qtype and shape)."""
        key = prefix + "weight"
        if key in state_dict and isinstance(self.weight, FP4Params) and state_dict[key].dtype == torch.uint8:
            data = state_dict[key]
            w = self.weight
            want = self.num_embeddings * self.embedding_dim // get_block_size(w.qtype) * get_type_size(w.qtype)
            if data.numel() != want:
                error_msgs.append(f"size mismatch for {key}: a packed [{self.num_embeddings}, {self.embedding_dim}] "
                                  f"table needs {want} bytes, the checkpoint holds {data.numel()}")
                return
            new = FP4Params(data.detach(), requires_grad=False, quantized=True,
                            _shape=torch.Size((self.num_embeddings, self.embedding_dim)), qtype=w.qtype,
                            in_features=self.embedding_dim)
            new.keep_canonical = True                          # tables are read row-wise on every device
            self._parameters["weight"] = new
            return
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)

    def _row_view(self):
        w = self.weight
        row_bytes = self.embedding_dim // get_block_size(w.qtype) * get_type_size(w.qtype)
        raw = w.data.view(torch.uint8) if w.data.dtype != torch.uint8 else w.data
        return raw.view(self.num_embeddings, row_bytes), row_bytes

    def forward(self, x: Tensor):
        w = self.weight
        if not w.quantized:
            w = w.quantize("cpu")
            self._parameters["weight"] = w
        if w.data.is_cuda:
            from . import cuda_ops
            return _scaled(self, cuda_ops.dequantize_rows(x, w, self.embedding_dim, self.num_embeddings,
                                                          self.torch_dtype))
        rows, _ = self._row_view()
        ids = x.reshape(-1).cpu()
        picked = rows.index_select(0, ids).contiguous()
        from ..quant.params import ggml_convert_fp32
        out = ggml_convert_fp32(picked, (ids.numel(), self.embedding_dim), ids.numel() * self.embedding_dim, w.qtype)
        return _scaled(self, out.view(*x.shape, self.embedding_dim).to(self.torch_dtype).to(x.device))

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding, qtype, convert_shape_only=False, device="cpu"):
        obj = cls(embedding.num_embeddings, embedding.embedding_dim, embedding.padding_idx, embedding.max_norm,
                  embedding.norm_type, embedding.scale_grad_by_freq, embedding.sparse,
                  embedding.weight.data.float(), True, embedding.weight.device, embedding.weight.dtype,
                  convert_shape_only, qtype)
        # embedding tables are read row-wise: they always keep the canonical (row-contiguous) byte order
        obj._parameters["weight"] = obj.weight.quantize("meta" if str(device) == "meta" else "cpu")
        obj.weight.keep_canonical = True
        return obj

    def _apply(self, fn, recurse=True):
        # move the canonical bytes as a plain tensor: rows stay contiguous on the device
        w = self.weight
        probe = fn(torch.empty(0))
        if w.quantized and probe.device != w.data.device and w.data.device.type != "meta":
            moved = FP4Params(w.data.to(probe.device), requires_grad=False, quantized=True, _shape=w._shape,
                              qtype=w.qtype)
            moved.keep_canonical = True
            self._parameters["weight"] = moved
        return self
