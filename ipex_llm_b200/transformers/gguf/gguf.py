"""GGUF container reader (and a small writer used by tools and tests).

Counterpart of python/llm/src/ipex_llm/transformers/gguf/gguf.py:1-424 (``GGUFFileLoader`` with ``config``,
``tensor_loader``, ``tokenizer_pieces``).  The file is memory-mapped; tensors are decoded to float one at a time, so
peak host memory is one tensor.  Block decoders for the classic ggml formats (q4_0, q4_1, q5_0, q5_1, q8_0, 32 values
per block as in llama.cpp files) are written here with numpy; the k-quant super-blocks go through the package's host
library, whose q2_k..q6_k block layouts are the ggml ones, and the code-book super-blocks (iq2_xxs, iq2_xs, iq1_s,
iq1_m) through ``quant/iq_codebooks.py``.
"""
from __future__ import annotations

import mmap
import struct
from typing import Callable, Dict, List, Tuple

import numpy as np
import torch

from ...utils.common import invalidInputError

GGUF_MAGIC = 0x46554747  # "GGUF" little endian
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
T_STRING, T_ARRAY = 8, 9

# ggml tensor types: id -> (name, values per block, bytes per block)
GGML_TYPES = {
    0: ("f32", 1, 4), 1: ("f16", 1, 2), 2: ("q4_0", 32, 18), 3: ("q4_1", 32, 20), 6: ("q5_0", 32, 22),
    7: ("q5_1", 32, 24), 8: ("q8_0", 32, 34), 10: ("q2_k", 256, 84), 11: ("q3_k", 256, 110), 12: ("q4_k", 256, 144),
    13: ("q5_k", 256, 176), 14: ("q6_k", 256, 210), 30: ("bf16", 1, 2),
    16: ("iq2_xxs", 256, 66), 17: ("iq2_xs", 256, 74), 19: ("iq1_s", 256, 50), 29: ("iq1_m", 256, 56),
}
_NAME_TO_TYPE = {v[0]: k for k, v in GGML_TYPES.items()}


def _library_types():
    """Tensor types this module has no decoder of its own for (iq3_xxs, iq3_s, iq2_s, iq4_nl, iq4_xs, tq1_0, tq2_0,
    mxfp4, ...): geometry and decoder of the ``gguf`` package when it is installed."""
    try:
        import gguf
        return {int(t): (t.name.lower(), qk, bs) for t, (qk, bs) in gguf.GGML_QUANT_SIZES.items()
                if int(t) not in GGML_TYPES}
    except Exception:  # noqa: BLE001
        return {}


def type_geometry(ttype: int):
    """``(name, values per block, bytes per block)`` of a ggml tensor type, or None when nothing here can read it."""
    return GGML_TYPES.get(ttype) or _library_types().get(ttype)


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def unpack(self, fmt):
        size = struct.calcsize(fmt)
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += size
        return v

    def string(self):
        n = self.unpack("<Q")
        s = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return s.decode("utf-8", errors="replace")

    def value(self, vtype):
        if vtype in _SCALARS:
            return self.unpack(_SCALARS[vtype])
        if vtype == T_STRING:
            return self.string()
        if vtype == T_ARRAY:
            et = self.unpack("<I")
            n = self.unpack("<Q")
            if et in _SCALARS and et != 7:
                fmt = _SCALARS[et]
                size = struct.calcsize(fmt)
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt[1]).newbyteorder("<"), count=n, offset=self.pos)
                self.pos += size * n
                return arr.tolist()
            return [self.value(et) for _ in range(n)]
        invalidInputError(False, f"unknown GGUF value type {vtype}")


def _f16(buf: np.ndarray) -> np.ndarray:
    return buf.view(np.float16).astype(np.float32)


def dequantize_blocks(raw: np.ndarray, ttype: int, n_values: int) -> np.ndarray:
    """Raw bytes of a ggml tensor -> float32 vector of ``n_values``."""
    if ttype not in GGML_TYPES:
        import gguf
        from gguf import quants as gq
        name, qk, bs = _library_types()[ttype]
        return gq.dequantize(raw.reshape(n_values // qk, bs), gguf.GGMLQuantizationType(ttype)).reshape(-1)
    name, qk, bs = GGML_TYPES[ttype]
    if name == "f32":
        return raw.view(np.float32).copy()
    if name == "f16":
        return _f16(raw)
    if name == "bf16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    nb = n_values // qk
    blk = raw.reshape(nb, bs)
    if name == "q8_0":
        d = _f16(blk[:, :2].copy()).reshape(nb, 1)
        return (blk[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)
    if name in ("q4_0", "q4_1"):
        off = 2 if name == "q4_0" else 4
        d = _f16(blk[:, :2].copy()).reshape(nb, 1)
        qs = blk[:, off:]
        lo, hi = (qs & 0x0F).astype(np.float32), (qs >> 4).astype(np.float32)
        q = np.concatenate([lo, hi], axis=1)           # first 16 values are the low nibbles, then the high ones
        if name == "q4_0":
            return ((q - 8.0) * d).reshape(-1)
        m = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
        return (q * d + m).reshape(-1)
    if name in ("q5_0", "q5_1"):
        off = 2 if name == "q5_0" else 4
        d = _f16(blk[:, :2].copy()).reshape(nb, 1)
        qh = blk[:, off:off + 4].copy().view(np.uint32).reshape(nb, 1)
        qs = blk[:, off + 4:]
        j = np.arange(16, dtype=np.uint32).reshape(1, 16)
        h_lo = ((qh >> j) & 1).astype(np.uint8) << 4
        h_hi = ((qh >> (j + 16)) & 1).astype(np.uint8) << 4
        q = np.concatenate([(qs & 0x0F) | h_lo, (qs >> 4) | h_hi], axis=1).astype(np.float32)
        if name == "q5_0":
            return ((q - 16.0) * d).reshape(-1)
        m = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
        return (q * d + m).reshape(-1)
    if name == "q3_k":
        return _dequantize_q3_k(blk)
    # k-quants: the host library's decoders use the ggml super-block layouts; the code-book formats go through
    # quant/iq_codebooks.py, whose byte layout is the GGUF one
    from ...quant import qtypes as qt
    from ...quant.params import ggml_convert_fp32
    kq = {"q2_k": "q2_k", "q4_k": "q4_k", "q5_k": "q5_k", "q6_k": "q6_k", "iq2_xxs": "gguf_iq2_xxs",
          "iq2_xs": "gguf_iq2_xs", "iq1_s": "gguf_iq1_s", "iq1_m": "gguf_iq1_m"}.get(name)
    invalidInputError(kq is not None, f"GGUF tensor type {name} is not supported")
    t = torch.from_numpy(raw.copy())
    return ggml_convert_fp32(t, (1, n_values), n_values, qt.qtype_from_name(kq)).reshape(-1).numpy()


def _dequantize_q3_k(blk: np.ndarray) -> np.ndarray:
    """q3_k super-blocks (110 bytes: 32 B high bits, 64 B low 2-bit codes, 12 B packed 6-bit scales, fp16 d).  A value
    is ``d * (scale - 32) * (low2 - (0 if its high bit is set else 4))``; 16 scales, one per 16 values."""
    nb = blk.shape[0]
    hmask, qs, sc = blk[:, :32], blk[:, 32:96], blk[:, 96:108]
    d = _f16(blk[:, 108:110].copy()).reshape(nb, 1, 1)
    # 16 six-bit scales: low nibbles in bytes 0..7, the upper two bits of scale j in bytes 8..11
    low = np.concatenate([sc[:, :8] & 0x0F, sc[:, :8] >> 4], axis=1)                        # [nb, 16]
    hi = np.stack([(sc[:, 8:12] >> s) & 3 for s in (0, 2, 4, 6)], axis=1).reshape(nb, 16)   # [nb, 16]
    scales = (low | (hi << 4)).astype(np.int8).astype(np.float32) - 32.0
    # values: two halves of 128; inside a half four 2-bit planes of the same 32 bytes, each plane 32 values
    q = qs.reshape(nb, 2, 1, 32) >> np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 4, 1) & 3  # [nb, 2, 4, 32]
    bit = np.arange(8, dtype=np.uint8).reshape(1, 2, 4, 1)                                    # plane p of half n: bit 4n+p
    h = (hmask.reshape(nb, 1, 1, 32) >> bit) & 1
    vals = q.astype(np.float32) - np.where(h == 1, 0.0, 4.0).astype(np.float32)              # [nb, 2, 4, 32]
    vals = vals.reshape(nb, 16, 16) * scales.reshape(nb, 16, 1) * d
    return vals.reshape(-1)


class GGUFTensorLoader:
    def __init__(self, buf, infos: List[Tuple[str, List[int], int, int]], data_start: int):
        self.buf, self.infos, self.base = buf, infos, data_start

    def __len__(self):
        return len(self.infos)

    def names(self):
        return [i[0] for i in self.infos]

    def load(self, index_or_name) -> torch.Tensor:
        if isinstance(index_or_name, str):
            index_or_name = self.names().index(index_or_name)
        name, dims, ttype, off = self.infos[index_or_name]
        geom = type_geometry(ttype)
        invalidInputError(geom is not None, f"tensor {name}: unsupported ggml type {ttype}")
        n = int(np.prod(dims))
        _, qk, bs = geom
        nbytes = n // qk * bs
        raw = np.frombuffer(self.buf, dtype=np.uint8, count=nbytes, offset=self.base + off)
        vals = dequantize_blocks(raw, ttype, n)
        # GGUF stores dims fastest-first: ne[0] is the row length
        return torch.from_numpy(np.ascontiguousarray(vals)).reshape(list(reversed(dims)))

    def load_while_process(self, process: Callable[[str, torch.Tensor], None]):
        for i, info in enumerate(self.infos):
            process(info[0], self.load(i))


class GGUFFileLoader:
    def __init__(self, fpath: str):
        self._f = open(fpath, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        buf = memoryview(self._mm)
        c = _Cursor(buf)
        invalidInputError(c.unpack("<I") == GGUF_MAGIC, "Invalid GGUF file: bad magic")
        self.version = c.unpack("<I")
        invalidInputError(self.version in (2, 3), f"Unsupported GGUF version {self.version}")
        n_tensors, n_kv = c.unpack("<Q"), c.unpack("<Q")
        self.config: Dict[str, object] = {}
        for _ in range(n_kv):
            key = c.string()
            self.config[key] = c.value(c.unpack("<I"))
        infos = []
        for _ in range(n_tensors):
            name = c.string()
            nd = c.unpack("<I")
            dims = [c.unpack("<Q") for _ in range(nd)]
            ttype = c.unpack("<I")
            off = c.unpack("<Q")
            infos.append((name, dims, ttype, off))
        align = int(self.config.get("general.alignment", 32))
        data_start = (c.pos + align - 1) // align * align
        self.tensor_loader = GGUFTensorLoader(buf, infos, data_start)

    def tensors(self, dtype: torch.dtype = torch.float):
        return {n: self.tensor_loader.load(i).to(dtype) for i, n in enumerate(self.tensor_loader.names())}

    def tokenizer_pieces(self):
        """sentencepiece pieces (text, score, type) rebuilt from the vocabulary arrays."""
        from transformers.convert_slow_tokenizer import import_protobuf
        spm_pb2 = import_protobuf("Failed to import protobuf")
        tokens = self.config["tokenizer.ggml.tokens"]
        scores = self.config.get("tokenizer.ggml.scores", [0.0] * len(tokens))
        types = self.config.get("tokenizer.ggml.token_type", [1] * len(tokens))
        return [spm_pb2.ModelProto.SentencePiece(piece=t, score=float(s), type=int(ty))
                for t, s, ty in zip(tokens, scores, types)]

    def close(self):
        self.tensor_loader = None
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


# ----------------------------------------------------------------------------------------------------------------
# writer (f32 / f16 / q8_0 / q4_0): enough to export small models and to build files for tests
# ----------------------------------------------------------------------------------------------------------------
def _w_string(out: bytearray, s: str):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _w_value(out: bytearray, v):
    if isinstance(v, bool):
        out += struct.pack("<I", 7) + struct.pack("<?", v)
    elif isinstance(v, int):
        out += struct.pack("<I", 4 if 0 <= v < 2 ** 32 else 11) + struct.pack("<I" if 0 <= v < 2 ** 32 else "<q", v)
    elif isinstance(v, float):
        out += struct.pack("<I", 6) + struct.pack("<f", v)
    elif isinstance(v, str):
        out += struct.pack("<I", T_STRING)
        _w_string(out, v)
    elif isinstance(v, (list, tuple)):
        out += struct.pack("<I", T_ARRAY)
        if len(v) > 0 and isinstance(v[0], str):
            out += struct.pack("<I", T_STRING) + struct.pack("<Q", len(v))
            for s in v:
                _w_string(out, s)
        elif len(v) > 0 and isinstance(v[0], float):
            out += struct.pack("<I", 6) + struct.pack("<Q", len(v)) + np.asarray(v, dtype="<f4").tobytes()
        else:
            out += struct.pack("<I", 5) + struct.pack("<Q", len(v)) + np.asarray(v, dtype="<i4").tobytes()
    else:
        invalidInputError(False, f"cannot write GGUF value of type {type(v)}")


def quantize_blocks(x: np.ndarray, name: str) -> bytes:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if name == "f32":
        return x.tobytes()
    if name == "f16":
        return x.astype(np.float16).tobytes()
    if name in ("iq2_xxs", "iq2_xs", "iq1_s", "iq1_m", "q2_k", "q4_k", "q5_k", "q6_k"):
        from ...quant import qtypes as qt
        from ...quant.params import ggml_convert_qtype
        qname = name if name.endswith("_k") else "gguf_" + name
        packed = ggml_convert_qtype(torch.from_numpy(x.copy()).view(1, -1), qt.qtype_from_name(qname))
        return packed.view(torch.uint8).numpy().tobytes()
    b = x.reshape(-1, 32)
    if name == "q8_0":
        d = np.abs(b).max(axis=1, keepdims=True) / 127.0
        q = np.where(d > 0, np.rint(b / np.where(d > 0, d, 1)), 0).astype(np.int8)
        return np.concatenate([d.astype(np.float16).view(np.uint8), q.view(np.uint8)], axis=1).tobytes()
    if name == "q4_0":
        idx = np.abs(b).argmax(axis=1)
        mx = b[np.arange(b.shape[0]), idx]
        d = (mx / -8.0).reshape(-1, 1)
        inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0)
        q = np.clip((b * inv + 8.5).astype(np.int32), 0, 15).astype(np.uint8)
        packed = q[:, :16] | (q[:, 16:] << 4)
        return np.concatenate([d.astype(np.float16).view(np.uint8), packed], axis=1).tobytes()
    invalidInputError(False, f"writer does not support {name}")


def write_gguf(fpath: str, metadata: Dict[str, object], tensors: Dict[str, Tuple[torch.Tensor, str]], align: int = 32):
    """``tensors``: name -> (float tensor, ggml type name)."""
    head = bytearray()
    head += struct.pack("<I", GGUF_MAGIC) + struct.pack("<I", 3)
    head += struct.pack("<Q", len(tensors)) + struct.pack("<Q", len(metadata))
    for k, v in metadata.items():
        _w_string(head, k)
        _w_value(head, v)
    blobs, off = [], 0
    for name, (t, tname) in tensors.items():
        data = quantize_blocks(t.detach().float().cpu().numpy(), tname)
        _w_string(head, name)
        dims = list(reversed(t.shape))
        head += struct.pack("<I", len(dims))
        for d in dims:
            head += struct.pack("<Q", d)
        head += struct.pack("<I", _NAME_TO_TYPE[tname]) + struct.pack("<Q", off)
        pad = (-len(data)) % align
        blobs.append(data + b"\0" * pad)
        off += len(data) + pad
    with open(fpath, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((-len(head)) % align))
        for b in blobs:
            f.write(b)
