"""KV caches: block-grown pre-allocated storage, fp8 (e5m2) storage, SnapKV compression.

Counterparts of the reference's ``DynamicNormalCache``, ``DynamicFp8Cache``, ``DynamicCompressCache`` and
``DynamicCompressFp8Cache`` (python/llm/src/ipex_llm/transformers/kv.py:32-449) and of its allocators
(python/llm/src/ipex_llm/transformers/models/utils.py:39-148), re-expressed on the transformers-5 cache API:
each cache is a ``Cache`` whose layers are ``CacheLayerMixin`` objects with

* pre-allocated ``[B, H, capacity, D]`` storage that grows in blocks of ``KV_CACHE_ALLOC_BLOCK_LENGTH`` tokens
  (no ``torch.cat`` per token),
* an O(1) ``crop`` (speculative / lookup decoding rejects drafted tokens by moving the length),
* for fp8: one byte per element (e5m2 = the upper byte of the fp16 value, round-to-nearest-even), stored as
  uint8 and handed to the attention op still packed.
"""
from __future__ import annotations

import os

import torch
from transformers.cache_utils import Cache, DynamicLayer

KV_CACHE_ALLOC_BLOCK_LENGTH = int(os.environ.get("KV_CACHE_ALLOC_BLOCK_LENGTH", 256))


def fp8_e5m2_quantize(x: torch.Tensor) -> torch.Tensor:
    """Float tensor -> uint8 tensor of e5m2 codes (saturating, round-to-nearest-even)."""
    if x.is_cuda:
        from . import cuda_ops
        return cuda_ops.quantize_kv_e5m2(x)
    return x.to(torch.float16).clamp(-57344.0, 57344.0).to(torch.float8_e5m2).view(torch.uint8)


def fp8_e5m2_dequantize(x: torch.Tensor, dtype=torch.float16) -> torch.Tensor:
    if x.is_cuda:
        from . import cuda_ops
        return cuda_ops.dequantize_kv_e5m2(x, dtype)
    return x.view(torch.float8_e5m2).to(dtype)


class NormalLayer(DynamicLayer):
    """Pre-allocated, block-grown KV storage for one layer."""

    storage_dtype = None  # None -> dtype of the incoming states
    extra_alloc = KV_CACHE_ALLOC_BLOCK_LENGTH

    def __init__(self):
        super().__init__()
        self.length = 0
        self._k = None
        self._v = None

    def lazy_initialization(self, key_states, value_states):
        self.dtype, self.device = key_states.dtype, key_states.device
        self.is_initialized = True

    def _encode(self, x):
        return x

    def _alloc(self, bsz, heads, cap, dk, dv, dtype, device):
        k = torch.empty(bsz, heads, cap, dk, dtype=dtype, device=device)
        v = torch.empty(bsz, heads, cap, dv, dtype=dtype, device=device)
        return k, v

    def preallocate(self, bsz, heads, capacity, dk, dv, act_dtype, device):
        """Reserve ``capacity`` tokens up front (the decode engine reads this storage in place)."""
        self.dtype, self.device = act_dtype, device
        self.is_initialized = True
        self._k, self._v = self._alloc(bsz, heads, capacity, dk, dv, self.storage_dtype or act_dtype, device)
        self.length = 0
        self.keys, self.values = self._k[:, :, :0], self._v[:, :, :0]

    def set_length(self, n: int):
        """The decode engine appends in place; it reports the new length here."""
        self.length = n
        self.keys, self.values = self._k[:, :, :n], self._v[:, :, :n]

    def _ensure(self, key_states, value_states, new_len):
        bsz, heads, _, dk = key_states.shape
        dv = value_states.shape[-1]
        sdtype = self.storage_dtype or key_states.dtype
        if self._k is None:
            cap = new_len + self.extra_alloc
            self._k, self._v = self._alloc(bsz, heads, cap, dk, dv, sdtype, key_states.device)
        elif new_len > self._k.shape[2]:
            cap = new_len + self.extra_alloc
            nk, nv = self._alloc(bsz, heads, cap, dk, dv, sdtype, key_states.device)
            nk[:, :, :self.length] = self._k[:, :, :self.length]
            nv[:, :, :self.length] = self._v[:, :, :self.length]
            self._k, self._v = nk, nv

    def update(self, key_states, value_states, *args, **kwargs):
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        q_len = key_states.shape[2]
        new_len = self.length + q_len
        self._ensure(key_states, value_states, new_len)
        self._k[:, :, self.length:new_len] = self._encode(key_states)
        self._v[:, :, self.length:new_len] = self._encode(value_states)
        self.length = new_len
        self.keys = self._k[:, :, :new_len]
        self.values = self._v[:, :, :new_len]
        return self.keys, self.values

    def reserve(self, extra_tokens: int):
        """Make room for ``extra_tokens`` more tokens (speculative decoding drafts several per round)."""
        if self._k is not None and self.length + extra_tokens > self._k.shape[2]:
            self._ensure(self._k[:, :, :1], self._v[:, :, :1], self.length + extra_tokens)
            self.keys = self._k[:, :, :self.length]
            self.values = self._v[:, :, :self.length]

    def get_seq_length(self) -> int:
        return self.length

    def get_mask_sizes(self, query_length: int):
        return self.length + query_length, 0

    def crop(self, max_length: int) -> None:
        if max_length < 0:
            max_length = self.length - abs(max_length)
        if self.length <= max_length:
            return
        self.length = max_length
        if self._k is not None:
            self.keys = self._k[:, :, :max_length]
            self.values = self._v[:, :, :max_length]

    def reset(self):
        self.length = 0
        if self._k is not None:
            self.keys = self._k[:, :, :0]
            self.values = self._v[:, :, :0]

    def batch_repeat_interleave(self, repeats: int):
        if self._k is not None:
            self._k = self._k.repeat_interleave(repeats, dim=0)
            self._v = self._v.repeat_interleave(repeats, dim=0)
            self.keys, self.values = self._k[:, :, :self.length], self._v[:, :, :self.length]

    def batch_select_indices(self, indices):
        if self._k is not None:
            self._k = self._k[indices, ...]
            self._v = self._v[indices, ...]
            self.keys, self.values = self._k[:, :, :self.length], self._v[:, :, :self.length]

    def reorder_cache(self, beam_idx):
        if self._k is not None:
            self._k = self._k.index_select(0, beam_idx.to(self._k.device))
            self._v = self._v.index_select(0, beam_idx.to(self._v.device))
            self.keys, self.values = self._k[:, :, :self.length], self._v[:, :, :self.length]


class Fp8Layer(NormalLayer):
    """One byte per element: e5m2 codes held as uint8 (+512 tokens of head-room per allocation)."""

    storage_dtype = torch.uint8
    extra_alloc = 2 * KV_CACHE_ALLOC_BLOCK_LENGTH

    def _encode(self, x):
        return fp8_e5m2_quantize(x)

    def restore(self, dtype=None):
        """Dequantized (keys, values) views, for consumers that cannot read packed KV."""
        dtype = dtype or self.dtype
        return fp8_e5m2_dequantize(self.keys, dtype), fp8_e5m2_dequantize(self.values, dtype)


def int4_kv_quantize(x: torch.Tensor) -> torch.Tensor:
    """``[..., D]`` float -> ``[..., D/2 + 2]`` uint8: symmetric 4-bit codes of every row (scale = amax / 7, two codes
    per byte, even element in the low nibble) followed by the row's fp16 scale."""
    xf = x.float()
    scale = (xf.abs().amax(dim=-1, keepdim=True) / 7.0).clamp_min(1e-8).to(torch.float16)
    q = torch.clamp(torch.round(xf / scale.float()), -8, 7).to(torch.int16) + 8
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).to(torch.uint8)
    return torch.cat([packed, scale.view(torch.uint8).reshape(*scale.shape[:-1], 2)], dim=-1)


def int4_kv_dequantize(p: torch.Tensor, dtype=torch.float16) -> torch.Tensor:
    codes, scale = p[..., :-2], p[..., -2:].contiguous().view(torch.float16)
    lo = (codes & 0xF).to(torch.int16) - 8
    hi = (codes >> 4).to(torch.int16) - 8
    q = torch.stack([lo, hi], dim=-1).reshape(*codes.shape[:-1], codes.shape[-1] * 2)
    return (q.to(torch.float32) * scale.float()).to(dtype)


class Int4Layer(NormalLayer):
    """Four bits per element plus one fp16 scale per (token, head): each stored row is ``D/2`` code bytes followed by
    the scale's two bytes, so the block-grown storage of ``NormalLayer`` serves unchanged.  ``update`` hands the
    attention the prompt's own K / V on the first call (like the engines, which attend to what they have just
    computed) and the dequantized cache afterwards; the fused decode kernels do not read this format."""

    storage_dtype = torch.uint8
    extra_alloc = 2 * KV_CACHE_ALLOC_BLOCK_LENGTH

    def _alloc(self, bsz, heads, cap, dk, dv, dtype, device):
        if getattr(self, "_pk", None) is None:
            self._pk, self._pv = dk // 2 + 2, dv // 2 + 2        # first call: widths of the float rows
        k = torch.empty(bsz, heads, cap, self._pk, dtype=torch.uint8, device=device)
        v = torch.empty(bsz, heads, cap, self._pv, dtype=torch.uint8, device=device)
        return k, v

    def _encode(self, x):
        return int4_kv_quantize(x)

    def update(self, key_states, value_states, *args, **kwargs):
        fresh = self.length == 0
        super().update(key_states, value_states, *args, **kwargs)
        if fresh:
            return key_states, value_states
        return self.restore(key_states.dtype)

    def restore(self, dtype=None):
        dtype = dtype or self.dtype
        return int4_kv_dequantize(self.keys, dtype), int4_kv_dequantize(self.values, dtype)


def compress_kv(query_states, key_states, value_states, attention_mask, num_key_value_groups, window_size=32,
                max_capacity_prompt=1024, kernel_size=7, pooling="maxpool"):
    """SnapKV prompt compression: keep the ``max_capacity_prompt - window_size`` prompt positions with the highest
    pooled attention mass from the last ``window_size`` queries, plus those last positions
    (reference kv.py:171-243)."""
    bsz, num_heads, q_len, head_dim = query_states.shape
    if q_len <= max_capacity_prompt:
        return key_states, value_states
    sliding_window_size = getattr(compress_kv, "sliding_window", None)
    if sliding_window_size is not None and q_len > sliding_window_size:
        key_states = key_states[:, :, -sliding_window_size:]
        value_states = value_states[:, :, -sliding_window_size:]
    kv_len = key_states.shape[2]
    k_rep = key_states.repeat_interleave(num_key_value_groups, dim=1) if num_key_value_groups > 1 else key_states
    q_win = query_states[..., -window_size:, :].float()
    attn = torch.matmul(q_win, k_rep.float().transpose(2, 3)) / (head_dim ** 0.5)
    mask = torch.full((window_size, window_size), torch.finfo(attn.dtype).min, device=attn.device)
    idx = torch.arange(window_size, device=attn.device)
    mask.masked_fill_(idx < (idx + 1).view(-1, 1), 0)
    attn[:, :, -window_size:, -window_size:] += mask[None, None]
    attn = torch.softmax(attn, dim=-1)
    score = attn[:, :, -window_size:, :-window_size].sum(dim=-2)
    if pooling == "avgpool":
        pooled = torch.nn.functional.avg_pool1d(score, kernel_size=kernel_size, padding=kernel_size // 2, stride=1)
    else:
        pooled = torch.nn.functional.max_pool1d(score, kernel_size=kernel_size, padding=kernel_size // 2, stride=1)
    if num_key_value_groups > 1:
        pooled = pooled.view(bsz, num_heads // num_key_value_groups, num_key_value_groups, -1).sum(dim=2)
    keep = pooled.topk(max_capacity_prompt - window_size, dim=-1).indices.sort(dim=-1).values
    keep = keep.unsqueeze(-1).expand(-1, -1, -1, head_dim)
    k_past = key_states[:, :, :kv_len - window_size].gather(dim=2, index=keep)
    v_past = value_states[:, :, :kv_len - window_size].gather(dim=2, index=keep)
    k_new = torch.cat([k_past, key_states[:, :, -window_size:]], dim=2)
    v_new = torch.cat([v_past, value_states[:, :, -window_size:]], dim=2)
    return k_new, v_new


class CompressLayer(NormalLayer):
    """SnapKV layer: the prefill call stores a compressed prompt; ``real_kv_len`` keeps the true position."""

    def __init__(self):
        super().__init__()
        self.real_kv_len = 0

    def update(self, key_states, value_states, *args, query_states=None, attention_mask=None,
               num_key_value_groups=1, window_size=32, max_capacity_prompt=1024, kernel_size=7, **kwargs):
        q_len = key_states.shape[2]
        first = self.length == 0 and query_states is not None and q_len > 1
        self.real_kv_len += q_len
        if first:
            k_c, v_c = compress_kv(query_states, key_states, value_states, attention_mask, num_key_value_groups,
                                   window_size, max_capacity_prompt, kernel_size)
            super().update(k_c, v_c)
            # prefill attends to the full prompt; later steps see the compressed cache
            return key_states, value_states
        return super().update(key_states, value_states)

    def get_mask_sizes(self, query_length: int):
        return self.length + query_length, 0


class CompressFp8Layer(CompressLayer):
    storage_dtype = torch.uint8
    extra_alloc = 2 * KV_CACHE_ALLOC_BLOCK_LENGTH

    def _encode(self, x):
        return fp8_e5m2_quantize(x)


class _BlockCache(Cache):
    layer_cls = NormalLayer

    def __init__(self, config=None, num_layers=None, **kwargs):
        super().__init__(layer_class_to_replicate=self.layer_cls)
        self.config = config

    def reserve(self, extra_tokens: int):
        for layer in self.layers:
            if hasattr(layer, "reserve"):
                layer.reserve(extra_tokens)

    @property
    def real_kv_len(self):
        layer = self.layers[0] if self.layers else None
        return getattr(layer, "real_kv_len", self.get_seq_length())


class DynamicNormalCache(_BlockCache):
    layer_cls = NormalLayer


class DynamicFp8Cache(_BlockCache):
    layer_cls = Fp8Layer


class DynamicInt4Cache(_BlockCache):
    """4-bit KV cache (IPEX_LLM_QUANTIZE_KV_CACHE=int4): 4.25 bits per element at head dim 128."""
    layer_cls = Int4Layer


class DynamicCompressCache(_BlockCache):
    layer_cls = CompressLayer


class DynamicCompressFp8Cache(_BlockCache):
    layer_cls = CompressFp8Layer


def is_fp8_cache(cache) -> bool:
    return isinstance(cache, (DynamicFp8Cache, DynamicCompressFp8Cache))


def is_ipex_cache(cache) -> bool:
    return isinstance(cache, _BlockCache)
