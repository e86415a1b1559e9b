"""RWKV-4 (``model_type == "rwkv"``) forwards on the fused token-shift and recurrence kernels.

Counterpart of python/llm/src/ipex_llm/transformers/models/rwkv4.py:40-110 (attention) and :150-190 (feed
forward), and of the weight rescale the reference applies before quantizing
(python/llm/src/ipex_llm/transformers/convert.py, ``rwkv`` branch of ``_optimize_pre``): the per-block division
of the output projections must happen on the half-precision weights, not on packed low-bit bytes.

State layout is the one of the transformers implementation: ``state[0]`` / ``state[1]`` hold the last hidden
row of the feed-forward / attention token shift as ``[B, C, n_layers]``, ``state[2..4]`` the fp32 numerator,
denominator and running maximum of the recurrence.
"""
from __future__ import annotations

import torch

from ..ops.rwkv import rwkv_linear_attention_v4, rwkv_time_shift


def rescale_before_quantization(module, config):
    """``pre`` hook: run the inference-time rescale of ``RwkvModel`` while the weights are still dense."""
    if module.__class__.__name__ == "RwkvModel" and hasattr(module, "_rescale_layers"):
        module.eval()
        module._rescale_layers()


def _mix(self, names, like):
    cached = self.__dict__.get("_ipex_mix")
    if cached is None or cached.dtype != like.dtype or cached.device != like.device:
        cached = torch.cat([getattr(self, n).data.reshape(1, -1) for n in names]).to(device=like.device,
                                                                                     dtype=like.dtype)
        self.__dict__["_ipex_mix"] = cached
    return cached


def rwkv4_attention_forward(self, hidden, state=None, use_cache=False):
    B, T, _ = hidden.shape
    lid = self.layer_id
    prev = state[1][:, :, lid] if state is not None else None
    mix = _mix(self, ("time_mix_key", "time_mix_value", "time_mix_receptance"), hidden)
    key, value, receptance = rwkv_time_shift(hidden, prev, mix)
    key = self.key(key)
    value = self.value(value)
    receptance = torch.sigmoid(self.receptance(receptance))
    if state is not None:
        state[1][:, :, lid] = hidden[:, -1]
    A = key.shape[-1]
    if state is not None:
        num, den, mx = (state[i][:, :, lid].float().contiguous() for i in (2, 3, 4))
    else:
        num = torch.zeros(B, A, dtype=torch.float32, device=hidden.device)
        den = torch.zeros_like(num)
        mx = torch.full_like(num, -1e38)
    wkv = rwkv_linear_attention_v4(-torch.exp(self.time_decay.float()), self.time_first.float(), key, value, num,
                                   den, mx)
    if state is not None:
        state[2][:, :, lid] = num
        state[3][:, :, lid] = den
        state[4][:, :, lid] = mx
    return self.output(receptance * wkv), state


def rwkv4_ffn_forward(self, hidden, state=None):
    lid = self.layer_id
    prev = state[0][:, :, lid] if state is not None else None
    mix = _mix(self, ("time_mix_key", "time_mix_receptance"), hidden)
    key, receptance = rwkv_time_shift(hidden, prev, mix)
    key = torch.square(torch.relu(self.key(key)))
    value = self.value(key)
    receptance = torch.sigmoid(self.receptance(receptance))
    if state is not None:
        state[0][:, :, lid] = hidden[:, -1]
    return receptance * value, state
