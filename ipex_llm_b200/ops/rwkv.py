"""RWKV operators: v4 scalar-state recurrence, v5 matrix-state linear attention, token-shift mixing.

Same names and argument order as the reference's custom ops (python/llm/src/ipex_llm/transformers/xpu_ops.py:40-56,
used by python/llm/src/ipex_llm/transformers/models/rwkv4.py:40-110 and models/rwkv5.py:40-130).  On CUDA tensors
they run the kernels of ``native/cuda/rwkv_kernels.cu``; on CPU tensors a plain PyTorch loop with the same
numerics (fp32 state) that also serves as the oracle of the GPU tests.
"""
from __future__ import annotations

from typing import Optional

import torch


def _lib():
    from ..native.lib import cuda_lib
    return cuda_lib()


def rwkv_linear_attention_v4(time_decay: torch.Tensor, time_first: torch.Tensor, key: torch.Tensor,
                             value: torch.Tensor, num_state: torch.Tensor, den_state: torch.Tensor,
                             max_state: torch.Tensor) -> torch.Tensor:
    """``time_decay`` is already ``-exp(decay)``.  ``key`` / ``value``: ``[B, T, C]``; the three states ``[B, C]``
    fp32 are updated in place.  Returns ``wkv [B, T, C]`` in the dtype of ``key``."""
    B, T, C = key.shape
    for s in (num_state, den_state, max_state):
        if s.dtype != torch.float32 or not s.is_contiguous() or tuple(s.shape) != (B, C):
            raise ValueError("rwkv states must be contiguous fp32 [B, C] tensors")
    if key.is_cuda:
        from ..native import cuda_api as api
        from ..native.lib import current_stream, ptr
        k, v = key.contiguous(), value.to(key.dtype).contiguous()
        w, u = time_decay.float().contiguous(), time_first.float().contiguous()
        out = torch.empty_like(k)
        rc = _lib().ipex_rwkv_wkv_v4(ptr(w), ptr(u), ptr(k), ptr(v), ptr(out), ptr(num_state), ptr(den_state),
                                     ptr(max_state), B, T, C, api.dtype_code(k.dtype), current_stream())
        api.check(rc, "rwkv_wkv_v4")
        return out
    w, u = time_decay.float(), time_first.float()
    out = torch.empty_like(key)
    a, d, m = num_state, den_state, max_state
    for t in range(T):
        kt, vt = key[:, t].float(), value[:, t].float()
        p = torch.maximum(m, u + kt)
        e1, e2 = torch.exp(m - p), torch.exp(u + kt - p)
        out[:, t] = ((e1 * a + e2 * vt) / (e1 * d + e2)).to(out.dtype)
        q = torch.maximum(m + w, kt)
        f1, f2 = torch.exp(m + w - q), torch.exp(kt - q)
        a.copy_(f1 * a + f2 * vt)
        d.copy_(f1 * d + f2)
        m.copy_(q)
    return out


def rwkv_linear_attention_v5(time_decay: torch.Tensor, time_first: torch.Tensor, receptance: torch.Tensor,
                             key: torch.Tensor, value: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """``time_decay`` is already ``exp(-exp(decay))``; it and ``time_first`` hold ``H * S`` values.
    ``receptance`` / ``key`` / ``value``: fp32 ``[B, H, T, S]``; ``state``: fp32 ``[B, H, S, S]`` updated in place.
    Returns fp32 ``[B, T, H, S]``."""
    B, H, T, S = key.shape
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape) != (B, H, S, S):
        raise ValueError("rwkv5 state must be a contiguous fp32 [B, H, S, S] tensor")
    w = time_decay.float().reshape(H, S).contiguous()
    u = time_first.float().reshape(H, S).contiguous()
    if key.is_cuda and S in (32, 64, 128):
        from ..native import cuda_api as api
        from ..native.lib import current_stream, ptr
        r, k, v = (t.float().contiguous() for t in (receptance, key, value))
        out = torch.empty(B, T, H, S, dtype=torch.float32, device=key.device)
        rc = _lib().ipex_rwkv_linear_attention_v5(ptr(w), ptr(u), ptr(r), ptr(k), ptr(v), ptr(state), ptr(out), B, H,
                                                  T, S, current_stream())
        api.check(rc, "rwkv_linear_attention_v5")
        return out
    out = torch.empty(B, T, H, S, dtype=torch.float32, device=key.device)
    wv, uv = w.view(1, H, S, 1), u.view(1, H, S, 1)
    for t in range(T):
        kv = key[:, :, t].float().unsqueeze(-1) * value[:, :, t].float().unsqueeze(-2)       # [B, H, S, S]
        rt = receptance[:, :, t].float().unsqueeze(-2)                                        # [B, H, 1, S]
        out[:, t] = (rt @ (uv * kv + state)).squeeze(-2)
        state.copy_(kv + wv * state)
    return out


def rwkv_time_shift(hidden: torch.Tensor, shifted: Optional[torch.Tensor], mix: torch.Tensor) -> torch.Tensor:
    """``out[n] = hidden * mix[n] + prev * (1 - mix[n])`` with ``prev[t] = hidden[t-1]`` and ``prev[0]`` = the row
    carried over from the previous call.  ``shifted`` is that carried row as ``[B, C]`` / ``[B, 1, C]``, an already
    shifted ``[B, T, C]`` tensor (the reference's calling convention: only its first row is read), or None for
    zeros.  ``mix``: ``[n, 1, C]`` or ``[n, C]``.  Returns ``[n, B, T, C]``."""
    B, T, C = hidden.shape
    n = mix.shape[0]
    prev = None
    if shifted is not None:
        prev = shifted[:, 0] if shifted.dim() == 3 else shifted
        prev = prev.to(hidden.dtype).contiguous()
    mix2 = mix.reshape(n, C).to(hidden.dtype).contiguous()
    if hidden.is_cuda:
        from ..native import cuda_api as api
        from ..native.lib import current_stream, ptr
        h = hidden.contiguous()
        out = torch.empty(n, B, T, C, dtype=h.dtype, device=h.device)
        rc = _lib().ipex_rwkv_time_shift(ptr(h), ptr(prev), ptr(mix2), ptr(out), B, T, C, n, api.dtype_code(h.dtype),
                                         current_stream())
        api.check(rc, "rwkv_time_shift")
        return out
    first = prev.unsqueeze(1) if prev is not None else torch.zeros(B, 1, C, dtype=hidden.dtype)
    sh = torch.cat([first, hidden[:, :-1]], dim=1)
    m = mix2.view(n, 1, 1, C)
    return hidden.unsqueeze(0) * m + sh.unsqueeze(0) * (1 - m)
