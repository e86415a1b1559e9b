"""Code-book ("i-quant") super-block formats: ``gguf_iq2_xxs``, ``gguf_iq2_xs``, ``gguf_iq1_s``, ``gguf_iq1_m``.

The reference reaches these through its closed quantizer library (qtype ids 21, 22, 24, 25 of
python/llm/src/ipex_llm/ggml/quantize.py:28-61; policy in python/llm/src/ipex_llm/transformers/utils.py:286-356).
Here the byte layout of a super-block is the public GGUF one, so a packed tensor can be exchanged with any GGUF
tool, and both directions are written in plain PyTorch tensor code: the same functions run on the CPU and, for a
weight that already sits on a GPU, on that GPU (a 2048-entry code-book search is a small matmul + arg-min per group
of eight weights, which is slow on a CPU and instant on a B200).

A group of eight weights is stored as the index of one entry of a fixed code-book ("grid"):

* iq2_xxs / iq2_xs: 256 / 512 entries of magnitudes in {8, 25, 43}; the eight signs are seven stored bits plus an
  implied parity bit (the number of negative signs in a group is even); value = d * (2 s + 1) / 8 * grid * sign with a
  4-bit ``s`` per 32 (xxs) or 16 (xs) weights.
* iq1_s / iq1_m: 2048 ternary entries (-1, 0, 1) shifted by +-1/8; value = d * (2 s + 1) * (grid + delta) with a 3-bit
  ``s`` per 32 (s) or 16 (m) weights and the shift sign per 32 (s) or 8 (m) weights.

The grids themselves are tables of the GGUF format; they are taken at run time from the ``gguf`` Python package
(``gguf.quants``).  Without that package these four qtypes raise ``NotImplementedError``.

The quantizer is this package's own: per scale group a few candidate scales are tried, every group of eight picks its
nearest grid entry under the (importance-)weighted squared error, the scale is re-fitted by least squares, the
per-super-block fp16 ``d`` and the small integer scales are derived from the fitted scales, and the entries are chosen
once more under the scales that will actually be stored.
"""
from __future__ import annotations

import functools

import torch

from . import qtypes as qt

QK = 256
TYPE_SIZE = {qt.IQ2_XXS: 66, qt.IQ2_XS: 74, qt.IQ1_S: 50, qt.IQ1_M: 56}
IQ_QTYPES = tuple(TYPE_SIZE)
_DELTA = 0.125
_F16_MAX = 65504.0          # block scales beyond the fp16 range saturate: the block clips instead of decoding to inf
# candidate scales, as fractions of (largest magnitude of the scale group / largest grid magnitude)
_IQ2_FRACTIONS = (0.7, 0.8, 0.9, 1.0, 1.1, 1.25)
_IQ1_FRACTIONS = (0.4, 0.55, 0.7, 0.9)
# blocks per pass: bounds the [groups, grid entries] score matrices to a few hundred MB
_CHUNK = {qt.IQ2_XXS: 4096, qt.IQ2_XS: 2048, qt.IQ1_S: 256, qt.IQ1_M: 256}


def is_iq(qtype: int) -> bool:
    return qtype in TYPE_SIZE


@functools.lru_cache(maxsize=None)
def _grid_cpu(qtype: int) -> torch.Tensor:
    try:
        from gguf import quants as gq
    except ImportError as e:                                          # pragma: no cover - depends on the image
        raise NotImplementedError(
            f"qtype {qt.qtype_name(qtype)} needs the GGUF code-book grids of the `gguf` package, which is not "
            "importable here; use q2_k / sym_int4 / nf4 instead") from e
    cls = {qt.IQ2_XXS: gq.IQ2_XXS, qt.IQ2_XS: gq.IQ2_XS, qt.IQ1_S: gq.IQ1_S, qt.IQ1_M: gq.IQ1_M}[qtype]
    cls.init_grid()
    return torch.from_numpy(cls.grid.reshape(cls.grid_shape).copy()).float()


_grid_dev = {}


def grid(qtype: int, device) -> torch.Tensor:
    """``[entries, 8]`` fp32 grid of the qtype on ``device``."""
    device = torch.device(device)
    key = (qtype, device)
    if key not in _grid_dev:
        _grid_dev[key] = _grid_cpu(qtype).to(device)
    return _grid_dev[key]


@functools.lru_cache(maxsize=None)
def _ksigns_cpu() -> torch.Tensor:
    """seven stored sign bits -> all eight: bit 7 is the parity of the other seven."""
    i = torch.arange(128, dtype=torch.int64)
    par = torch.zeros_like(i)
    for b in range(7):
        par ^= (i >> b) & 1
    return i | (par << 7)


def _sign_table(device) -> torch.Tensor:
    """``[128, 8]`` of +-1."""
    k = _ksigns_cpu().to(device)
    bits = (k.unsqueeze(1) >> torch.arange(8, device=device)) & 1
    return 1.0 - 2.0 * bits.float()


def _u16(b: torch.Tensor) -> torch.Tensor:
    """``[..., 2n]`` bytes -> ``[..., n]`` little-endian unsigned 16-bit values (int64)."""
    b = b.to(torch.int64)
    return b[..., 0::2] | (b[..., 1::2] << 8)


def _bytes16(v: torch.Tensor) -> torch.Tensor:
    """``[..., n]`` 16-bit values -> ``[..., 2n]`` bytes."""
    return torch.stack((v & 0xFF, (v >> 8) & 0xFF), dim=-1).flatten(-2).to(torch.uint8)


def _f16(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float16).float()


# ------------------------------------------------------------------------------------------------
# dequantize
# ------------------------------------------------------------------------------------------------
def dequantize(packed: torch.Tensor, shape, qtype: int, dtype=torch.float32) -> torch.Tensor:
    """Packed super-blocks (uint8, any device) -> dense tensor of ``shape``."""
    ts = TYPE_SIZE[qtype]
    raw = packed.contiguous().view(torch.uint8).reshape(-1)
    n = int(torch.Size(shape).numel())
    nb = n // QK
    blocks = raw[: nb * ts].view(nb, ts)
    dev = blocks.device
    g = grid(qtype, dev)
    if qtype == qt.IQ2_XXS:
        d = _f16(blocks[:, :2])                                              # [nb, 1]
        h = _u16(blocks[:, 2:])                                              # [nb, 32]
        q = (h[:, 0::2] | (h[:, 1::2] << 16)).view(nb, 8, 2)
        q0, q1 = q[..., 0], q[..., 1]
        sh8 = torch.arange(4, device=dev) * 8
        sh7 = torch.arange(4, device=dev) * 7
        idx = (q0.unsqueeze(-1) >> sh8) & 0xFF                               # [nb, 8, 4]
        sidx = (q1.unsqueeze(-1) >> sh7) & 0x7F
        db = d.view(nb, 1, 1, 1) * (0.5 + (q1 >> 28).float()).view(nb, 8, 1, 1) * 0.25
        vals = db * g[idx] * _sign_table(dev)[sidx]                          # [nb, 8, 4, 8]
    elif qtype == qt.IQ2_XS:
        d = _f16(blocks[:, :2])
        qs = _u16(blocks[:, 2:66])                                           # [nb, 32]
        sc = blocks[:, 66:74].to(torch.int64)                                # [nb, 8]
        s = torch.stack((sc & 0xF, sc >> 4), dim=-1).view(nb, 16)            # one per 16 weights
        db = d.view(nb, 1, 1, 1) * (0.5 + s.float()).view(nb, 16, 1, 1) * 0.25
        vals = db * (g[qs & 511] * _sign_table(dev)[qs >> 9]).view(nb, 16, 2, 8)
    elif qtype == qt.IQ1_S:
        d = _f16(blocks[:, :2])
        qs = blocks[:, 2:34].to(torch.int64).view(nb, 8, 4)
        qh = _u16(blocks[:, 34:50])                                          # [nb, 8]
        dl = d.view(nb, 1, 1, 1) * (2 * ((qh >> 12) & 7) + 1).float().view(nb, 8, 1, 1)
        delta = torch.where((qh & 0x8000) == 0, _DELTA, -_DELTA).view(nb, 8, 1, 1)
        hi = (qh.unsqueeze(-1) >> (torch.arange(4, device=dev) * 3)) & 7     # [nb, 8, 4]
        vals = dl * (g[qs | (hi << 8)] + delta)
    elif qtype == qt.IQ1_M:
        qs = blocks[:, :32].to(torch.int64)
        qh = blocks[:, 32:48].to(torch.int64)
        sc = _u16(blocks[:, 48:56])                                          # [nb, 4]
        dbits = ((sc[:, 0] >> 12) & 0xF) | ((sc[:, 1] >> 8) & 0xF0) | ((sc[:, 2] >> 4) & 0xF00) | (sc[:, 3] & 0xF000)
        d = dbits.to(torch.int16).view(torch.float16).float()
        s = ((sc.unsqueeze(-1) >> (torch.arange(4, device=dev) * 3)) & 7).view(nb, 16)
        dl = d.view(nb, 1, 1, 1) * (2 * s + 1).float().view(nb, 16, 1, 1)
        nib = torch.stack((qh & 0xF, qh >> 4), dim=-1).view(nb, 32)          # one per group of eight
        delta = torch.where((nib & 8) == 0, _DELTA, -_DELTA).view(nb, 16, 2, 1)
        vals = dl * (g[qs | ((nib & 7) << 8)].view(nb, 16, 2, 8) + delta)
    else:
        raise NotImplementedError(qt.qtype_name(qtype))
    return vals.reshape(shape).to(dtype)


# ------------------------------------------------------------------------------------------------
# quantize
# ------------------------------------------------------------------------------------------------
def _pick(P, Q, sc):
    """Entry minimising ``sum w (t - sc * g)^2`` for every group: ``P = (w t) . g``, ``Q = w . g^2`` are ``[G, C]``,
    ``sc`` is ``[G, 1]``.  Returns (index, P at index, Q at index)."""
    idx = torch.argmin(sc * (sc * Q - 2.0 * P), dim=1, keepdim=True)
    return idx.squeeze(1), P.gather(1, idx).squeeze(1), Q.gather(1, idx).squeeze(1)


def _fit_scales(assign, amax, fractions, gmax, per):
    """Best scale per scale group.  ``assign(sc_groups) -> (state, Pm, Qm)`` picks entries for one scale per group of
    eight; ``per`` groups of eight share a scale.  Returns the least-squares scale of the best candidate."""
    nsub = amax.numel()
    best_err = torch.full((nsub,), float("inf"), device=amax.device)
    best_sc = torch.zeros(nsub, device=amax.device)
    for f in fractions:
        sc = (amax * (f / gmax)).clamp_min(1e-30)
        _, Pm, Qm = assign(sc.repeat_interleave(per).unsqueeze(1))
        num = Pm.view(nsub, per).sum(1)
        den = Qm.view(nsub, per).sum(1).clamp_min(1e-30)
        err = -num * num / den                               # weighted error at the refitted scale, up to a constant
        take = err < best_err
        best_err = torch.where(take, err, best_err)
        best_sc = torch.where(take, (num / den).clamp_min(0.0), best_sc)
    return best_sc


def _quantize_chunk(x: torch.Tensor, w: torch.Tensor, qtype: int) -> torch.Tensor:
    nb = x.shape[0]
    dev = x.device
    g = grid(qtype, dev)
    gt, g2t = g.t().contiguous(), (g * g).t().contiguous()
    xg, wg = x.view(nb * 32, 8), w.view(nb * 32, 8)
    if qtype in (qt.IQ2_XXS, qt.IQ2_XS):
        per = 4 if qtype == qt.IQ2_XXS else 2                               # groups of eight per scale
        nsc = 32 // per
        neg = xg < 0
        mag = xg.abs()
        # parity: an odd number of negative signs cannot be stored; the cheapest element changes side
        odd = (neg.sum(1) % 2) == 1
        cheapest = torch.argmin(wg * mag * mag, dim=1, keepdim=True)
        flip = torch.zeros_like(neg).scatter_(1, cheapest, True) & odd.unsqueeze(1)
        neg = neg ^ flip
        t = torch.where(flip, -mag, mag)                                     # target in the sign-free space
        P, Q = (wg * t) @ gt, wg @ g2t
        amax = mag.view(nb * nsc, per * 8).amax(1)

        def assign(sc):
            return _pick(P, Q, sc)
        sc = _fit_scales(assign, amax, _IQ2_FRACTIONS, 43.0, per).view(nb, nsc)
        d = (sc.amax(1, keepdim=True) * (8.0 / 31.0)).clamp_max(_F16_MAX).to(torch.float16)
        df = d.float()
        s = torch.where(df > 0, ((sc * 8.0 / df.clamp_min(1e-30) - 1.0) * 0.5).round(), torch.zeros_like(sc))
        s = s.clamp_(0, 15)
        db = df * (2.0 * s + 1.0) * 0.125
        idx, Pm, Qm = assign(db.reshape(-1).repeat_interleave(per).unsqueeze(1).clamp_min(1e-30))
        # refit d for the stored integer scales and entries
        coef = ((2.0 * s + 1.0) * 0.125).reshape(-1).repeat_interleave(per)
        num = (coef * Pm).view(nb, 32).sum(1, keepdim=True)
        den = (coef * coef * Qm).view(nb, 32).sum(1, keepdim=True)
        d = torch.where(den > 0, num / den.clamp_min(1e-30), df).clamp(0.0, _F16_MAX).to(torch.float16)
        pw = (1 << torch.arange(7, device=dev)).to(torch.int64)
        sidx = (neg[:, :7].to(torch.int64) * pw).sum(1)                      # the eighth sign is the parity
        out = torch.empty((nb, TYPE_SIZE[qtype]), dtype=torch.uint8, device=dev)
        out[:, :2] = d.view(torch.uint8)
        s = s.to(torch.int64)
        if qtype == qt.IQ2_XXS:
            idx4, sidx4 = idx.view(nb, 8, 4), sidx.view(nb, 8, 4)
            q0 = (idx4 << (torch.arange(4, device=dev) * 8)).sum(-1)
            q1 = (sidx4 << (torch.arange(4, device=dev) * 7)).sum(-1) | (s << 28)
            words = torch.stack((q0 & 0xFFFF, q0 >> 16, q1 & 0xFFFF, q1 >> 16), dim=-1).view(nb, 32)
            out[:, 2:] = _bytes16(words)
        else:
            out[:, 2:66] = _bytes16((idx | (sidx << 9)).view(nb, 32))
            s2 = s.view(nb, 8, 2)
            out[:, 66:] = (s2[..., 0] | (s2[..., 1] << 4)).to(torch.uint8)
        return out

    # ternary grids with a shift
    per = 4 if qtype == qt.IQ1_S else 2
    nsc = 32 // per
    P0, Q0, R0 = (wg * xg) @ gt, wg @ g2t, wg @ gt
    Sx, Sw = (wg * xg).sum(1, keepdim=True), wg.sum(1, keepdim=True)
    shifted = []
    for dl in (_DELTA, -_DELTA):
        shifted.append((P0 + dl * Sx, Q0 + 2.0 * dl * R0 + dl * dl * Sw))
    del P0, Q0, R0
    amax = xg.abs().view(nb * nsc, per * 8).amax(1)

    def assign_shift(sc, which):
        return _pick(shifted[which][0], shifted[which][1], sc)

    def assign_free(sc):
        """The shift sign is free per group of eight (iq1_m): the one with the smaller error at this scale."""
        i0, p0, q0 = assign_shift(sc, 0)
        i1, p1, q1 = assign_shift(sc, 1)
        s1 = sc.squeeze(1)
        minus = s1 * (s1 * q1 - 2.0 * p1) < s1 * (s1 * q0 - 2.0 * p0)
        return (torch.where(minus, i1, i0), minus), torch.where(minus, p1, p0), torch.where(minus, q1, q0)

    if qtype == qt.IQ1_S:
        # the shift sign belongs to the scale group: fit both, keep the better
        fits = []
        for which in (0, 1):
            sc = _fit_scales(lambda v, k=which: assign_shift(v, k), amax, _IQ1_FRACTIONS, 1.0, per)
            _, Pm, Qm = assign_shift(sc.repeat_interleave(per).unsqueeze(1).clamp_min(1e-30), which)
            err = (sc * (sc * Qm.view(-1, per).sum(1) - 2.0 * Pm.view(-1, per).sum(1)))
            fits.append((sc, err))
        minus_sub = fits[1][1] < fits[0][1]
        sc = torch.where(minus_sub, fits[1][0], fits[0][0]).view(nb, nsc)
    else:
        sc = _fit_scales(assign_free, amax, _IQ1_FRACTIONS, 1.0, per).view(nb, nsc)
    d = (sc.amax(1, keepdim=True) / 15.0).clamp_max(_F16_MAX).to(torch.float16)
    df = d.float()
    s = torch.where(df > 0, ((sc / df.clamp_min(1e-30) - 1.0) * 0.5).round(), torch.zeros_like(sc)).clamp_(0, 7)
    dl = (df * (2.0 * s + 1.0)).reshape(-1).repeat_interleave(per).unsqueeze(1).clamp_min(1e-30)
    if qtype == qt.IQ1_S:
        i0, p0, q0 = assign_shift(dl, 0)
        i1, p1, q1 = assign_shift(dl, 1)
        minus = minus_sub.repeat_interleave(per)
        idx, Pm, Qm = torch.where(minus, i1, i0), torch.where(minus, p1, p0), torch.where(minus, q1, q0)
    else:
        (idx, minus), Pm, Qm = assign_free(dl)
    coef = (2.0 * s + 1.0).reshape(-1).repeat_interleave(per)
    num = (coef * Pm).view(nb, 32).sum(1, keepdim=True)
    den = (coef * coef * Qm).view(nb, 32).sum(1, keepdim=True)
    d = torch.where(den > 0, num / den.clamp_min(1e-30), df).clamp(0.0, _F16_MAX).to(torch.float16)
    out = torch.empty((nb, TYPE_SIZE[qtype]), dtype=torch.uint8, device=dev)
    s = s.to(torch.int64)
    hi = idx >> 8
    if qtype == qt.IQ1_S:
        out[:, :2] = d.view(torch.uint8)
        out[:, 2:34] = (idx & 0xFF).view(nb, 32).to(torch.uint8)
        qh = (hi.view(nb, 8, 4) << (torch.arange(4, device=dev) * 3)).sum(-1) | (s << 12) \
            | (minus_sub.view(nb, 8).to(torch.int64) << 15)
        out[:, 34:] = _bytes16(qh)
    else:
        out[:, :32] = (idx & 0xFF).view(nb, 32).to(torch.uint8)
        nib = (hi | (minus.to(torch.int64) << 3)).view(nb, 16, 2)
        out[:, 32:48] = (nib[..., 0] | (nib[..., 1] << 4)).to(torch.uint8)
        dbits = d.view(torch.int16).to(torch.int64).view(nb) & 0xFFFF
        sc16 = (s.view(nb, 4, 4) << (torch.arange(4, device=dev) * 3)).sum(-1)          # [nb, 4], 12 bits each
        for u in range(4):
            sc16[:, u] |= ((dbits >> (4 * u)) & 0xF) << 12
        out[:, 48:] = _bytes16(sc16)
    return out


def quantize(tensor: torch.Tensor, qtype: int, imatrix: torch.Tensor = None) -> torch.Tensor:
    """fp32 tensor ``[..., K]`` (``K % 256 == 0``) -> packed uint8 super-blocks on the tensor's device.  ``imatrix``
    holds one importance weight per input column (the llama.cpp importance matrix); without it every weight counts
    the same."""
    if tensor.shape[-1] % QK != 0:
        raise ValueError(f"Last dim of input tensor must be multiple of {QK}")
    x = tensor.detach().float().contiguous()
    K = x.shape[-1]
    nb = x.numel() // QK
    xb = x.view(nb, QK)
    if imatrix is not None:
        im = imatrix.to(device=x.device, dtype=torch.float32).reshape(-1)
        if im.numel() != K:
            raise ValueError(f"imatrix has {im.numel()} entries for rows of {K}")
        wb = im.clamp_min(1e-12).view(1, K // QK, QK).expand(x.numel() // K, -1, -1).reshape(nb, QK)
    else:
        wb = None
    out = torch.empty((nb, TYPE_SIZE[qtype]), dtype=torch.uint8, device=x.device)
    step = _CHUNK[qtype]
    for b0 in range(0, nb, step):
        xs = xb[b0:b0 + step]
        ws = wb[b0:b0 + step].contiguous() if wb is not None else torch.ones_like(xs)
        out[b0:b0 + step] = _quantize_chunk(xs, ws, qtype)
    return out.reshape(-1)
