"""Per-layer qtype policy and importance-matrix lookup.

Counterpart of python/llm/src/ipex_llm/transformers/utils.py:186-356 of the reference
(``load_imatrix_data``, ``module_name_process``, ``get_cur_qtype_and_imatrix``): very-low-bit and gguf
mixed presets give some layers more bits (``v_proj``, early ``down_proj``, ``lm_head``), and a llama.cpp
``imatrix`` file supplies per-input-channel importance weights keyed by ``<layer>_<proj>[_<expert>]``.
"""
from __future__ import annotations

import re
import struct

import numpy as np
import torch

from . import qtypes as qt

# "blk.14.attn_output.weight" / "blk.0.ffn_down.3.weight" / "blk.17.ffn_gate_inp.weight"
_IMATRIX_NAME = re.compile(r"^blk\.(\d+)\.(attn|ffn)_([a-z_]+?)(?:\.(\d+))?\.weight$")
_ATTN_SHORT = {"q": "q", "k": "k", "v": "v", "output": "o", "qkv": "qkv"}


def _imatrix_key(layer, proj, expert=None):
    key = f"{layer}_{proj}"
    return key if expert is None else f"{key}_{expert}"


def load_imatrix_data(imatrix_file: str):
    """Read a llama.cpp importance-matrix file: ``n_entries`` records of
    ``(name_len, name, ncall, nval, float32[nval])``; values are averaged over ``ncall``."""
    out = {}
    with open(imatrix_file, "rb") as f:
        (n_entries,) = struct.unpack("<i", f.read(4))
        if n_entries < 1:
            raise ValueError(f"failed reading entries from {imatrix_file}")
        for i in range(n_entries):
            (ln,) = struct.unpack("<i", f.read(4))
            name = f.read(ln).decode("utf-8")
            ncall, nval = struct.unpack("<ii", f.read(8))
            if nval < 1:
                raise ValueError(f"failed reading number of values for entry {i}")
            data = np.frombuffer(f.read(4 * nval), dtype=np.float32).copy()
            if ncall > 0:
                data /= ncall
            m = _IMATRIX_NAME.match(name)
            if m is None:
                key = name
            else:
                layer, kind, proj, expert = m.groups()
                if kind == "attn":
                    proj = _ATTN_SHORT.get(proj, proj[:1])
                key = _imatrix_key(layer, proj, expert)
            out[key] = torch.from_numpy(data).float()
    return out


_LAYER_RE = re.compile(r"layers\.(\d+)\.")
_EXPERT_RE = re.compile(r"experts\.(\d+)\.(w[123])$")
_MOE_MAP = {"w1": "gate", "w2": "down", "w3": "up"}


def module_name_process(full_module_name: str):
    """``model.layers.31.self_attn.o_proj`` -> ("31_o", "31", "o");
    ``model.layers.0.block_sparse_moe.experts.3.w1`` -> ("0_gate_3", "0", "gate"); ``lm_head`` -> itself."""
    if "." not in full_module_name:
        return full_module_name, None, None, None
    lm = _LAYER_RE.search(full_module_name)
    if lm is None:
        return None, None, None, None
    layer = lm.group(1)
    leaf = full_module_name.rsplit(".", 1)[-1]
    em = _EXPERT_RE.search(full_module_name)
    if em is not None:
        cur = _MOE_MAP[em.group(2)]
        return _imatrix_key(layer, cur, em.group(1)), layer, cur, None
    if leaf == "gate" and ("moe" in full_module_name or "mlp" in full_module_name):
        return _imatrix_key(layer, "gate_inp"), layer, "gate_inp", None
    cur = leaf[:-5] if leaf.endswith("_proj") else leaf
    return _imatrix_key(layer, cur), layer, cur, None


def get_cur_qtype_and_imatrix(qtype, full_module_name, imatrix_data, model_config=None):
    cur_qtype, cur_imatrix = qtype, None
    model_type = getattr(model_config, "model_type", None)
    n_layers = getattr(model_config, "num_hidden_layers", None) or 0
    if qtype in (qt.IQ2_XXS, qt.IQ2_XS, qt.IQ1_S, qt.Q2_K):
        key, layer, cur, _ = module_name_process(full_module_name)
        li = int(layer) if layer is not None else -1
        if qtype != qt.Q2_K:
            if model_type == "mixtral":
                if cur == "v":
                    cur_qtype = qt.SYM_INT4
                elif cur == "down" and li in (0, 1, 2, 3):
                    cur_qtype = qt.Q2_K
            elif model_type == "llama" and getattr(model_config, "hidden_size", 0) == 8192:
                if cur == "v":
                    cur_qtype = qt.SYM_INT4
                if cur == "down" and li < n_layers // 8:
                    cur_qtype = qt.Q2_K
            elif cur == "v" or (cur == "down" and li in (0, 1, 10, 11)):
                cur_qtype = qt.Q2_K
            if qtype == qt.IQ1_S and cur == "o":
                cur_qtype = qt.IQ2_XXS
        if imatrix_data is not None and key in imatrix_data:
            cur_imatrix = imatrix_data[key]
        elif key == "lm_head":
            cur_qtype = qt.SYM_INT8
    elif isinstance(qtype, int) and qtype > 100:
        key, layer, cur, _ = module_name_process(full_module_name)
        li = int(layer) if layer is not None else -1
        if key == "lm_head":
            cur_qtype = qt.Q6_K
        elif qtype == qt.gguf_mixed_qtype["gguf_q4k_m"]:
            cur_qtype = qt.Q6_K if (li < n_layers // 2 and cur in ("v", "down")) else qt.Q4_K
        else:
            cur_qtype = qt.Q5_K if (li < n_layers // 8 and cur in ("v", "down")) else qt.Q4_K
    elif imatrix_data is not None:
        key, _, _, _ = module_name_process(full_module_name)
        if key in imatrix_data:
            cur_imatrix = imatrix_data[key]
    return cur_qtype, cur_imatrix


def check_hidden_size(qtype, hidden_size):
    """k-quants need ``hidden_size % 256 == 0``; otherwise fall back to the nearest 64-block type
    (reference utils.py:380-400)."""
    if hidden_size % 256 != 0:
        if qtype == qt.Q4_K:
            return qt.ASYM_INT4
        if qtype == qt.Q5_K:
            return qt.ASYM_INT5
        if qtype == qt.Q6_K:
            return qt.SYM_INT8
        if qtype == qt.FP6_K:
            return qt.FP6
        if qtype == qt.Q2_K:
            return qt.SYM_INT4
    return qtype
