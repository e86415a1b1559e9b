"""Checkpoints of "remote code" families loaded WITHOUT their remote code.

The reference supports ChatGLM2/3 / GLM-4, Baichuan(2), InternLM / InternLM2, Qwen (v1), MiniCPM(3) and Aquila by
patching the forwards of the modeling files those checkpoints ship (``trust_remote_code=True``;
python/llm/src/ipex_llm/transformers/convert.py:1337 chatglm, :1463 baichuan, :1513-1524 internlm / internlm2, :1559
qwen, :1676 aquila, :1876 minicpm; models/chatglm2.py, baichuan.py, internlm.py, qwen.py, minicpm.py).  Each of these
architectures is, tensor for tensor, an architecture that ``transformers`` implements natively under another name:

    chatglm (v2 / v3 / glm-4-9b)  ->  Glm      (interleaved rotary on half of every head, fused gate/up, qkv bias)
    baichuan (7B / 13B, v1 / v2)  ->  Llama    (fused W_pack; Baichuan2 normalises the lm_head rows; the 13B
                                               models replace rotary positions by linear attention biases)
    internlm                      ->  Llama    (biases on q, k, v, o)
    internlm2                     ->  Llama    (wqkv interleaved per kv head)
    qwen (v1)                     ->  Qwen2    (fused c_attn with bias; w2 is the gate, w1 the up projection)
    minicpm (1B / 2B)             ->  Granite  (embedding, residual and logit multipliers)
    minicpm3                      ->  DeepseekV2, dense (latent attention; multipliers folded into the weights)
    aquila / aquila2              ->  Llama

So this module reads ``config.json`` and the weight shards, renames / splits the tensors, and builds the native class;
from there the family's registry entry (merged qkv, fused kernels, graph engine for the llama-like ones) applies as for
any other checkpoint, and nothing of the checkpoint's Python files is executed.  Not covered: ChatGLM-6B v1 (2-D
positions), Yuan (convolutional filter) - those return ``None``
here and fall through to ``transformers``' own loader.
"""
from __future__ import annotations

import glob
import json
import math
import os
from typing import Callable, Dict, Optional, Tuple

import torch


def _read_state_dict(path: str) -> Dict[str, torch.Tensor]:
    state: Dict[str, torch.Tensor] = {}
    st = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if st:
        from safetensors.torch import load_file
        for f in st:
            state.update(load_file(f))
        return state
    for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
        state.update(torch.load(f, map_location="cpu", weights_only=True))
    return state


def _rename(state, table):
    """``table``: list of (old substring, new substring) applied in order to every key."""
    out = {}
    for k, v in state.items():
        for a, b in table:
            k = k.replace(a, b)
        out[k] = v
    return out


# ------------------------------------------------------------------------------------------------
# chatglm2 / chatglm3 / glm-4-9b  ->  Glm
# ------------------------------------------------------------------------------------------------
def _chatglm(c: dict):
    from transformers import GlmConfig
    if c.get("position_encoding_2d") or "ffn_hidden_size" not in c:
        return None          # ChatGLM-6B v1
    nh, hd = c["num_attention_heads"], c.get("kv_channels", c["hidden_size"] // c["num_attention_heads"])
    ng = c.get("multi_query_group_num", nh) if c.get("multi_query_attention", False) else nh
    cfg = GlmConfig(vocab_size=c.get("padded_vocab_size", c.get("vocab_size")), hidden_size=c["hidden_size"],
                    intermediate_size=c["ffn_hidden_size"], num_hidden_layers=c["num_layers"],
                    num_attention_heads=nh, num_key_value_heads=ng, head_dim=hd, partial_rotary_factor=0.5,
                    rms_norm_eps=c.get("layernorm_epsilon", 1e-5), attention_bias=c.get("add_qkv_bias", True),
                    rope_theta=10000.0 * c.get("rope_ratio", 1.0), max_position_embeddings=c.get("seq_length", 8192),
                    tie_word_embeddings=False, hidden_act="silu", pad_token_id=c.get("pad_token_id", 0),
                    eos_token_id=c.get("eos_token_id", 2))

    def convert(state):
        out = {}
        for k, v in state.items():
            if k.endswith("rotary_pos_emb.inv_freq"):
                continue
            k = k.replace("transformer.embedding.word_embeddings.", "model.embed_tokens.")
            k = k.replace("transformer.encoder.final_layernorm.", "model.norm.")
            k = k.replace("transformer.output_layer.", "lm_head.")
            k = k.replace("transformer.encoder.layers.", "model.layers.")
            k = k.replace(".self_attention.dense.", ".self_attn.o_proj.")
            k = k.replace(".mlp.dense_h_to_4h.", ".mlp.gate_up_proj.")
            k = k.replace(".mlp.dense_4h_to_h.", ".mlp.down_proj.")
            if ".self_attention.query_key_value." in k:
                q, kk, vv = torch.split(v, [nh * hd, ng * hd, ng * hd], dim=0)
                for name, t in (("q_proj", q), ("k_proj", kk), ("v_proj", vv)):
                    out[k.replace(".self_attention.query_key_value.", f".self_attn.{name}.")] = t.contiguous()
                continue
            out[k] = v
        return out
    return cfg, convert


# ------------------------------------------------------------------------------------------------
# baichuan-7B / Baichuan2-7B  ->  Llama
# ------------------------------------------------------------------------------------------------
def _baichuan(c: dict):
    from transformers import LlamaConfig
    # 13B checkpoints have no rotary positions: attention carries linear biases (ALiBi).  The Llama classes are kept
    # and the config field ``ipex_alibi`` tells the package's attention forward to skip the rotation and add the bias.
    alibi = "max_position_embeddings" not in c and "model_max_length" in c
    v2 = c.get("vocab_size") == 125696
    cfg = LlamaConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"],
                      intermediate_size=c["intermediate_size"], num_hidden_layers=c["num_hidden_layers"],
                      num_attention_heads=c["num_attention_heads"], rms_norm_eps=c.get("rms_norm_eps", 1e-6),
                      max_position_embeddings=c.get("max_position_embeddings", c.get("model_max_length", 4096)),
                      tie_word_embeddings=False, pad_token_id=c.get("pad_token_id", 0),
                      bos_token_id=c.get("bos_token_id", 1), eos_token_id=c.get("eos_token_id", 2))
    if alibi:
        cfg.ipex_alibi = True
    H = c["hidden_size"]

    def convert(state):
        out = {}
        for k, v in state.items():
            if ".self_attn.W_pack." in k:
                q, kk, vv = torch.split(v, [H, H, H], dim=0)
                for name, t in (("q_proj", q), ("k_proj", kk), ("v_proj", vv)):
                    out[k.replace(".self_attn.W_pack.", f".self_attn.{name}.")] = t.contiguous()
            elif k == "lm_head.weight" and v2:
                out[k] = torch.nn.functional.normalize(v.float()).to(v.dtype)   # NormHead at inference time
            elif not k.endswith("rotary_emb.inv_freq"):
                out[k] = v
        return out
    return cfg, convert


# ------------------------------------------------------------------------------------------------
# internlm (v1)  ->  Llama with attention biases;  aquila  ->  Llama
# ------------------------------------------------------------------------------------------------
def _llama_named(c: dict, bias_key: Optional[str] = None):
    from transformers import LlamaConfig
    cfg = LlamaConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"],
                      intermediate_size=c["intermediate_size"], num_hidden_layers=c["num_hidden_layers"],
                      num_attention_heads=c["num_attention_heads"],
                      num_key_value_heads=c.get("num_key_value_heads") or c["num_attention_heads"],
                      rms_norm_eps=c.get("rms_norm_eps", 1e-6), rope_theta=c.get("rope_theta", 10000.0),
                      max_position_embeddings=c.get("max_position_embeddings", 2048),
                      attention_bias=bool(c.get(bias_key, True)) if bias_key else False, tie_word_embeddings=False,
                      pad_token_id=c.get("pad_token_id", 0), bos_token_id=c.get("bos_token_id", 1),
                      eos_token_id=c.get("eos_token_id", 2))

    def convert(state):
        return {k: v for k, v in state.items() if not k.endswith("rotary_emb.inv_freq")}
    return cfg, convert


def _internlm(c: dict):
    return _llama_named(c, "bias")


def _aquila(c: dict):
    return _llama_named(c)


# ------------------------------------------------------------------------------------------------
# internlm2  ->  Llama
# ------------------------------------------------------------------------------------------------
def _internlm2(c: dict):
    from transformers import LlamaConfig
    nh = c["num_attention_heads"]
    nkv = c.get("num_key_value_heads") or nh
    hd = c["hidden_size"] // nh
    groups = nh // nkv
    kw = {}
    if c.get("rope_scaling"):
        kw["rope_scaling"] = c["rope_scaling"]
    cfg = LlamaConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"],
                      intermediate_size=c["intermediate_size"], num_hidden_layers=c["num_hidden_layers"],
                      num_attention_heads=nh, num_key_value_heads=nkv, rms_norm_eps=c.get("rms_norm_eps", 1e-6),
                      rope_theta=c.get("rope_theta", 10000.0),
                      max_position_embeddings=c.get("max_position_embeddings", 2048),
                      attention_bias=bool(c.get("bias", False)), tie_word_embeddings=False,
                      pad_token_id=c.get("pad_token_id", 0), bos_token_id=c.get("bos_token_id", 1),
                      eos_token_id=c.get("eos_token_id", 2), **kw)

    def convert(state):
        out = {}
        for k, v in state.items():
            if k.endswith("rotary_emb.inv_freq"):
                continue
            k = k.replace("model.tok_embeddings.", "model.embed_tokens.")
            k = k.replace("output.", "lm_head.") if k.startswith("output.") else k
            k = k.replace(".attention_norm.", ".input_layernorm.").replace(".ffn_norm.", ".post_attention_layernorm.")
            k = k.replace(".attention.wo.", ".self_attn.o_proj.")
            k = k.replace(".feed_forward.w1.", ".mlp.gate_proj.").replace(".feed_forward.w3.", ".mlp.up_proj.")
            k = k.replace(".feed_forward.w2.", ".mlp.down_proj.")
            if ".attention.wqkv." in k:
                # rows are grouped per kv head: [groups query heads | key | value] x head_dim
                w = v.view(nkv, groups + 2, hd, *v.shape[1:])
                q = w[:, :groups].reshape(nh * hd, *v.shape[1:])
                kk = w[:, groups].reshape(nkv * hd, *v.shape[1:])
                vv = w[:, groups + 1].reshape(nkv * hd, *v.shape[1:])
                for name, t in (("q_proj", q), ("k_proj", kk), ("v_proj", vv)):
                    out[k.replace(".attention.wqkv.", f".self_attn.{name}.")] = t.contiguous()
                continue
            out[k] = v
        return out
    return cfg, convert


# ------------------------------------------------------------------------------------------------
# qwen (v1)  ->  Qwen2
# ------------------------------------------------------------------------------------------------
def _qwen(c: dict):
    from transformers import Qwen2Config
    H = c["hidden_size"]
    cfg = Qwen2Config(vocab_size=c["vocab_size"], hidden_size=H, intermediate_size=c["intermediate_size"] // 2,
                      num_hidden_layers=c["num_hidden_layers"], num_attention_heads=c["num_attention_heads"],
                      num_key_value_heads=c["num_attention_heads"], rms_norm_eps=c.get("layer_norm_epsilon", 1e-6),
                      rope_theta=c.get("rotary_emb_base", 10000.0),
                      max_position_embeddings=c.get("seq_length", c.get("max_position_embeddings", 8192)),
                      tie_word_embeddings=False, use_sliding_window=False)

    def convert(state):
        out = {}
        for k, v in state.items():
            k = k.replace("transformer.wte.", "model.embed_tokens.").replace("transformer.ln_f.", "model.norm.")
            k = k.replace("transformer.h.", "model.layers.")
            k = k.replace(".ln_1.", ".input_layernorm.").replace(".ln_2.", ".post_attention_layernorm.")
            k = k.replace(".attn.c_proj.", ".self_attn.o_proj.")
            k = k.replace(".mlp.w1.", ".mlp.up_proj.").replace(".mlp.w2.", ".mlp.gate_proj.")
            k = k.replace(".mlp.c_proj.", ".mlp.down_proj.")
            if ".attn.c_attn." in k:
                q, kk, vv = torch.split(v, [H, H, H], dim=0)
                for name, t in (("q_proj", q), ("k_proj", kk), ("v_proj", vv)):
                    out[k.replace(".attn.c_attn.", f".self_attn.{name}.")] = t.contiguous()
                continue
            if "rotary_emb" in k:
                continue
            out[k] = v
        return out
    return cfg, convert


# ------------------------------------------------------------------------------------------------
# minicpm (1B / 2B)  ->  Granite
# ------------------------------------------------------------------------------------------------
def _minicpm(c: dict):
    from transformers import GraniteConfig
    nh = c["num_attention_heads"]
    hd = c["hidden_size"] // nh
    cfg = GraniteConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"],
                        intermediate_size=c["intermediate_size"], num_hidden_layers=c["num_hidden_layers"],
                        num_attention_heads=nh, num_key_value_heads=c.get("num_key_value_heads") or nh,
                        rms_norm_eps=c.get("rms_norm_eps", 1e-5), rope_theta=c.get("rope_theta", 10000.0),
                        max_position_embeddings=c.get("max_position_embeddings", 2048),
                        embedding_multiplier=float(c.get("scale_emb", 1.0)),
                        residual_multiplier=float(c.get("scale_depth", 1.0)) / math.sqrt(c["num_hidden_layers"]),
                        logits_scaling=float(c["hidden_size"]) / float(c.get("dim_model_base", c["hidden_size"])),
                        attention_multiplier=1.0 / math.sqrt(hd), tie_word_embeddings=False,
                        pad_token_id=c.get("pad_token_id", 0), bos_token_id=c.get("bos_token_id", 1),
                        eos_token_id=c.get("eos_token_id", 2))

    def convert(state):
        out = {k: v for k, v in state.items() if not k.endswith("rotary_emb.inv_freq")}
        if "lm_head.weight" not in out:          # the 2B checkpoints tie the output layer to the embedding
            out["lm_head.weight"] = out["model.embed_tokens.weight"]
        return out
    return cfg, convert


# ------------------------------------------------------------------------------------------------
# minicpm3  ->  DeepseekV2 (dense): multi-head latent attention with the MiniCPM multipliers folded into the weights
# ------------------------------------------------------------------------------------------------
def _interleave_rows(w, start: int, n: int):
    """Rows ``start .. start+n`` hold a rotary block in half-split order (pair = (i, i + n/2), what ``rotate_half``
    rotates); reorder them to interleaved order (pair = (2i, 2i+1), what a complex multiplication rotates).  Applied
    to the rows that produce q and k alike, the scores do not change."""
    half = n // 2
    idx = torch.arange(n).view(2, half).t().reshape(-1) + start
    out = w.clone()
    out[start:start + n] = w[idx]
    return out


def _minicpm3(c: dict):
    """MiniCPM3 (reference models/minicpm3.py:116-230) is DeepSeek-V2's latent attention on a dense MLP, plus the
    MiniCPM multipliers.  The native DeepseekV2 classes have no multipliers, so they are folded into weights that
    follow them: ``scale_emb`` into the embedding, ``scale_depth / sqrt(layers)`` into ``o_proj`` and ``down_proj`` (the
    last linear of each residual branch), ``dim_model_base / hidden`` into the output layer.  MiniCPM3 rotates the
    two halves of the rotary block, the native class rotates adjacent pairs: the rotary rows of ``q_b_proj`` and
    ``kv_a_proj_with_mqa`` are reordered accordingly."""
    from transformers import DeepseekV2Config
    L, H, nh = c["num_hidden_layers"], c["hidden_size"], c["num_attention_heads"]
    nope, rope_d = c["qk_nope_head_dim"], c["qk_rope_head_dim"]
    v_dim = c.get("v_head_dim") or H // nh
    rp = {"rope_type": "default", "rope_theta": float(c.get("rope_theta", 10000.0))}
    rs = c.get("rope_scaling") or {}
    if (rs.get("type") or rs.get("rope_type")) == "longrope":
        rp.update(rope_type="longrope", short_factor=list(rs["short_factor"]), long_factor=list(rs["long_factor"]),
                  original_max_position_embeddings=int(rs["original_max_position_embeddings"]))
    cfg = DeepseekV2Config(vocab_size=c["vocab_size"], hidden_size=H, intermediate_size=c["intermediate_size"],
                           num_hidden_layers=L, num_attention_heads=nh, num_key_value_heads=nh,
                           max_position_embeddings=c.get("max_position_embeddings", 32768),
                           rms_norm_eps=c.get("rms_norm_eps", 1e-5), rope_parameters=rp,
                           q_lora_rank=c.get("q_lora_rank"), kv_lora_rank=c["kv_lora_rank"], qk_nope_head_dim=nope,
                           qk_rope_head_dim=rope_d, v_head_dim=v_dim, head_dim=rope_d,
                           first_k_dense_replace=L, n_routed_experts=1, n_shared_experts=0, num_experts_per_tok=1,
                           moe_intermediate_size=c["intermediate_size"], tie_word_embeddings=False,
                           pad_token_id=c.get("pad_token_id", 0), bos_token_id=c.get("bos_token_id", 1),
                           eos_token_id=c.get("eos_token_id", 2))
    if rp["rope_type"] == "longrope":
        cfg.original_max_position_embeddings = rp["original_max_position_embeddings"]
    scale_emb = float(c.get("scale_emb", 1.0))
    resid = float(c.get("scale_depth", 1.0)) / math.sqrt(L)
    logit = float(c.get("dim_model_base", H)) / float(H)
    qk = nope + rope_d
    kv_rank = c["kv_lora_rank"]

    def convert(state):
        out = {}
        emb = state["model.embed_tokens.weight"]
        head = state.get("lm_head.weight", emb)                       # tied in the released checkpoints
        for k, v in state.items():
            if k.endswith("rotary_emb.inv_freq") or k == "lm_head.weight":
                continue
            if k.endswith("self_attn.q_b_proj.weight") or k.endswith("self_attn.q_proj.weight"):
                for h in range(nh):
                    v = _interleave_rows(v, h * qk + nope, rope_d)
            elif k.endswith("self_attn.kv_a_proj_with_mqa.weight"):
                v = _interleave_rows(v, kv_rank, rope_d)
            elif k.endswith("self_attn.o_proj.weight") or k.endswith("mlp.down_proj.weight"):
                v = (v.float() * resid).to(v.dtype)
            elif k == "model.embed_tokens.weight":
                v = (v.float() * scale_emb).to(v.dtype)
            out[k] = v
        out["lm_head.weight"] = (head.float() * logit).to(head.dtype)
        return out
    return cfg, convert


REMOTE_ARCHS: Dict[str, Callable[[dict], Optional[Tuple[object, Callable]]]] = {
    "chatglm": _chatglm, "baichuan": _baichuan, "internlm": _internlm, "internlm2": _internlm2, "qwen": _qwen,
    "minicpm": _minicpm, "minicpm3": _minicpm3, "aquila": _aquila,
}


def maybe_load_remote_arch(path, torch_dtype=None):
    """A natively built model for a checkpoint directory of one of ``REMOTE_ARCHS``, else ``None``.  The returned
    model's ``config.ipex_remote_model_type`` names the family the checkpoint came from."""
    if not isinstance(path, (str, os.PathLike)) or not os.path.isfile(os.path.join(path, "config.json")):
        return None
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    mt = c.get("model_type")
    if mt not in REMOTE_ARCHS:
        return None
    from transformers import AutoModelForCausalLM
    from transformers.models.auto.configuration_auto import CONFIG_MAPPING
    if mt in CONFIG_MAPPING:
        return None                     # this transformers version knows the family itself
    made = REMOTE_ARCHS[mt](c)
    if made is None:
        return None
    cfg, convert = made
    state = convert(_read_state_dict(str(path)))
    dtype = torch_dtype if isinstance(torch_dtype, torch.dtype) else None
    if dtype is None:
        name = c.get("torch_dtype") or c.get("dtype")
        dtype = getattr(torch, name) if isinstance(name, str) and hasattr(torch, name) else torch.float32
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(cfg, dtype=dtype)
    missing, unexpected = model.load_state_dict({k: v.to(dtype) if v.is_floating_point() else v
                                                 for k, v in state.items()}, strict=False, assign=True)
    missing = [m for m in missing if "rotary_emb" not in m]
    if missing or unexpected:
        raise RuntimeError(f"{mt} checkpoint does not match its native architecture: missing {missing[:5]}, "
                           f"unexpected {unexpected[:5]}")
    # buffers (rotary tables) were created on the meta device: rebuild them
    for mod in model.modules():
        if hasattr(mod, "inv_freq") and getattr(mod.inv_freq, "is_meta", False):
            fresh = type(mod)(config=cfg)
            mod.inv_freq = fresh.inv_freq
            if hasattr(mod, "original_inv_freq"):
                mod.original_inv_freq = fresh.inv_freq
    model.config.update({"ipex_remote_model_type": mt})
    if getattr(cfg, "ipex_alibi", False):
        # the native class would rotate q / k: a model with linear attention biases always runs the package's
        # attention forward, also when no low-bit conversion (and with it no forward replacement) was asked for
        from ..models.decoder import decoder_attention_forward
        from .convert import convert_forward
        convert_forward(model, "LlamaAttention", decoder_attention_forward)
    return model.eval()
