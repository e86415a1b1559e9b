"""Family registry: which weight surgery and which forward replacements each ``model_type`` gets.

Replaces the per-``model_type`` if/elif chains of the reference's ``_optimize_pre`` / ``_optimize_post``
(python/llm/src/ipex_llm/transformers/convert.py:886-1076, 1253-2042).  Classes are named by string so that no
modeling module is imported until a model of that family is converted.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

from . import common as C
from . import decoder as D
from . import phi3 as P3
from . import rwkv as R


@dataclass
class Family:
    pre: List[Callable] = field(default_factory=list)              # fn(module, config), applied with model.apply
    post: List[Tuple[str, Callable]] = field(default_factory=list)  # (class name, new forward)
    attrs: List[Tuple[str, str, object]] = field(default_factory=list)  # (class name, attribute, value)
    post_hook: Optional[Callable] = None
    engine: Optional[str] = None                                   # native decode-engine flavour, if any


def _merge_qkv(attn_cls):
    def fn(module, config):
        C.merge_qkv_base(module, attn_cls)
    return fn


def _split_fused_gate_up(mlp_cls):
    """Families whose checkpoint already fuses gate/up in one Linear keep it; nothing to split on B200
    (the reference splits Phi-3's ``gate_up_proj`` for its decode kernel, convert.py:947-951)."""
    def fn(module, config):
        return None
    return fn


def _llama_like(prefix, mlp_forward=C.mlp_silu_forward, norm_forward=C.rms_norm_forward, spec=None, engine=None,
                extra_post=(), merge=True, post_hook=None):
    attrs = []
    if spec is not None:
        attrs.append((f"{prefix}Attention", "_ipex_attn", spec))
    return Family(
        pre=[_merge_qkv(f"{prefix}Attention")] if merge else [],
        post=[(f"{prefix}RMSNorm", norm_forward), (f"{prefix}MLP", mlp_forward),
              (f"{prefix}Attention", D.decoder_attention_forward), (f"{prefix}Model", D.decoder_model_forward),
              *extra_post],
        attrs=attrs,
        engine=engine,
        post_hook=post_hook,
    )


def _moe_block_forward(self, hidden_states):
    """Sparse-MoE block on the transformers-5 layout (router ``gate`` + fused ``experts``): routing through the
    fused router kernel, experts through ``LowBitExperts``."""
    from ..ops.moe import softmax_topk_router
    import torch.nn.functional as F
    bsz, seq, hid = hidden_states.shape
    x = hidden_states.reshape(-1, hid)
    gate = self.gate
    logits = F.linear(x.to(gate.weight.dtype), gate.weight)     # (a disk-resident embedding hands out fp16 rows)
    top_k = getattr(gate, "top_k", None) or getattr(self, "top_k", 2)
    renorm = getattr(gate, "norm_topk_prob", True)
    _, w, idx = softmax_topk_router(logits, top_k, renorm)
    out = self.experts(x, idx, w.to(x.dtype))
    shared = getattr(self, "shared_expert", None)
    if shared is not None:
        s = shared(x)
        sg = getattr(self, "shared_expert_gate", None)
        if sg is not None:
            import torch
            s = torch.sigmoid(sg(x)) * s
        out = out + s
    # (under tensor parallelism the bank sums its partial outputs over the group itself, see parallel/tp.py)
    return out.reshape(bsz, seq, hid)


def _deepseek_v3_route(self, router_logits):
    """``DeepseekV3MoE.route_tokens_to_experts`` through the grouped top-k router (one kernel on the GPU; reference
    models/deepseek.py:283-287 calls ``xe_addons.moe_group_topk`` at the same place)."""
    from ..ops.moe import moe_group_topk
    idx, w = moe_group_topk(router_logits, self.gate.e_score_correction_bias, self.n_group, self.topk_group,
                            self.top_k, bool(self.norm_topk_prob), float(self.routed_scaling_factor))
    return idx, w


def _deepseek_v3_hook(model):
    from ..transformers.convert import replace_func
    replace_func(model, "DeepseekV3MoE", "route_tokens_to_experts", _deepseek_v3_route)
    return model


FAMILIES = {
    "llama": _llama_like("Llama", engine="llama"),
    "mistral": _llama_like("Mistral", engine="llama"),
    "mixtral": _llama_like("Mixtral", engine="mixtral",
                           extra_post=[("MixtralSparseMoeBlock", _moe_block_forward)]),
    "qwen2": _llama_like("Qwen2", engine="llama"),
    "qwen2_moe": _llama_like("Qwen2Moe", extra_post=[("Qwen2MoeSparseMoeBlock", _moe_block_forward)]),
    "qwen3": _llama_like("Qwen3", spec=D.AttnSpec(qk_norm=True, sliding=True)),
    "qwen3_moe": _llama_like("Qwen3Moe", spec=D.AttnSpec(qk_norm=True, sliding=True),
                             extra_post=[("Qwen3MoeSparseMoeBlock", _moe_block_forward)]),
    "gemma": _llama_like("Gemma", mlp_forward=C.mlp_gelu_forward, norm_forward=C.gemma_rms_norm_forward),
    "gemma2": _llama_like("Gemma2", mlp_forward=C.mlp_gelu_forward, norm_forward=C.gemma_rms_norm_forward,
                          spec=D.AttnSpec(softcap_attr="attn_logit_softcapping", sliding=True)),
    "phi3": _llama_like("Phi3", merge=False, post_hook=P3.install),
    # GLM: GPT-J style ("two") rotary on half of the head dims, fused gate_up_proj (reference models/glm.py,
    # chatglm2.py:225-262 for the rotary pairing)
    "glm": _llama_like("Glm", spec=D.AttnSpec(interleaved_rope=True)),
    "glm4": _llama_like("Glm4", spec=D.AttnSpec(interleaved_rope=True)),
    "starcoder2": Family(pre=[_merge_qkv("Starcoder2Attention")],
                         post=[("Starcoder2Attention", D.decoder_attention_forward),
                               ("Starcoder2Model", D.decoder_model_forward)]),
    "stablelm": Family(post=[("StableLmModel", D.decoder_model_forward)]),
    # families that reach the package kernels through the attention interface (transformers/convert.py) plus the
    # norm / MLP replacements below; their attention modules keep their own projections and rotary handling
    "cohere": Family(post=[("CohereMLP", C.mlp_silu_forward)]),
    "gemma3_text": Family(post=[("Gemma3RMSNorm", C.gemma_rms_norm_forward), ("Gemma3MLP", C.mlp_gelu_forward)]),
    "gemma3": Family(post=[("Gemma3RMSNorm", C.gemma_rms_norm_forward), ("Gemma3MLP", C.mlp_gelu_forward)]),
    "olmo2": Family(post=[("Olmo2RMSNorm", C.rms_norm_forward), ("Olmo2MLP", C.mlp_silu_forward)]),
    "granite": Family(post=[("GraniteRMSNorm", C.rms_norm_forward), ("GraniteMLP", C.mlp_silu_forward)]),
    "qwen2_vl": Family(post=[("Qwen2VLRMSNorm", C.rms_norm_forward), ("Qwen2MLP", C.mlp_silu_forward)]),
    "gptj": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "yi": _llama_like("Llama", engine="llama"),
    "deci": _llama_like("Llama"),
    "internlm2": Family(post=[("InternLM2RMSNorm", C.rms_norm_forward)]),
    "baichuan": Family(post=[("RMSNorm", C.rms_norm_forward), ("MLP", C.mlp_silu_forward)]),
    "chatglm": Family(post=[("RMSNorm", C.rms_norm_forward)]),
    "minicpm": _llama_like("MiniCPM"),
    "aquila": Family(post=[("AquilaRMSNorm", C.rms_norm_forward)]),
    "deepseek_v3": Family(post=[("DeepseekV3RMSNorm", C.rms_norm_forward), ("DeepseekV3MLP", C.mlp_silu_forward)],
                          post_hook=_deepseek_v3_hook),
    # multi-head latent attention keeps its own projections (q_a / q_b, kv_a / kv_b) and reaches the package's SDPA
    # through the attention interface; experts are converted as a fused bank, the router stays in full precision
    "deepseek_v2": Family(post=[("DeepseekV2RMSNorm", C.rms_norm_forward), ("DeepseekV2MLP", C.mlp_silu_forward)],
                          post_hook=P3.install),      # MiniCPM3 checkpoints arrive here with LongRoPE factors
    "phimoe": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "mllama": Family(post=[("MllamaTextRMSNorm", C.rms_norm_forward), ("MllamaTextMLP", C.mlp_silu_forward)]),
    # encoder-decoder text models of the T5 line: their feed-forward casts activations to the weight's dtype
    **{mt: Family(post=[(f"{prefix}DenseActDense", C.t5_dense_forward),
                        (f"{prefix}DenseGatedActDense", C.t5_dense_forward)])
       for mt, prefix in (("t5", "T5"), ("mt5", "MT5"), ("umt5", "UMT5"))},
    "rwkv": Family(pre=[R.rescale_before_quantization],
                   post=[("RwkvSelfAttention", R.rwkv4_attention_forward), ("RwkvFeedForward", R.rwkv4_ffn_forward)]),
    # LayerNorm families without a dedicated forward file: low-bit linears + the fused LayerNorm kernel
    "gpt_neox": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "bloom": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "gpt2": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "gpt_bigcode": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "falcon": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "mpt": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "phi": Family(post=[("LayerNorm", C.layer_norm_forward)]),
    "opt": Family(post=[("LayerNorm", C.layer_norm_forward)]),
}


def family_for(model) -> Optional[Family]:
    cfg = getattr(model, "config", None)
    mt = getattr(cfg, "model_type", None)
    if mt is None:
        return None
    if mt == "phi-msft":
        mt = "phixtral"
    return FAMILIES.get(mt)


def register_family(model_type: str, family: Family):
    FAMILIES[model_type] = family
