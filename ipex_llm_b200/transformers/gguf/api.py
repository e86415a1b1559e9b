"""``load_gguf_model``: build a low-bit model (and a tokenizer) straight from a ``.gguf`` file.

Counterpart of python/llm/src/ipex_llm/transformers/gguf/api.py:30-75 and the per-family loaders under
``gguf/models/`` (llama, mistral, mixtral, baichuan, bloom, falcon, mpt, yuan2).  One table-driven loader covers the
llama-shaped families (llama, mistral, mixtral, qwen2, qwen3, gemma, gemma2, phi3, baichuan, yuan2's llama base): the
GGUF tensor names are mapped to Hugging Face module names, the conventions of llama.cpp's exporter are undone (q / k
rows re-ordered for the llama-type architectures, Gemma norm weights stored as 1 + w), every matrix is re-quantized to ``low_bit`` as it is read, and nothing of the model is ever held in
full precision beyond one tensor.
"""
from __future__ import annotations

import re
from typing import Optional

import torch

from ...utils.common import invalidInputError

# GGUF file_type -> the qtype the file was exported with (informational; tensors are decoded individually)
qtype_map = {2: "sym_int4", 3: "asym_int4", 7: "sym_int8", 8: "sym_int5", 9: "asym_int5", 0: "fp32", 1: "fp16",
             15: "q4_k", 17: "q5_k", 18: "q6_k", 10: "q2_k"}

_LLAMA_LIKE = ("llama", "mistral", "mixtral", "qwen2", "qwen3", "gemma", "gemma2", "phi3", "baichuan", "yuan")
# llama.cpp's exporter re-orders the q / k rows of these architectures for its interleaved rotary kernel; the others
# (qwen2, qwen3, gemma, gemma2, phi3: "neox" rotary there) keep the Hugging Face row order
_PERMUTED_QK = ("llama", "mistral", "mixtral", "baichuan", "yuan")
# its Gemma exporter stores norm weights as (1 + w), because its RMSNorm multiplies by the stored value
_NORM_PLUS_ONE = ("gemma", "gemma2")

_BLOCK_MAP = {
    "attn_norm.weight": "input_layernorm.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_q.bias": "self_attn.q_proj.bias",
    "attn_k.weight": "self_attn.k_proj.weight", "attn_k.bias": "self_attn.k_proj.bias",
    "attn_v.weight": "self_attn.v_proj.weight", "attn_v.bias": "self_attn.v_proj.bias",
    "attn_output.weight": "self_attn.o_proj.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
    "ffn_gate_inp.weight": "block_sparse_moe.gate.weight",
    "attn_q_norm.weight": "self_attn.q_norm.weight", "attn_k_norm.weight": "self_attn.k_norm.weight",      # qwen3
    "attn_qkv.weight": "self_attn.qkv_proj.weight",                                                        # phi3
}
# per-architecture differences from the table above
_BLOCK_MAP_ARCH = {
    # four norms per layer: around attention and around the MLP
    "gemma2": {"post_attention_norm.weight": "post_attention_layernorm.weight",
               "ffn_norm.weight": "pre_feedforward_layernorm.weight",
               "post_ffw_norm.weight": "post_feedforward_layernorm.weight"},
    # gate and up projections fused in one matrix, stored under the "up" name
    "phi3": {"ffn_up.weight": "mlp.gate_up_proj.weight"},
}


def get_llama_module_name(name: str, arch: str = "llama") -> Optional[str]:
    """GGUF tensor name -> Hugging Face parameter name (None for tensors that have no counterpart)."""
    if name == "token_embd.weight":
        return "model.embed_tokens.weight"
    if name == "output_norm.weight":
        return "model.norm.weight"
    if name == "output.weight":
        return "lm_head.weight"
    m = re.match(r"blk\.(\d+)\.(.+)", name)
    if not m:
        return None
    layer, rest = m.group(1), m.group(2)
    if rest in _BLOCK_MAP_ARCH.get(arch, {}):
        return f"model.layers.{layer}.{_BLOCK_MAP_ARCH[arch][rest]}"
    if rest in _BLOCK_MAP:
        return f"model.layers.{layer}.{_BLOCK_MAP[rest]}"
    e = re.match(r"ffn_(gate|up|down)\.(\d+)\.weight", rest)     # mixtral experts stored one by one
    if e:
        w = {"gate": "w1", "down": "w2", "up": "w3"}[e.group(1)]
        return f"model.layers.{layer}.block_sparse_moe.experts.{e.group(2)}.{w}.weight"
    return None


def _unpermute(t: torch.Tensor, n_head: int) -> torch.Tensor:
    """Undo llama.cpp's q/k row permutation (pairs interleaved for its rotary kernel)."""
    rows = t.shape[0]
    return t.reshape(n_head, rows // n_head // 2, 2, *t.shape[1:]).swapaxes(1, 2).reshape(t.shape)


def _hf_config(cfg: dict, arch: str, vocab: int):
    import transformers
    g = lambda k, d=None: cfg.get(f"{arch}.{k}", d)  # noqa: E731
    common = dict(vocab_size=vocab, hidden_size=g("embedding_length"), intermediate_size=g("feed_forward_length"),
                  num_hidden_layers=g("block_count"), num_attention_heads=g("attention.head_count"),
                  num_key_value_heads=g("attention.head_count_kv", g("attention.head_count")),
                  max_position_embeddings=g("context_length", 4096),
                  rms_norm_eps=g("attention.layer_norm_rms_epsilon", 1e-5),
                  bos_token_id=cfg.get("tokenizer.ggml.bos_token_id"), eos_token_id=cfg.get("tokenizer.ggml.eos_token_id"),
                  tie_word_embeddings=False, use_cache=True)
    rope = g("rope.freq_base")
    if rope:
        common["rope_theta"] = float(rope)
    # long-context variants: linear position interpolation or YaRN, as llama.cpp records them
    scaling, factor = g("rope.scaling.type"), g("rope.scaling.factor")
    if scaling in ("linear", "yarn") and factor and float(factor) != 1.0:
        rp = {"rope_type": scaling, "factor": float(factor), "rope_theta": float(rope or 10000.0)}
        if scaling == "yarn" and g("rope.scaling.original_context_length"):
            rp["original_max_position_embeddings"] = int(g("rope.scaling.original_context_length"))
        common["rope_parameters"] = rp
        common.pop("rope_theta", None)
    name = str(cfg.get("general.name", "")).lower()
    if arch == "qwen2":
        return transformers.Qwen2Config(**common), "qwen2"
    if arch == "qwen3":
        common["head_dim"] = g("attention.key_length", common["hidden_size"] // common["num_attention_heads"])
        return transformers.Qwen3Config(**common), "qwen3"
    if arch == "gemma":
        common["head_dim"] = g("attention.key_length", common["hidden_size"] // common["num_attention_heads"])
        return transformers.GemmaConfig(**common), "gemma"
    if arch == "gemma2":
        common["head_dim"] = g("attention.key_length", common["hidden_size"] // common["num_attention_heads"])
        extra = dict(attn_logit_softcapping=g("attn_logit_softcapping", 50.0),
                     final_logit_softcapping=g("final_logit_softcapping", 30.0),
                     sliding_window=g("attention.sliding_window", 4096),
                     query_pre_attn_scalar=common["head_dim"])
        return transformers.Gemma2Config(**common, **extra), "gemma2"
    if arch == "phi3":
        if g("attention.sliding_window"):
            common["sliding_window"] = g("attention.sliding_window")
        common["pad_token_id"] = cfg.get("tokenizer.ggml.padding_token_id", 0)
        return transformers.Phi3Config(**common), "phi3"
    if g("expert_count"):
        return transformers.MixtralConfig(num_local_experts=g("expert_count"),
                                          num_experts_per_tok=g("expert_used_count", 2), **common), "mixtral"
    if "mistral" in name:
        return transformers.MistralConfig(**common), "mistral"
    return transformers.LlamaConfig(**common), "llama"


# ---------------------------------------------------------------------------------------------------------------
# LayerNorm / fused-qkv families (reference gguf/models/bloom.py, falcon.py, mpt.py)
# ---------------------------------------------------------------------------------------------------------------
_GPT_LIKE = ("bloom", "falcon", "mpt")

_GPT_TOP = {
    "bloom": {"token_embd": "transformer.word_embeddings", "token_embd_norm": "transformer.word_embeddings_layernorm",
              "output_norm": "transformer.ln_f", "output": "lm_head"},
    "falcon": {"token_embd": "transformer.word_embeddings", "output_norm": "transformer.ln_f", "output": "lm_head"},
    "mpt": {"token_embd": "transformer.wte", "output_norm": "transformer.norm_f", "output": "lm_head"},
}
_GPT_BLOCK = {
    "bloom": ("transformer.h", {"attn_norm": "input_layernorm", "attn_qkv": "self_attention.query_key_value",
                                "attn_output": "self_attention.dense", "ffn_norm": "post_attention_layernorm",
                                "ffn_up": "mlp.dense_h_to_4h", "ffn_down": "mlp.dense_4h_to_h"}),
    # new_decoder_architecture (40B-style) files carry two norms: attn_norm is ln_mlp there and attn_norm_2 ln_attn
    "falcon": ("transformer.h", {"attn_norm": "input_layernorm", "attn_norm_2": "ln_attn",
                                 "attn_qkv": "self_attention.query_key_value", "attn_output": "self_attention.dense",
                                 "ffn_up": "mlp.dense_h_to_4h", "ffn_down": "mlp.dense_4h_to_h"}),
    "mpt": ("transformer.blocks", {"attn_norm": "norm_1", "attn_qkv": "attn.Wqkv", "attn_output": "attn.out_proj",
                                   "ffn_norm": "norm_2", "ffn_up": "ffn.up_proj", "ffn_down": "ffn.down_proj"}),
}


def get_gpt_module_name(arch: str, name: str, new_decoder_architecture: bool = False) -> Optional[str]:
    """GGUF tensor name -> Hugging Face parameter name for bloom / falcon / mpt."""
    stem, _, kind = name.rpartition(".")           # "...weight" / "...bias"
    if stem in _GPT_TOP[arch]:
        return f"{_GPT_TOP[arch][stem]}.{kind}"
    m = re.match(r"blk\.(\d+)\.(.+)", stem)
    if not m:
        return None
    prefix, table = _GPT_BLOCK[arch]
    sub = table.get(m.group(2))
    if sub is None:
        return None
    if arch == "falcon" and new_decoder_architecture and m.group(2) == "attn_norm":
        sub = "ln_mlp"
    return f"{prefix}.{m.group(1)}.{sub}.{kind}"


def _qkv_to_hf(arch: str, t: torch.Tensor, n_head: int, n_kv: int) -> torch.Tensor:
    """llama.cpp stores fused qkv as ``[all Q; all K; all V]``; bloom and falcon checkpoints interleave them per
    (kv) head: ``[n_kv, q heads of the group + k + v, head_dim, ...]``.  MPT already is ``[Q; K; V]``."""
    if arch == "mpt":
        return t
    rest = t.shape[1:]
    hd = t.shape[0] // (n_head + 2 * n_kv)
    q, k, v = t.split([n_head * hd, n_kv * hd, n_kv * hd], dim=0)
    q = q.reshape(n_kv, n_head // n_kv, hd, *rest)
    k = k.reshape(n_kv, 1, hd, *rest)
    v = v.reshape(n_kv, 1, hd, *rest)
    return torch.cat([q, k, v], dim=1).reshape(t.shape)


def _gpt_like_config(cfg: dict, arch: str, vocab: int):
    import transformers
    g = lambda k, d=None: cfg.get(f"{arch}.{k}", d)  # noqa: E731
    E, L, Hn = g("embedding_length"), g("block_count"), g("attention.head_count")
    eps = g("attention.layer_norm_epsilon", 1e-5)
    tok = dict(bos_token_id=cfg.get("tokenizer.ggml.bos_token_id"), eos_token_id=cfg.get("tokenizer.ggml.eos_token_id"))
    if arch == "bloom":
        return transformers.BloomConfig(vocab_size=vocab, hidden_size=E, n_layer=L, n_head=Hn,
                                        layer_norm_epsilon=eps, **tok), Hn, Hn
    if arch == "falcon":
        n_kv = g("attention.head_count_kv", 1) or 1
        new_arch = 1 < n_kv < Hn
        return transformers.FalconConfig(vocab_size=vocab, hidden_size=E, num_hidden_layers=L, num_attention_heads=Hn,
                                         num_kv_heads=n_kv, new_decoder_architecture=new_arch,
                                         multi_query=n_kv == 1, parallel_attn=True, bias=False, alibi=False,
                                         layer_norm_epsilon=eps, **tok), Hn, n_kv
    ffn = g("feed_forward_length", 4 * E)
    attn_cfg = {"alibi": True, "alibi_bias_max": int(g("attention.max_alibi_bias", 8) or 8)}
    clip = g("attention.clamp_kqv")
    if clip:
        attn_cfg["clip_qkv"] = float(clip)
    return transformers.MptConfig(vocab_size=vocab, d_model=E, n_layers=L, n_heads=Hn, expansion_ratio=ffn // E,
                                  max_seq_len=g("context_length", 2048), no_bias=True, layer_norm_epsilon=eps,
                                  attn_config=attn_cfg, **tok), Hn, Hn


class GGUFTokenizer:
    """Minimal tokenizer over the vocabulary stored in the file (sentencepiece pieces rebuilt into a processor)."""

    def __init__(self, loader):
        import sentencepiece as spm
        from transformers.convert_slow_tokenizer import import_protobuf
        spm_pb2 = import_protobuf("Failed to import protobuf")
        trainer = spm_pb2.TrainerSpec(byte_fallback=True, model_type=spm_pb2.TrainerSpec.ModelType.BPE)
        proto = spm_pb2.ModelProto(pieces=loader.tokenizer_pieces(), trainer_spec=trainer)
        self.sp = spm.SentencePieceProcessor(model_proto=proto.SerializeToString())
        self.bos_token_id = loader.config.get("tokenizer.ggml.bos_token_id")
        self.eos_token_id = loader.config.get("tokenizer.ggml.eos_token_id")
        self.pad_token_id = loader.config.get("tokenizer.ggml.padding_token_id", self.eos_token_id)
        self.padding_side = "left"
        self.vocab_size = self.sp.get_piece_size()

    def encode(self, text, add_special_tokens=True):
        ids = self.sp.encode(text)
        return ([self.bos_token_id] if add_special_tokens and self.bos_token_id is not None else []) + ids

    def decode(self, ids, skip_special_tokens=True, **kw):
        ids = [int(i) for i in (ids.tolist() if hasattr(ids, "tolist") else ids)]
        if skip_special_tokens:
            ids = [i for i in ids if i not in (self.bos_token_id, self.eos_token_id, self.pad_token_id)]
        return self.sp.decode(ids)

    def __call__(self, text, return_tensors=None, padding=False, **kw):
        batch = [text] if isinstance(text, str) else list(text)
        enc = [self.encode(t) for t in batch]
        n = max(len(e) for e in enc)
        pad = self.pad_token_id if self.pad_token_id is not None else 0
        ids = [[pad] * (n - len(e)) + e for e in enc]
        mask = [[0] * (n - len(e)) + [1] * len(e) for e in enc]
        if return_tensors == "pt":
            return {"input_ids": torch.tensor(ids), "attention_mask": torch.tensor(mask)}
        return {"input_ids": ids if not isinstance(text, str) else ids[0],
                "attention_mask": mask if not isinstance(text, str) else mask[0]}


# split patterns of the byte-level BPE vocabularies llama.cpp names in ``tokenizer.ggml.pre`` (they are part of each
# model's published tokenizer definition); anything else falls back to the GPT-2 pattern
_BPE_SPLIT = {
    "llama-bpe": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
                 r"|\s+(?!\S)|\s+",
    "qwen2": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
             r"|\s+(?!\S)|\s+",
}


def build_bpe_tokenizer(cfg: dict):
    """Byte-level BPE tokenizer (``tokenizer.ggml.model == "gpt2"``: Llama-3, Qwen2, GPT-2, Falcon, ...) rebuilt from the
    vocabulary and merge list of the file as a ``PreTrainedTokenizerFast``."""
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    tokens = cfg["tokenizer.ggml.tokens"]
    merges = [tuple(m.split(" ", 1)) for m in cfg.get("tokenizer.ggml.merges", [])]
    tk = Tokenizer(models.BPE(vocab={t: i for i, t in enumerate(tokens)}, merges=merges, fuse_unk=False,
                              byte_fallback=False))
    pattern = _BPE_SPLIT.get(str(cfg.get("tokenizer.ggml.pre", "")))
    if pattern is None:
        tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        tk.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(pattern), behavior="isolated"),
            pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tk.decoder = decoders.ByteLevel()
    types = cfg.get("tokenizer.ggml.token_type") or []
    special = [tokens[i] for i, ty in enumerate(types) if ty in (3, 4)]          # control / user-defined tokens
    if special:
        tk.add_special_tokens(special)

    def tok(key):
        i = cfg.get(key)
        return tokens[i] if isinstance(i, int) and 0 <= i < len(tokens) else None
    fast = PreTrainedTokenizerFast(tokenizer_object=tk, bos_token=tok("tokenizer.ggml.bos_token_id"),
                                   eos_token=tok("tokenizer.ggml.eos_token_id"),
                                   pad_token=tok("tokenizer.ggml.padding_token_id") or tok("tokenizer.ggml.eos_token_id"))
    fast.padding_side = "left"
    template = cfg.get("tokenizer.chat_template")
    if template:
        fast.chat_template = template
    return fast


def load_gguf_model(fpath: str, dtype: torch.dtype = torch.float, low_bit: str = "sym_int4"):
    """Returns ``(model, tokenizer)``; ``model`` is a low-bit model ready for ``.to('cuda')`` / ``generate``."""
    from ..convert import ggml_convert_low_bit
    from ..model import _attach_api
    from ...quant import qtypes as qt
    from .gguf import GGUFFileLoader
    import transformers

    loader = GGUFFileLoader(fpath)
    cfg = loader.config
    arch = cfg.get("general.architecture")
    print("model_family:" + str(arch))
    invalidInputError(arch in _LLAMA_LIKE or arch in _GPT_LIKE, f"Unsupported model family: {arch}")
    vocab = len(cfg["tokenizer.ggml.tokens"]) if "tokenizer.ggml.tokens" in cfg else None
    names = loader.tensor_loader.names()
    if vocab is None:
        vocab = loader.tensor_loader.infos[names.index("token_embd.weight")][1][1]
    gpt_like = arch in _GPT_LIKE
    if gpt_like:
        hf_cfg, n_head, n_kv = _gpt_like_config(cfg, arch, vocab)
    else:
        hf_cfg, family = _hf_config(cfg, arch, vocab)
        n_head, n_kv = hf_cfg.num_attention_heads, hf_cfg.num_key_value_heads
    hf_cfg.tie_word_embeddings = "output.weight" not in names

    try:
        from transformers.initialization import no_init_weights
    except ImportError:  # older layouts
        from transformers.modeling_utils import no_init_weights
    with no_init_weights(), torch.device("meta"):
        model = transformers.AutoModelForCausalLM.from_config(hf_cfg, dtype=dtype)
    model.to_empty(device="cpu")
    params = dict(model.named_parameters())
    loaded = set()

    new_arch = bool(getattr(hf_cfg, "new_decoder_architecture", False))

    rope_factors = []

    def process(name, tensor):
        if name == "rope_freqs.weight":
            # Llama-3.1 style long-context scaling: llama.cpp stores the per-frequency divisors as a tensor
            rope_factors.append(tensor.float().reshape(-1))
            return
        if gpt_like:
            target = get_gpt_module_name(arch, name, new_arch)
            if target is None or target not in params:
                return
            if ".attn_qkv." in name:
                tensor = _qkv_to_hf(arch, tensor, n_head, n_kv)
            with torch.no_grad():
                params[target].copy_(tensor.to(params[target].dtype).reshape(params[target].shape))
            loaded.add(target)
            return
        target = get_llama_module_name(name, arch)
        if target is None or target not in params:
            return
        if arch in _PERMUTED_QK:
            if target.endswith("q_proj.weight") or target.endswith("q_proj.bias"):
                tensor = _unpermute(tensor, n_head)
            elif target.endswith("k_proj.weight") or target.endswith("k_proj.bias"):
                tensor = _unpermute(tensor, n_kv)
        if arch in _NORM_PLUS_ONE and target.endswith("norm.weight"):
            tensor = tensor - 1.0
        with torch.no_grad():
            params[target].copy_(tensor.to(params[target].dtype).reshape(params[target].shape))
        loaded.add(target)

    loader.tensor_loader.load_while_process(process)
    missing = [n for n in params if n not in loaded and not (hf_cfg.tie_word_embeddings and n == "lm_head.weight")]
    invalidInputError(not missing, f"GGUF file lacks tensors for: {missing[:5]}{' ...' if len(missing) > 5 else ''}")
    if hf_cfg.tie_word_embeddings:
        model.tie_weights()
    # buffers created on meta (rotary tables) are rebuilt by re-instantiating them
    from ..model import _rebuild_nonpersistent
    _rebuild_nonpersistent(model)
    if rope_factors:
        for mod in model.modules():
            inv = getattr(mod, "inv_freq", None)
            if inv is not None and inv.numel() == rope_factors[0].numel():
                mod.inv_freq = inv / rope_factors[0].to(inv.device)
                if hasattr(mod, "original_inv_freq"):
                    mod.original_inv_freq = mod.inv_freq.clone()
    model = ggml_convert_low_bit(model.eval(), qt.qtype_from_name(low_bit), optimize_model=True)
    model = _attach_api(model, low_bit)
    try:
        if "tokenizer.ggml.tokens" not in cfg:
            tokenizer = None
        elif cfg.get("tokenizer.ggml.model") == "gpt2":
            tokenizer = build_bpe_tokenizer(cfg)
        else:
            tokenizer = GGUFTokenizer(loader)
    except Exception:  # noqa: BLE001 - a vocabulary kind that cannot be rebuilt here: model only
        tokenizer = None
    loader.close()
    return model, tokenizer
