"""GGUF import: write a tiny llama-shaped file (f32 / f16 / q8_0 / q4_0 tensors), read it back, compare with the
source model."""
import os

import numpy as np
import pytest
import torch


def _export(model, cfg, path, wtype):
    from ipex_llm_b200.transformers.gguf.gguf import write_gguf
    n_head, n_kv = cfg.num_attention_heads, cfg.num_key_value_heads

    def permute(t, heads):      # llama.cpp's export permutation of q/k rows
        rows = t.shape[0]
        return t.reshape(heads, 2, rows // heads // 2, *t.shape[1:]).swapaxes(1, 2).reshape(t.shape)
    sd = model.state_dict()
    tensors = {"token_embd.weight": (sd["model.embed_tokens.weight"], "f16"),
               "output_norm.weight": (sd["model.norm.weight"], "f32"),
               "output.weight": (sd["lm_head.weight"], wtype)}
    names = {"input_layernorm.weight": ("attn_norm.weight", "f32"),
             "post_attention_layernorm.weight": ("ffn_norm.weight", "f32"),
             "self_attn.q_proj.weight": ("attn_q.weight", wtype), "self_attn.k_proj.weight": ("attn_k.weight", wtype),
             "self_attn.v_proj.weight": ("attn_v.weight", wtype), "self_attn.o_proj.weight": ("attn_output.weight", wtype),
             "mlp.gate_proj.weight": ("ffn_gate.weight", wtype), "mlp.up_proj.weight": ("ffn_up.weight", wtype),
             "mlp.down_proj.weight": ("ffn_down.weight", wtype)}
    for i in range(cfg.num_hidden_layers):
        for hf, (gg, ty) in names.items():
            t = sd[f"model.layers.{i}.{hf}"]
            if "q_proj" in hf:
                t = permute(t, n_head)
            elif "k_proj" in hf:
                t = permute(t, n_kv)
            tensors[f"blk.{i}.{gg}"] = (t, ty)
    meta = {"general.architecture": "llama", "general.name": "tiny-llama", "general.file_type": 7,
            "llama.embedding_length": cfg.hidden_size, "llama.feed_forward_length": cfg.intermediate_size,
            "llama.block_count": cfg.num_hidden_layers, "llama.attention.head_count": n_head,
            "llama.attention.head_count_kv": n_kv, "llama.context_length": 256,
            "llama.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), "llama.rope.freq_base": 10000.0,
            "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2}
    write_gguf(path, meta, tensors)


def test_block_codecs_roundtrip():
    from ipex_llm_b200.transformers.gguf.gguf import _NAME_TO_TYPE, dequantize_blocks, quantize_blocks
    rng = np.random.default_rng(0)
    x = rng.standard_normal(32 * 40).astype(np.float32)
    for name, tol in (("f32", 0), ("f16", 1e-3), ("q8_0", 0.02), ("q4_0", 0.3)):
        raw = np.frombuffer(quantize_blocks(x, name), dtype=np.uint8)
        y = dequantize_blocks(raw, _NAME_TO_TYPE[name], x.size)
        assert np.abs(x - y).max() <= tol * max(1.0, np.abs(x).max()) + 1e-12, name


def test_superblock_tensor_types_read_back(tmp_path):
    """k-quant and code-book tensors in a GGUF file decode through the reader (type ids 10-14, 16, 17, 19, 29)."""
    pytest.importorskip("gguf.quants")
    from ipex_llm_b200.transformers.gguf.gguf import GGUFFileLoader, write_gguf
    torch.manual_seed(0)
    w = torch.randn(8, 512)
    kinds = {"q4_k": 0.12, "q6_k": 0.03, "iq2_xxs": 0.4, "iq2_xs": 0.35, "iq1_s": 0.5, "iq1_m": 0.5}
    path = str(tmp_path / "t.gguf")
    write_gguf(path, {"general.architecture": "llama"}, {f"w.{k}": (w, k) for k in kinds})
    loader = GGUFFileLoader(path)
    got = dict(loader.tensors())
    for k, tol in kinds.items():
        y = got[f"w.{k}"]
        assert y.shape == w.shape and ((y - w).norm() / w.norm()).item() < tol, k
    loader.close()


def test_native_quantize_executable_rewrites_a_gguf_file(tmp_path):
    """``ipex-quantize`` (C++): metadata kept, matrices with rows of a multiple of 256 packed to the k-quant asked for
    (``output.weight`` to q6_k), small and kept tensors copied; the result reads back through the GGUF reader."""
    from ipex_llm_b200.ggml.quantize import quantize, quantize_gguf
    from ipex_llm_b200.transformers.gguf.gguf import GGUFFileLoader, write_gguf
    torch.manual_seed(0)
    tensors = {"blk.0.attn_q.weight": (torch.randn(64, 512), "f32"), "blk.0.ffn_down.weight": (torch.randn(32, 256), "f16"),
               "blk.0.attn_norm.weight": (torch.randn(512), "f32"), "output.weight": (torch.randn(40, 512), "f32"),
               "blk.0.odd.weight": (torch.randn(8, 96), "f32"), "blk.0.keepme.weight": (torch.randn(4, 256), "f32")}
    src, dst = str(tmp_path / "in.gguf"), str(tmp_path / "out.gguf")
    write_gguf(src, {"general.architecture": "llama", "llama.block_count": 1, "tokenizer.ggml.tokens": ["a", "b"]}, tensors)
    quantize_gguf(src, dst, "q4_k", keep=["keepme"])
    loader = GGUFFileLoader(dst)
    assert loader.config["general.architecture"] == "llama" and loader.config["tokenizer.ggml.tokens"] == ["a", "b"]
    types = {name: t for name, _, t, _ in loader.tensor_loader.infos}
    assert types["blk.0.attn_q.weight"] == 12 and types["blk.0.ffn_down.weight"] == 12 and types["output.weight"] == 14
    assert types["blk.0.attn_norm.weight"] == 0 and types["blk.0.odd.weight"] == 0 and types["blk.0.keepme.weight"] == 0
    got = loader.tensors()
    for name, (t, kind) in tensors.items():
        ref = t.half().float() if kind == "f16" else t
        err = ((got[name] - ref).norm() / ref.norm()).item()
        assert got[name].shape == t.shape and err < (0.12 if types[name] in (12, 14) else 1e-6), (name, err)
    loader.close()
    assert os.path.getsize(dst) < 0.35 * os.path.getsize(src)
    # the Python entry point takes the same route for file-to-file k-quant requests
    dst2 = str(tmp_path / "out2.gguf")
    assert quantize(src, dst2, "llama", "q6_k") == dst2 and os.path.getsize(dst2) > os.path.getsize(dst)
    with pytest.raises(RuntimeError):
        quantize_gguf(str(tmp_path / "out.gguf"), str(tmp_path / "x.gguf"), "q9_k")
    # truncated and corrupt files end in an error message: no crash, no giant allocation, no endless loop
    import random
    import subprocess
    from ipex_llm_b200.native.build import build_tools
    data = open(src, "rb").read()
    rnd = random.Random(0)
    blobs = [data[:n] for n in (0, 3, 8, 24, 60, 150, len(data) // 2, len(data) - 10)]
    for _ in range(40):
        b = bytearray(data)
        for _ in range(rnd.randint(1, 4)):
            b[rnd.randrange(0, 300)] = rnd.randrange(256)
        blobs.append(bytes(b))
    bad = str(tmp_path / "bad.gguf")
    for blob in blobs:
        with open(bad, "wb") as f:
            f.write(blob)
        r = subprocess.run([build_tools(), bad, str(tmp_path / "o.gguf"), "q4_k"], capture_output=True, timeout=60)
        assert r.returncode in (0, 1), (r.returncode, r.stderr[-200:])


def test_load_gguf_llama(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM
    from ipex_llm.transformers import AutoModelForCausalLM
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=320, max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(0)
    src = LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in src.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
    path = str(tmp_path / "tiny.gguf")
    _export(src, cfg, path, "q8_0")
    model, tok = AutoModelForCausalLM.from_gguf(path, low_bit="sym_int8")
    assert tok is None                                   # the file carries no vocabulary
    ids = torch.randint(0, 320, (2, 10))
    with torch.no_grad():
        a = src(ids).logits[:, -1].float()
        b = model(ids).logits[:, -1].float()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.995, cos
    out = model.generate(ids, max_new_tokens=4, do_sample=False)
    assert out.shape == (2, 14)


def _qkv_to_gguf(t, n_head, n_kv):
    """Checkpoint layout [n_kv, q heads of the group + k + v, head_dim, ...] -> llama.cpp's [all Q; all K; all V]."""
    rest = t.shape[1:]
    hd = t.shape[0] // (n_head + 2 * n_kv)
    g = t.reshape(n_kv, n_head // n_kv + 2, hd, *rest)
    q = g[:, :-2].reshape(n_head * hd, *rest)
    k = g[:, -2].reshape(n_kv * hd, *rest)
    v = g[:, -1].reshape(n_kv * hd, *rest)
    return torch.cat([q, k, v], dim=0)


def _export_gpt_like(model, arch, path, n_head, n_kv, meta_extra):
    from ipex_llm_b200.transformers.gguf.api import _GPT_BLOCK, _GPT_TOP
    from ipex_llm_b200.transformers.gguf.gguf import write_gguf
    sd = model.state_dict()
    tensors = {}
    for gg, hf in _GPT_TOP[arch].items():
        for kind in ("weight", "bias"):
            key = f"{hf}.{kind}"
            if key in sd and not (gg == "output" and getattr(model.config, "tie_word_embeddings", False)):
                tensors[f"{gg}.{kind}"] = (sd[key], "f16" if sd[key].dim() > 1 else "f32")
    prefix, table = _GPT_BLOCK[arch]
    n_layers = len([k for k in sd if k.startswith(prefix + ".") and k.endswith(table["attn_qkv"] + ".weight")])
    for i in range(n_layers):
        for gg, hf in table.items():
            for kind in ("weight", "bias"):
                key = f"{prefix}.{i}.{hf}.{kind}"
                if key not in sd and arch == "falcon" and gg == "attn_norm":
                    key = f"{prefix}.{i}.ln_mlp.{kind}"          # two-norm (40B-style) blocks: attn_norm is ln_mlp
                if key not in sd:
                    continue
                t = sd[key]
                if gg == "attn_qkv" and arch != "mpt":
                    t = _qkv_to_gguf(t, n_head, n_kv)
                tensors[f"blk.{i}.{gg}.{kind}"] = (t, "q8_0" if t.dim() > 1 else "f32")
    meta = {"general.architecture": arch, "general.name": "tiny-" + arch, "general.file_type": 7,
            "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2}
    meta.update(meta_extra)
    write_gguf(path, meta, tensors)


def _randomize(model):
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
            else:
                p.add_(torch.randn_like(p) * 0.05)


import pytest


@pytest.mark.parametrize("arch", ["bloom", "falcon", "falcon-gqa", "mpt"])
def test_load_gguf_layernorm_families(tmp_path, arch):
    """bloom / falcon / mpt files: tensor-name maps, fused-qkv re-interleaving, configs rebuilt from the metadata."""
    import transformers as tf
    from ipex_llm.transformers import AutoModelForCausalLM
    torch.manual_seed(0)
    if arch == "bloom":
        cfg = tf.BloomConfig(hidden_size=128, n_layer=2, n_head=4, vocab_size=320, tie_word_embeddings=False)
        n_head = n_kv = 4
        meta = {"bloom.embedding_length": 128, "bloom.block_count": 2, "bloom.attention.head_count": 4,
                "bloom.attention.layer_norm_epsilon": float(cfg.layer_norm_epsilon), "bloom.context_length": 256}
    elif arch.startswith("falcon"):
        gqa = arch.endswith("gqa")
        n_head, n_kv = 4, (2 if gqa else 1)
        cfg = tf.FalconConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=320,
                              num_kv_heads=n_kv, new_decoder_architecture=gqa, multi_query=not gqa,
                              parallel_attn=True, bias=False, alibi=False, tie_word_embeddings=False)
        meta = {"falcon.embedding_length": 128, "falcon.block_count": 2, "falcon.attention.head_count": 4,
                "falcon.attention.head_count_kv": n_kv, "falcon.context_length": 256,
                "falcon.attention.layer_norm_epsilon": float(cfg.layer_norm_epsilon)}
    else:
        cfg = tf.MptConfig(d_model=128, n_layers=2, n_heads=4, vocab_size=320, max_seq_len=256, no_bias=True)
        n_head = n_kv = 4
        meta = {"mpt.embedding_length": 128, "mpt.block_count": 2, "mpt.attention.head_count": 4,
                "mpt.feed_forward_length": 512, "mpt.context_length": 256, "mpt.attention.max_alibi_bias": 8.0,
                "mpt.attention.layer_norm_epsilon": float(cfg.layer_norm_epsilon)}
    src = tf.AutoModelForCausalLM.from_config(cfg).eval()
    _randomize(src)
    file_arch = "falcon" if arch.startswith("falcon") else arch
    path = str(tmp_path / f"{arch}.gguf")
    _export_gpt_like(src, file_arch, path, n_head, n_kv, meta)
    model, tok = AutoModelForCausalLM.from_gguf(path, low_bit="sym_int8")
    assert tok is None
    assert model.config.model_type == file_arch
    ids = torch.randint(0, 320, (2, 10))
    with torch.no_grad():
        a = src(ids).logits[:, -1].float()
        b = model(ids).logits[:, -1].float()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.995, (arch, cos)
    out = model.generate(ids, max_new_tokens=3, do_sample=False)
    assert out.shape == (2, 13)


def test_interoperates_with_the_official_gguf_package(tmp_path):
    """Against the ``gguf`` Python package (the format's own reader / writer): k-quant bytes packed by the quant core
    decode identically through its decoder, and a file its writer produced (metadata incl. non-ASCII strings and
    arrays; f32, f16, bf16, q8_0, q4_0, q4_1, q5_0, q5_1 tensors) reads back exactly through this package's reader."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants as gq
    from gguf.constants import GGMLQuantizationType as T
    from ipex_llm_b200.quant import qtypes as qt
    from ipex_llm_b200.quant.params import ggml_convert_fp32, ggml_convert_qtype
    from ipex_llm_b200.transformers.gguf.gguf import GGUFFileLoader
    torch.manual_seed(0)
    w = torch.randn(16, 512)
    for name, t in (("q2_k", T.Q2_K), ("q4_k", T.Q4_K), ("q5_k", T.Q5_K), ("q6_k", T.Q6_K)):
        q = qt.qtype_from_name(name)
        p = ggml_convert_qtype(w, q)
        ours = ggml_convert_fp32(p, w.shape, w.numel(), q)
        theirs = torch.from_numpy(gq.dequantize(p.numpy().reshape(16, -1), t))
        assert torch.equal(ours, theirs), name
    path = str(tmp_path / "official.gguf")
    wr = gguf.GGUFWriter(path, "llama")
    wr.add_block_count(1)
    wr.add_string("custom.note", "héllo")
    wr.add_array("custom.list", [1, 2, 3])
    expect = {}
    for name, t in (("f32", T.F32), ("f16", T.F16), ("bf16", T.BF16), ("q8_0", T.Q8_0), ("q4_0", T.Q4_0),
                    ("q4_1", T.Q4_1), ("q5_0", T.Q5_0), ("q5_1", T.Q5_1)):
        data = gq.quantize(w.numpy(), t)
        wr.add_tensor(f"t.{name}", data, raw_shape=None if t in (T.F32, T.F16) else data.shape, raw_dtype=t)
        expect[f"t.{name}"] = gq.dequantize(data, t)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    loader = GGUFFileLoader(path)
    assert loader.config["custom.note"] == "héllo" and loader.config["custom.list"] == [1, 2, 3]
    assert loader.config["llama.block_count"] == 1
    got = loader.tensors()
    for k, e in expect.items():
        assert tuple(got[k].shape) == (16, 512) and np.array_equal(got[k].numpy(), e), k
    loader.close()


def test_q3_k_decoder_and_library_types_match_the_official_decoder():
    """q3_k super-blocks are decoded by this module's own numpy code, the rarer types (iq3 / iq4 / iq2_s / ternary) by
    the ``gguf`` package when it is installed: both against that package on random blocks."""
    pytest.importorskip("gguf")
    from gguf import quants as gq
    from gguf.constants import GGMLQuantizationType as T
    from ipex_llm_b200.transformers.gguf.gguf import GGML_TYPES, dequantize_blocks, type_geometry
    assert 11 in GGML_TYPES and type_geometry(int(T.IQ4_XS)) == ("iq4_xs", 256, 136)
    rng = np.random.default_rng(0)
    for t, bs, qk, tail in ((T.Q3_K, 110, 256, True), (T.IQ4_NL, 18, 32, False), (T.IQ4_XS, 136, 256, False),
                            (T.IQ3_XXS, 98, 256, False), (T.TQ2_0, 66, 256, True)):
        raw = rng.integers(0, 256, size=(9, bs), dtype=np.uint8)
        d = np.array([0.0123], dtype=np.float16).view(np.uint8)
        if tail:
            raw[:, -2:] = d
        else:
            raw[:, :2] = d
        ours = dequantize_blocks(raw.reshape(-1), int(t), 9 * qk)
        assert np.array_equal(ours, gq.dequantize(raw, t).reshape(-1)), t.name


def _export_llama_cpp_style(model, arch, path):
    """A GGUF file of a llama-shaped model as llama.cpp's exporter lays it out: q / k rows re-ordered only for the
    llama-type architectures, Gemma norms stored as 1 + w, Phi-3's fused matrices under ``attn_qkv`` / ``ffn_up``,
    Gemma-2's four norms per layer, Qwen-3's q / k norms."""
    from ipex_llm_b200.transformers.gguf.gguf import write_gguf
    cfg = model.config
    n_head, n_kv = cfg.num_attention_heads, cfg.num_key_value_heads

    def permute(t, heads):
        rows = t.shape[0]
        return t.reshape(heads, 2, rows // heads // 2, *t.shape[1:]).swapaxes(1, 2).reshape(t.shape)
    names = {"input_layernorm.weight": "attn_norm.weight", "self_attn.q_proj.weight": "attn_q.weight",
             "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
             "self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.bias": "attn_k.bias",
             "self_attn.v_proj.bias": "attn_v.bias", "self_attn.o_proj.weight": "attn_output.weight",
             "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
             "self_attn.qkv_proj.weight": "attn_qkv.weight", "mlp.gate_up_proj.weight": "ffn_up.weight",
             "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
             "mlp.down_proj.weight": "ffn_down.weight", "post_attention_layernorm.weight": "ffn_norm.weight"}
    if arch == "gemma2":
        names.update({"post_attention_layernorm.weight": "post_attention_norm.weight",
                      "pre_feedforward_layernorm.weight": "ffn_norm.weight",
                      "post_feedforward_layernorm.weight": "post_ffw_norm.weight"})
    tensors = {}
    for k, v in model.state_dict().items():
        v = v.clone()
        if arch in ("gemma", "gemma2") and k.endswith("norm.weight"):
            v = v + 1.0
        kind = "f32" if v.dim() == 1 else "f16"
        if k == "model.embed_tokens.weight":
            tensors["token_embd.weight"] = (v, kind)
        elif k == "model.norm.weight":
            tensors["output_norm.weight"] = (v, kind)
        elif k == "lm_head.weight":
            if not cfg.tie_word_embeddings:
                tensors["output.weight"] = (v, kind)
        else:
            _, _, layer, rest = k.split(".", 3)
            if arch == "llama" and "q_proj" in rest:
                v = permute(v, n_head)
            elif arch == "llama" and "k_proj" in rest:
                v = permute(v, n_kv)
            tensors[f"blk.{layer}.{names[rest]}"] = (v, kind)
    hd = getattr(cfg, "head_dim", None) or cfg.hidden_size // n_head
    meta = {"general.architecture": arch, "general.name": "tiny", f"{arch}.embedding_length": cfg.hidden_size,
            f"{arch}.feed_forward_length": cfg.intermediate_size, f"{arch}.block_count": cfg.num_hidden_layers,
            f"{arch}.attention.head_count": n_head, f"{arch}.attention.head_count_kv": n_kv,
            f"{arch}.attention.key_length": hd, f"{arch}.context_length": 256,
            f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), f"{arch}.rope.freq_base": 10000.0,
            "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2}
    if arch == "gemma2":
        meta.update({"gemma2.attn_logit_softcapping": 50.0, "gemma2.final_logit_softcapping": 30.0,
                     "gemma2.attention.sliding_window": 16})
    write_gguf(path, meta, tensors)


@pytest.mark.parametrize("arch", ["llama", "qwen2", "qwen3", "gemma", "gemma2", "phi3"])
def test_load_gguf_llama_shaped_architectures(tmp_path, arch):
    """Every llama-shaped architecture the loader names, exported with the conventions llama.cpp uses for it, loads
    to the logits of the source model."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    base = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, vocab_size=320, max_position_embeddings=256, rms_norm_eps=1e-5,
                bos_token_id=1, eos_token_id=2)
    cfgs = {"llama": transformers.LlamaConfig(**base, tie_word_embeddings=False),
            "qwen2": transformers.Qwen2Config(**base, tie_word_embeddings=False),
            "qwen3": transformers.Qwen3Config(**base, head_dim=32, tie_word_embeddings=False),
            "gemma": transformers.GemmaConfig(**base, head_dim=32, tie_word_embeddings=True),
            "gemma2": transformers.Gemma2Config(**base, head_dim=32, sliding_window=16, query_pre_attn_scalar=32,
                                                tie_word_embeddings=True),
            "phi3": transformers.Phi3Config(**base, pad_token_id=0, tie_word_embeddings=False)}
    torch.manual_seed(0)
    src = transformers.AutoModelForCausalLM.from_config(cfgs[arch]).eval()
    with torch.no_grad():
        for n, p in src.named_parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
            elif "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)                  # norms that are not the identity
            else:
                p.normal_(0, 0.05)                                 # biases (qwen2)
    path = str(tmp_path / f"{arch}.gguf")
    _export_llama_cpp_style(src, arch, path)
    model, _ = AutoModelForCausalLM.from_gguf(path, low_bit="sym_int8")
    assert model.config.model_type == arch
    ids = torch.randint(0, 320, (2, 12))
    with torch.no_grad():
        a = src(ids).logits[:, -1].float()
        b = model(ids).logits[:, -1].float()
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item() > 0.995


@pytest.mark.parametrize("pre", ["gpt-2", "llama-bpe", "qwen2"])
def test_byte_level_bpe_tokenizer_is_rebuilt_from_gguf_metadata(pre):
    """A byte-level BPE vocabulary (``tokenizer.ggml.model = gpt2``) stored as token and merge lists gives back a
    tokenizer with the encodings of the original, including the split pattern named by ``tokenizer.ggml.pre``."""
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    from ipex_llm_b200.transformers.gguf.api import _BPE_SPLIT, build_bpe_tokenizer
    corpus = ["The quick brown fox jumps over 12345 lazy dogs.", "Qu'est-ce que c'est? It's 2024-01-05!",
              "def f(x):\n    return x ** 2  # squared\n", "naïve café — 你好，世界 9876543210", "    indented\tline\r\n"] * 20
    orig = Tokenizer(models.BPE())
    if pre == "gpt-2":
        orig.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        orig.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(_BPE_SPLIT[pre]), behavior="isolated"),
            pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    orig.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<|begin|>", "<|end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    orig.train_from_iterator(corpus, trainer)
    vocab = orig.get_vocab()
    tokens = [t for t, _ in sorted(vocab.items(), key=lambda kv: kv[1])]
    import json
    merges = [" ".join(m) if not isinstance(m, str) else m for m in json.loads(orig.to_str())["model"]["merges"]]
    cfg = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": pre, "tokenizer.ggml.tokens": tokens,
           "tokenizer.ggml.merges": merges, "tokenizer.ggml.token_type": [3, 3] + [1] * (len(tokens) - 2),
           "tokenizer.ggml.bos_token_id": 0, "tokenizer.ggml.eos_token_id": 1}
    tok = build_bpe_tokenizer(cfg)
    assert tok.bos_token == "<|begin|>" and tok.eos_token == "<|end|>" and tok.padding_side == "left"
    for text in corpus[:5] + ["unseen words 007, mixed CASE and   spaces", "<|begin|>hello<|end|>"]:
        want = orig.encode(text).ids
        got = tok(text, add_special_tokens=False)["input_ids"]
        assert got == want, text
        if "<|" not in text:
            assert tok.decode(got) == text


def test_load_gguf_llama3_rope_factors(tmp_path):
    """Llama-3.1 files carry their long-context rotary scaling as a ``rope_freqs.weight`` tensor of per-frequency
    divisors: the loaded model rotates like the source model with ``rope_type = llama3``."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.transformers.gguf.gguf import GGUFFileLoader, write_gguf
    rope = {"rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0, "low_freq_factor": 1.0,
            "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    cfg = transformers.LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=320, max_position_embeddings=512,
                                   rope_parameters=rope, tie_word_embeddings=False, bos_token_id=1, eos_token_id=2)
    torch.manual_seed(0)
    src = transformers.AutoModelForCausalLM.from_config(cfg).eval()
    with torch.no_grad():
        for p in src.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
    plain = 1.0 / (10000.0 ** (torch.arange(0, 32, 2).float() / 32))
    factors = plain / src.model.rotary_emb.inv_freq
    assert factors.max() > 7.9 and factors.min() == 1.0
    path = str(tmp_path / "l31.gguf")
    _export_llama_cpp_style(src, "llama", path)
    # add the factor tensor to the file
    loader = GGUFFileLoader(path)
    meta = dict(loader.config)
    tensors = {n: (t, "f32" if t.dim() == 1 else "f16") for n, t in loader.tensors().items()}
    loader.close()
    tensors["rope_freqs.weight"] = (factors, "f32")
    write_gguf(path, meta, tensors)
    model, _ = AutoModelForCausalLM.from_gguf(path, low_bit="sym_int8")
    ids = torch.randint(0, 320, (1, 200))                       # long enough for the scaled frequencies to matter
    with torch.no_grad():
        a = src(ids).logits[:, -1].float()
        b = model(ids).logits[:, -1].float()
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item() > 0.995


def test_files_written_here_open_in_the_official_reader(tmp_path):
    """The package's writer and the native ``ipex-quantize`` produce files that ``gguf.GGUFReader`` opens: metadata
    (non-ASCII strings, arrays, floats, booleans) and tensors (dense, q8_0, k-quant) come back as written."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants as gq
    from ipex_llm_b200.ggml.quantize import quantize_gguf
    from ipex_llm_b200.transformers.gguf.gguf import write_gguf
    torch.manual_seed(0)
    w = {"blk.0.attn_q.weight": (torch.randn(8, 256), "f32"), "blk.0.ffn_up.weight": (torch.randn(4, 512), "f16"),
         "n.weight": (torch.randn(16), "f32"), "q.weight": (torch.randn(4, 64), "q8_0")}
    src, dst = str(tmp_path / "a.gguf"), str(tmp_path / "b.gguf")
    write_gguf(src, {"general.architecture": "llama", "llama.block_count": 1, "general.name": "tést",
                     "arr.list": [1, 2, 3], "strs": ["a", "bb"], "f": 1.5, "flag": True}, w)
    quantize_gguf(src, dst, "q4_k")
    dense = (gguf.GGMLQuantizationType.F32, gguf.GGMLQuantizationType.F16)
    for path, packed in ((src, False), (dst, True)):
        r = gguf.GGUFReader(path)
        assert bytes(r.fields["general.name"].parts[-1]).decode() == "tést"
        seen = {}
        for t in r.tensors:
            data = np.asarray(t.data, dtype=np.float32) if t.tensor_type in dense else gq.dequantize(t.data, t.tensor_type)
            ref = w[t.name][0].numpy()
            seen[t.name] = (t.tensor_type.name, float(np.linalg.norm(data.reshape(ref.shape) - ref) / np.linalg.norm(ref)))
        assert set(seen) == set(w)
        assert seen["blk.0.attn_q.weight"][0] == ("Q4_K" if packed else "F32")
        assert all(err < (0.1 if kind == "Q4_K" else 0.01) for kind, err in seen.values()), seen


def test_load_gguf_rope_scaling_metadata(tmp_path):
    """``<arch>.rope.scaling.type / factor`` (linear position interpolation) reaches the rebuilt model's rotary tables."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.transformers.gguf.gguf import GGUFFileLoader, write_gguf
    cfg = transformers.LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=320, max_position_embeddings=512,
                                   rope_parameters={"rope_type": "linear", "factor": 4.0, "rope_theta": 10000.0},
                                   tie_word_embeddings=False, bos_token_id=1, eos_token_id=2)
    torch.manual_seed(0)
    src = transformers.AutoModelForCausalLM.from_config(cfg).eval()
    with torch.no_grad():
        for p in src.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
    path = str(tmp_path / "lin.gguf")
    _export_llama_cpp_style(src, "llama", path)
    loader = GGUFFileLoader(path)
    meta = dict(loader.config)
    tensors = {n: (t, "f32" if t.dim() == 1 else "f16") for n, t in loader.tensors().items()}
    loader.close()
    meta.update({"llama.rope.scaling.type": "linear", "llama.rope.scaling.factor": 4.0})
    write_gguf(path, meta, tensors)
    model, _ = AutoModelForCausalLM.from_gguf(path, low_bit="sym_int8")
    assert torch.allclose(model.model.rotary_emb.inv_freq, src.model.rotary_emb.inv_freq)
    ids = torch.randint(0, 320, (1, 120))
    with torch.no_grad():
        a, b = src(ids).logits[:, -1].float(), model(ids).logits[:, -1].float()
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item() > 0.995
