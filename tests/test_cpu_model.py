"""CPU plumbing: tiny Llama through the public API (from_pretrained / generate / save_low_bit / load_low_bit /
optimize_model), family forward replacements, caches."""
import json
import os

import pytest
import torch


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().float(), b.flatten().float(), dim=0).item()


@pytest.fixture(scope="module")
def fp32_model(tiny_llama_dir):
    from transformers import LlamaForCausalLM
    return LlamaForCausalLM.from_pretrained(tiny_llama_dir).eval()


@pytest.fixture(scope="module")
def int4_model(tiny_llama_dir):
    from ipex_llm.transformers import AutoModelForCausalLM
    return AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_4bit=True)


def test_conversion_structure(int4_model):
    from ipex_llm_b200.ops.linear import LowBitLinear
    attn = int4_model.model.layers[0].self_attn
    assert isinstance(attn.qkv_proj, LowBitLinear) and not hasattr(attn, "q_proj")
    assert attn.qkv_proj.out_len == 768 and attn.qkv_proj.weight.data.dtype == torch.uint8
    # K = 688 is not a multiple of 64: the layer stays unquantized (reference convert.py:611-613)
    assert type(int4_model.model.layers[0].mlp.down_proj) is torch.nn.Linear
    assert isinstance(int4_model.lm_head, LowBitLinear) and int4_model.lm_head.optimize_lm_head
    assert int4_model.config.bigdl_transformers_low_bit == "sym_int4"


def test_logits_vs_fp32(int4_model, fp32_model, tiny_llama_dir):
    from ipex_llm.transformers import AutoModelForCausalLM
    torch.manual_seed(0)
    ids = torch.randint(0, 32000, (1, 32))
    os.environ["IPEX_LLM_LAST_LM_HEAD"] = "0"
    try:
        with torch.no_grad():
            ref = fp32_model(ids).logits
            out = int4_model(ids).logits
            # an unquantized random-weight model amplifies 4-bit noise layer by layer (there is no learned
            # structure to average it out): the same weights in 8 bits must be near exact, 4 bits well aligned
            int8 = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8")
            out8 = int8(ids).logits
    finally:
        os.environ.pop("IPEX_LLM_LAST_LM_HEAD")
    assert out.shape == ref.shape
    assert _cos(ref, out8) > 0.999
    assert _cos(ref, out) > 0.95
    # against an fp32 model that holds exactly the dequantized weights the converted model must agree (> 0.99
    # with a wide margin): the forward replacements and the low-bit matmul add no error of their own
    import copy
    deq = copy.deepcopy(fp32_model)
    for (n, mod) in int4_model.named_modules():
        if hasattr(mod, "weight") and getattr(mod.weight, "quantized", False):
            w = mod.weight.dequantize()
            if n.endswith("qkv_proj"):
                parent = deq.get_submodule(n.rsplit(".", 1)[0])
                q, k, v = w.split([256, 256, 256], dim=0)
                parent.q_proj.weight.data, parent.k_proj.weight.data, parent.v_proj.weight.data = q, k, v
            else:
                deq.get_submodule(n).weight.data = w
    with torch.no_grad():
        ref_deq = deq(ids).logits
    assert _cos(ref_deq[:, -1], int4_model(ids).logits[:, -1]) > 0.9999


def test_generate_32_tokens_matches_dequantized_reference(int4_model):
    torch.manual_seed(1)
    ids = torch.randint(0, 32000, (1, 32))
    out = int4_model.generate(ids, max_new_tokens=32, do_sample=False)
    assert out.shape == (1, 64)
    again = int4_model.generate(ids, max_new_tokens=32, do_sample=False)
    assert torch.equal(out, again)


def test_save_load_low_bit_roundtrip(int4_model, tmp_path):
    from ipex_llm.transformers import AutoModelForCausalLM
    d = str(tmp_path / "lowbit")
    int4_model.save_low_bit(d)
    for f in ("pytorch_model.bin", "config.json", "load_keys.json", "generation_config.json"):
        assert os.path.exists(os.path.join(d, f)), f
    cfg = json.load(open(os.path.join(d, "config.json")))
    assert cfg["bigdl_transformers_low_bit"] == "sym_int4" and cfg["tie_word_embeddings"] is False
    keys = json.load(open(os.path.join(d, "load_keys.json")))["all_checkpoint_keys"]
    assert "model.layers.0.self_attn.qkv_proj.weight" in keys
    sd = torch.load(os.path.join(d, "pytorch_model.bin"), weights_only=True)
    w = sd["model.layers.0.self_attn.qkv_proj.weight"]
    assert w.dtype == torch.uint8 and w.dim() == 1 and w.numel() == 768 * 256 // 64 * 34
    loaded = AutoModelForCausalLM.load_low_bit(d)
    ids = torch.randint(0, 32000, (1, 16))
    with torch.no_grad():
        assert torch.equal(int4_model(ids).logits, loaded(ids).logits)
    with pytest.raises(RuntimeError):
        AutoModelForCausalLM.from_pretrained(d, load_in_4bit=True)   # low-bit dirs go through load_low_bit


def test_load_low_bit_detects_missing_shard(int4_model, tmp_path):
    from ipex_llm.transformers import AutoModelForCausalLM
    d = str(tmp_path / "sharded")
    int4_model.save_low_bit(d, max_shard_size="4MB")
    idx = json.load(open(os.path.join(d, "pytorch_model.bin.index.json")))
    files = sorted(set(idx["weight_map"].values()))
    assert len(files) > 1
    loaded = AutoModelForCausalLM.load_low_bit(d)
    ids = torch.randint(0, 32000, (1, 8))
    with torch.no_grad():
        assert torch.equal(int4_model(ids).logits, loaded(ids).logits)
    os.remove(os.path.join(d, files[0]))
    with pytest.raises(RuntimeError):
        AutoModelForCausalLM.load_low_bit(d)


def test_optimize_model_api_and_low_memory_init(fp32_model, tmp_path):
    import copy
    from ipex_llm import optimize_model
    from ipex_llm.optimize import load_low_bit, low_memory_init
    m = optimize_model(copy.deepcopy(fp32_model), low_bit="sym_int8")
    d = str(tmp_path / "opt")
    m.save_low_bit(d)
    assert json.load(open(os.path.join(d, "bigdl_config.json")))["bigdl_transformers_low_bit"] == "sym_int8"
    from transformers import LlamaForCausalLM
    with low_memory_init():
        shell = LlamaForCausalLM(fp32_model.config)
    assert next(shell.parameters()).device.type == "meta"
    m2 = load_low_bit(shell, d)
    ids = torch.randint(0, 32000, (1, 12))
    with torch.no_grad():
        assert torch.allclose(m(ids).logits, m2(ids).logits, atol=1e-5)


def test_optimize_model_true_vs_false(tiny_llama_dir):
    """Forward replacements must not change the numerics of the low-bit model (reference test:
    test_transformers_api.py:151-169, mean relative difference < 5%)."""
    from ipex_llm.transformers import AutoModelForCausalLM
    a = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8", optimize_model=True)
    b = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8", optimize_model=False)
    ids = torch.randint(0, 32000, (2, 24))
    with torch.no_grad():
        la, lb = a(ids).logits, b(ids).logits
    la = la[:, -1] if la.shape[1] == 1 else la[:, -1]
    lb = lb[:, -1]
    assert _cos(la, lb) > 0.9999


def test_modules_to_not_convert_and_mixed_precision(tiny_llama_dir):
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.ops.linear import LowBitLinear
    from ipex_llm_b200.quant import qtypes as qt
    m = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_4bit=True, modules_to_not_convert=["lm_head", "o_proj"])
    assert type(m.lm_head) is torch.nn.Linear
    assert type(m.model.layers[0].self_attn.o_proj) is torch.nn.Linear
    m = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_4bit=True, mixed_precision=True)
    assert isinstance(m.lm_head, LowBitLinear) and m.lm_head.weight.qtype == qt.Q6_K


# multi-head latent attention + routed / shared experts of the DeepSeek families, at toy size
_MLA = dict(kv_lora_rank=32, q_lora_rank=48, qk_nope_head_dim=16, qk_rope_head_dim=16, v_head_dim=32,
            n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, n_shared_experts=1,
            first_k_dense_replace=1, num_key_value_heads=4)

FAMILY_CONFIGS = {
    "mistral": ("MistralConfig", dict(sliding_window=None)),
    "qwen2": ("Qwen2Config", dict()),
    "qwen3": ("Qwen3Config", dict(head_dim=32)),
    "gemma": ("GemmaConfig", dict(head_dim=32)),
    "gemma2": ("Gemma2Config", dict(head_dim=32, sliding_window=16, query_pre_attn_scalar=32)),
    "phi3": ("Phi3Config", dict(pad_token_id=0)),
    "glm": ("GlmConfig", dict(head_dim=32, pad_token_id=0)),
    "glm4": ("Glm4Config", dict(head_dim=32, pad_token_id=0)),
    "starcoder2": ("Starcoder2Config", dict()),
    "stablelm": ("StableLmConfig", dict()),
    "cohere": ("CohereConfig", dict(pad_token_id=0)),
    "gemma3_text": ("Gemma3TextConfig", dict(head_dim=32, sliding_window=16, query_pre_attn_scalar=32)),
    "olmo2": ("Olmo2Config", dict(pad_token_id=0)),
    "granite": ("GraniteConfig", dict()),
    "mixtral": ("MixtralConfig", dict(num_local_experts=4, num_experts_per_tok=2)),
    "qwen2_moe": ("Qwen2MoeConfig", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                                        shared_expert_intermediate_size=128)),
    "deepseek_v2": ("DeepseekV2Config", dict(_MLA, n_group=1, topk_group=1)),
    "deepseek_v3": ("DeepseekV3Config", dict(_MLA, n_group=2, topk_group=1)),
    "phimoe": ("PhimoeConfig", dict(num_local_experts=4, num_experts_per_tok=2)),
    "gptj": ("GPTJConfig", dict(n_embd=128, n_layer=2, n_head=4, rotary_dim=16)),
}


@pytest.mark.parametrize("family", list(FAMILY_CONFIGS))
def test_family_forward_replacement(family):
    """optimize_model on/off agree for every registered family (tiny random model, 8-bit weights)."""
    import copy
    import transformers
    from ipex_llm import optimize_model
    cls_name, extra = FAMILY_CONFIGS[family]
    kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256)
    kw.update(extra)
    cfg = getattr(transformers, cls_name)(**kw)
    torch.manual_seed(0)
    base = transformers.AutoModelForCausalLM.from_config(cfg).eval()
    a = optimize_model(copy.deepcopy(base), low_bit="sym_int8", optimize_llm=True)
    b = optimize_model(copy.deepcopy(base), low_bit="sym_int8", optimize_llm=False)
    ids = torch.randint(0, 1000, (2, 20))
    with torch.no_grad():
        la, lb = a(ids).logits[:, -1], b(ids).logits[:, -1]
        ref = base(ids).logits[:, -1]
    assert _cos(la, lb) > 0.999, family
    assert _cos(la, ref) > 0.99, family
    # incremental decoding through the package's caches agrees with a full forward
    out = a.generate(ids, max_new_tokens=4, do_sample=False)
    with torch.no_grad():
        full = a(out[:, :-1]).logits[:, -1].argmax(-1)
    assert torch.equal(full, out[:, -1]), family


def test_kv_caches():
    from ipex_llm_b200.ops.kv_cache import (DynamicCompressCache, DynamicFp8Cache, DynamicNormalCache,
                                            fp8_e5m2_dequantize)
    c = DynamicNormalCache()
    k, v = torch.randn(1, 2, 5, 16), torch.randn(1, 2, 5, 16)
    kk, vv = c.update(k, v, 0)
    assert kk.shape == (1, 2, 5, 16) and c.get_seq_length() == 5
    kk, _ = c.update(k[:, :, :1], v[:, :, :1], 0)
    assert kk.shape[2] == 6 and torch.equal(kk[:, :, :5], k)
    storage = c.layers[0]._k
    c.crop(4)
    assert c.get_seq_length() == 4 and c.layers[0]._k is storage      # O(1) crop keeps the allocation
    c.update(k[:, :, :3], v[:, :, :3], 0)
    assert c.get_seq_length() == 7
    f = DynamicFp8Cache()
    kq, vq = f.update(k, v, 0)
    assert kq.dtype == torch.uint8
    assert torch.allclose(fp8_e5m2_dequantize(kq, torch.float32), k, atol=0.13, rtol=0.13)
    s = DynamicCompressCache()
    q = torch.randn(1, 2, 2000, 16)
    kl, vl = torch.randn(1, 2, 2000, 16), torch.randn(1, 2, 2000, 16)
    s.layers.append(s.layer_class_to_replicate())
    k_ret, _ = s.update(kl, vl, 0, query_states=q, attention_mask=None, num_key_value_groups=1)
    assert k_ret.shape[2] == 2000 and s.get_seq_length() == 1024 and s.real_kv_len == 2000


def test_kv_caches_random_walk():
    """Random sequences of appends (prompt-sized and single-token, several layers) and crops on the normal, e5m2 and
    4-bit caches against a list-concatenation model: shapes, sequence length, old rows bit-stable, new rows within the
    format's step."""
    import random
    from ipex_llm_b200.ops.kv_cache import (DynamicFp8Cache, DynamicInt4Cache, DynamicNormalCache, fp8_e5m2_dequantize,
                                            fp8_e5m2_quantize, int4_kv_dequantize, int4_kv_quantize)
    rnd = random.Random(0)
    torch.manual_seed(0)

    def roundtrip(kind, x):
        if kind == "fp8":
            return fp8_e5m2_dequantize(fp8_e5m2_quantize(x), torch.float32)
        if kind == "int4":
            return int4_kv_dequantize(int4_kv_quantize(x), torch.float32)
        return x

    for trial in range(60):
        kind = rnd.choice(["normal", "fp8", "int4"])
        cache = {"normal": DynamicNormalCache, "fp8": DynamicFp8Cache, "int4": DynamicInt4Cache}[kind]()
        L, B, H, D = rnd.randint(1, 3), rnd.randint(1, 2), rnd.randint(1, 3), rnd.choice([16, 64])
        ref = [None] * L
        n = 0
        for step in range(rnd.randint(1, 10)):
            if rnd.random() < 0.75 or n == 0:
                s = rnd.choice([1, 1, 1, 2, 5, 17, 300]) if n else rnd.choice([1, 7, 33, 257, 600])
                for l in range(L):
                    k, v = torch.randn(B, H, s, D), torch.randn(B, H, s, D)
                    kk, vv = cache.update(k, v, l)
                    rk, rv = roundtrip(kind, k), roundtrip(kind, v)
                    ref[l] = (rk, rv) if ref[l] is None else (torch.cat([ref[l][0], rk], 2), torch.cat([ref[l][1], rv], 2))
                    if kind == "fp8":
                        kk, vv = fp8_e5m2_dequantize(kk, torch.float32), fp8_e5m2_dequantize(vv, torch.float32)
                    kk, vv = kk.float(), vv.float()
                    assert kk.shape == ref[l][0].shape, (kind, trial, step)
                    old = ref[l][0].shape[2] - s
                    if old:                  # (a prompt pass may hand back its own unquantized rows; old rows never change)
                        assert torch.allclose(kk[:, :, :old], ref[l][0][:, :, :old], atol=1e-6), (kind, trial, step)
                        assert torch.allclose(vv[:, :, :old], ref[l][1][:, :, :old], atol=1e-6), (kind, trial, step)
                    tol = {"normal": 1e-6, "fp8": 0.6, "int4": 1.0}[kind]
                    assert (kk[:, :, old:] - ref[l][0][:, :, old:]).abs().max() <= tol, (kind, trial, step)
                n += s
            else:
                n = rnd.randint(0, n)
                cache.crop(n)
                ref = [None if r is None or n == 0 else (r[0][:, :, :n], r[1][:, :, :n]) for r in ref]
            assert cache.get_seq_length() == n, (kind, trial, step)


def test_int4_kv_cache(tiny_llama_dir, monkeypatch):
    """IPEX_LLM_QUANTIZE_KV_CACHE=int4: codes + per-row scale round-trip within the 4-bit step, the cache keeps
    D/2 + 2 bytes per row, and generation through it stays close to the fp16 cache."""
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.ops.kv_cache import DynamicInt4Cache, int4_kv_dequantize, int4_kv_quantize
    x = torch.randn(2, 3, 5, 64)
    p = int4_kv_quantize(x)
    assert p.dtype == torch.uint8 and p.shape == (2, 3, 5, 34)
    step = x.abs().amax(-1, keepdim=True) / 7
    assert ((int4_kv_dequantize(p, torch.float32) - x).abs() <= 0.51 * step + 1e-3).all()
    c = DynamicInt4Cache()
    k, v = torch.randn(1, 2, 6, 64), torch.randn(1, 2, 6, 64)
    kk, vv = c.update(k, v, 0)
    assert torch.equal(kk, k)                                   # the prompt attends to its own K / V
    kk, vv = c.update(k[:, :, :1], v[:, :, :1], 0)
    assert kk.shape == (1, 2, 7, 64) and c.get_seq_length() == 7 and c.layers[0]._k.shape[-1] == 34
    assert (kk[:, :, :6] - k).abs().max() < 0.51 * float(k.abs().max()) / 7 + 1e-3
    c.crop(4)
    assert c.get_seq_length() == 4
    m = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8")
    ids = torch.randint(0, 1000, (1, 24))
    ref = m.generate(ids, max_new_tokens=8, do_sample=False)
    monkeypatch.setenv("IPEX_LLM_QUANTIZE_KV_CACHE", "int4")
    seen = []
    orig = DynamicInt4Cache.__init__

    def spy(self, *a, **kw):
        seen.append(1)
        orig(self, *a, **kw)
    monkeypatch.setattr(DynamicInt4Cache, "__init__", spy)
    out = m.generate(ids, max_new_tokens=8, do_sample=False)
    assert seen, "generation did not pick the 4-bit cache"
    assert out.shape == ref.shape and torch.equal(out[:, :25], ref[:, :25])
    # a random tiny model has near-ties between tokens, so the decode step is compared by its logits
    with torch.no_grad():
        step = []
        for cache in (None, DynamicInt4Cache()):
            kw = {} if cache is None else {"past_key_values": cache}
            o = m(ids, use_cache=True, **kw)
            step.append(m(ref[:, 24:25], past_key_values=o.past_key_values, use_cache=True).logits[0, -1].float())
    assert torch.nn.functional.cosine_similarity(step[0], step[1], dim=0) > 0.98


def test_env_flags(monkeypatch):
    from ipex_llm_b200 import config as cfg
    monkeypatch.setenv("IPEX_LLM_QUANTIZE_KV_CACHE", "1")
    assert cfg.quantize_kv_cache_flag() is True
    monkeypatch.setenv("IPEX_LLM_QUANTIZE_KV_CACHE", "0")
    assert cfg.quantize_kv_cache_flag() is False
    monkeypatch.delenv("IPEX_LLM_QUANTIZE_KV_CACHE")
    assert cfg.quantize_kv_cache_flag() is None
    monkeypatch.setenv("IPEX_LLM_LOW_MEM", "1")
    assert cfg.low_mem()


@pytest.mark.parametrize("with_keys_file", [True, False])
@pytest.mark.parametrize("victim", ["model.layers.1.self_attn.o_proj.weight", "truncate"])
def test_load_low_bit_rejects_absent_or_truncated_tensor(int4_model, tmp_path, with_keys_file, victim):
    """A packed weight that is missing from the checkpoint, or shorter than its shape needs, fails at load time
    whether or not load_keys.json is there to list it (reference model.py:593-739 errors at load as well)."""
    from ipex_llm.transformers import AutoModelForCausalLM
    d = str(tmp_path / "ckpt")
    int4_model.save_low_bit(d)
    f = os.path.join(d, "pytorch_model.bin")
    sd = torch.load(f, map_location="cpu", weights_only=True)
    if victim == "truncate":
        k = "model.layers.0.mlp.gate_proj.weight"
        sd[k] = sd[k][: sd[k].numel() // 2].clone()
    else:
        assert victim in sd
        del sd[victim]
    torch.save(sd, f)
    if not with_keys_file:
        os.remove(os.path.join(d, "load_keys.json"))
    with pytest.raises(RuntimeError):
        AutoModelForCausalLM.load_low_bit(d)


def _write_imatrix(path, n_layers, hidden, inter):
    """A llama.cpp importance-matrix file with one record per projection."""
    import struct
    recs = []
    for l in range(n_layers):
        for name, n in (("attn_q", hidden), ("attn_k", hidden), ("attn_v", hidden), ("attn_qkv", hidden),
                        ("attn_output", hidden), ("ffn_gate", hidden), ("ffn_up", hidden), ("ffn_down", inter)):
            recs.append((f"blk.{l}.{name}.weight", torch.rand(n) + 0.1))
    with open(path, "wb") as f:
        f.write(struct.pack("<i", len(recs)))
        for name, vals in recs:
            b = name.encode()
            f.write(struct.pack("<i", len(b)) + b + struct.pack("<ii", 2, vals.numel()))
            f.write((vals * 2).numpy().astype("float32").tobytes())


@pytest.mark.parametrize("low_bit", ["gguf_iq2_xxs", "gguf_iq1_s"])
def test_codebook_low_bit_model(tiny_llama_dir, tmp_path, low_bit):
    """load_in_low_bit="gguf_iq2_xxs" / "gguf_iq1_s" with an importance matrix (reference model.py:325-341,
    utils.py:286-356): per-layer types follow the policy, the model runs, and the packed model reloads bit-exactly."""
    pytest.importorskip("gguf.quants")
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.quant import qtypes as qt
    with pytest.raises(Exception):
        AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit=low_bit)        # imatrix is required
    im = str(tmp_path / "imatrix.dat")
    _write_imatrix(im, 2, 256, 688)
    m = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit=low_bit, imatrix=im)
    attn = m.model.layers[0].self_attn
    want = qt.qtype_from_name(low_bit)
    assert attn.qkv_proj.weight.qtype == want
    assert m.model.layers[0].mlp.gate_proj.weight.qtype == want
    assert attn.o_proj.weight.qtype == (qt.IQ2_XXS if low_bit == "gguf_iq1_s" else want)
    assert m.lm_head.weight.qtype == qt.SYM_INT8
    ids = torch.randint(0, 32000, (1, 12))
    with torch.no_grad():
        logits = m(ids).logits
    assert torch.isfinite(logits).all()
    out = m.generate(ids, max_new_tokens=4, do_sample=False)
    assert out.shape == (1, 16)
    d = str(tmp_path / "packed")
    m.save_low_bit(d)
    again = AutoModelForCausalLM.load_low_bit(d)
    from ipex_llm_b200.quant.params import FP4Params
    assert isinstance(again.model.embed_tokens.weight, FP4Params) and again.model.embed_tokens.weight.qtype == qt.Q2_K
    with torch.no_grad():
        assert torch.equal(again(ids).logits, logits)


def test_phi3_longrope_generation_switches_factor_sets():
    """Phi-3 LongRoPE (reference models/phi3.py:62-86): forward agrees with the fp32 model below and above
    ``original_max_position_embeddings``, and greedy generation that crosses the switch point equals greedy decoding by
    full recomputation (the cache is rebuilt once with the long factors)."""
    import copy
    import transformers
    from ipex_llm import optimize_model
    hd = 32
    rope = {"rope_type": "longrope", "rope_theta": 10000.0, "original_max_position_embeddings": 32,
            "short_factor": [1.0 + 0.05 * i for i in range(hd // 2)],
            "long_factor": [2.0 + 0.3 * i for i in range(hd // 2)]}
    cfg = transformers.Phi3Config(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                  num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256,
                                  original_max_position_embeddings=32, pad_token_id=0, rope_parameters=rope)
    torch.manual_seed(0)
    base = transformers.AutoModelForCausalLM.from_config(cfg).eval()
    low = optimize_model(copy.deepcopy(base), low_bit="sym_int8")
    for n in (20, 80):
        ids = torch.randint(0, 1000, (2, n))
        with torch.no_grad():
            assert _cos(low(ids).logits[:, -1], base(ids).logits[:, -1]) > 0.999, n
    ids = torch.randint(0, 1000, (1, 28))
    out = low.generate(ids, max_new_tokens=10, do_sample=False)
    cur = ids
    with torch.no_grad():
        for _ in range(10):
            cur = torch.cat([cur, low(cur).logits[:, -1].argmax(-1, keepdim=True)], 1)
    assert torch.equal(out, cur)


def test_deepseek_v3_routing_goes_through_the_grouped_topk_router():
    """The converted DeepSeek-V3 MoE block routes with ``ops.moe.moe_group_topk`` (reference models/deepseek.py:283-287)
    and picks the same experts and weights as the transformers formulation, also with a non-zero correction bias."""
    import copy
    import transformers
    from ipex_llm import optimize_model
    kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, vocab_size=1000,
              max_position_embeddings=256)
    kw.update(dict(_MLA, n_routed_experts=8, n_group=4, topk_group=2, num_experts_per_tok=3, norm_topk_prob=True,
                   routed_scaling_factor=2.5))
    cfg = transformers.DeepseekV3Config(**kw)
    torch.manual_seed(0)
    base = transformers.AutoModelForCausalLM.from_config(cfg).eval()
    moe = [m for m in base.modules() if type(m).__name__ == "DeepseekV3MoE"][0]
    moe.gate.e_score_correction_bias.copy_(torch.rand(8) * 0.2)
    low = optimize_model(copy.deepcopy(base), low_bit="sym_int8")
    low_moe = [m for m in low.modules() if type(m).__name__ == "DeepseekV3MoE"][0]
    assert low_moe.route_tokens_to_experts.__func__.__name__ == "_deepseek_v3_route"
    logits = torch.randn(11, 8)
    i0, w0 = moe.route_tokens_to_experts(logits.clone())
    i1, w1 = low_moe.route_tokens_to_experts(logits.clone())
    assert torch.equal(i0.sort(-1).values, i1.sort(-1).values)
    assert torch.allclose(w0.gather(1, i0.argsort(-1)), w1.gather(1, i1.argsort(-1)).to(w0.dtype), atol=1e-6)
    ids = torch.randint(0, 1000, (2, 16))
    with torch.no_grad():
        assert _cos(low(ids).logits[:, -1], base(ids).logits[:, -1]) > 0.999


@pytest.mark.parametrize("family", list(FAMILY_CONFIGS))
def test_low_bit_checkpoint_round_trip_across_families(family, tmp_path):
    """``save_low_bit`` -> ``load_low_bit`` reproduces the logits bit for bit for every family, including those with
    buffers that are not part of a checkpoint (rotary tables, Gemma's embedding scale, GPT-J's sinusoidal table) and
    with fused expert banks."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    cls_name, extra = FAMILY_CONFIGS[family]
    kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256)
    kw.update(extra)
    torch.manual_seed(0)
    src = transformers.AutoModelForCausalLM.from_config(getattr(transformers, cls_name)(**kw)).eval()
    d0, d1 = str(tmp_path / "hf"), str(tmp_path / "low")
    src.save_pretrained(d0)
    m = AutoModelForCausalLM.from_pretrained(d0, load_in_low_bit="sym_int8")
    m.save_low_bit(d1)
    again = AutoModelForCausalLM.load_low_bit(d1)
    ids = torch.randint(0, 1000, (2, 11))
    with torch.no_grad():
        a, b = m(ids).logits, again(ids).logits
    assert torch.equal(a, b) and a.abs().max() > 0


@pytest.mark.parametrize("family", ["gemma2", "gemma3_text", "qwen3", "mixtral", "deepseek_v3", "gptj", "glm"])
def test_left_padded_batch_generates_like_single_prompts(family):
    """A short prompt left-padded beside a longer one generates the tokens it generates alone (position ids, padding
    masks, and, under a sliding window, padding rows that see no key at all must not leak NaN into real rows)."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    cls_name, extra = FAMILY_CONFIGS[family]
    kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256)
    kw.update(extra)
    torch.manual_seed(0)
    m = AutoModelForCausalLM.from_config(getattr(transformers, cls_name)(**kw), load_in_low_bit="sym_int8",
                                         device="cpu", torch_dtype=torch.float32)
    m.generation_config.pad_token_id = 0
    g = torch.Generator().manual_seed(0)
    a, b = torch.randint(5, 900, (1, 9), generator=g), torch.randint(5, 900, (1, 16), generator=g)
    batch = torch.cat([torch.cat([torch.zeros(1, 7, dtype=torch.long), a], 1), b], 0)
    mask = torch.ones_like(batch)
    mask[0, :7] = 0
    both = m.generate(batch, attention_mask=mask, max_new_tokens=6, do_sample=False)
    alone_a = m.generate(a, attention_mask=torch.ones_like(a), max_new_tokens=6, do_sample=False)
    alone_b = m.generate(b, attention_mask=torch.ones_like(b), max_new_tokens=6, do_sample=False)
    assert torch.equal(both[0, 16:], alone_a[0, 9:]) and torch.equal(both[1, 16:], alone_b[0, 16:])


@pytest.mark.parametrize("family", ["gemma2", "mixtral"])
def test_embedding_variants_across_families(family, tmp_path, monkeypatch):
    """``cpu_embedding``, ``disk_embedding`` and a packed ``embedding_qtype`` on a family with scaled word embeddings
    (Gemma-2: the factor survives the replacement of the table) and on one whose router reads the hidden states
    directly (Mixtral: a disk-resident table hands out fp16 rows)."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.ops.embedding import CPUEmbedding, DiskEmbedding, LowBitEmbedding
    monkeypatch.chdir(tmp_path)                                # DiskEmbedding writes embeddings.bin beside the process
    cls_name, extra = FAMILY_CONFIGS[family]
    kw = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256)
    kw.update(extra)
    torch.manual_seed(0)
    src = transformers.AutoModelForCausalLM.from_config(getattr(transformers, cls_name)(**kw)).eval()
    d = str(tmp_path / "hf")
    src.save_pretrained(d)
    ids = torch.randint(0, 900, (2, 11))
    with torch.no_grad():
        ref = src(ids).logits[:, -1]
    scaled = family == "gemma2"
    for kwargs, cls, floor in ((dict(cpu_embedding=True), CPUEmbedding, 0.999),
                               (dict(embedding_qtype="q4_k"), LowBitEmbedding, 0.99),
                               (dict(disk_embedding=True), None if scaled else DiskEmbedding, 0.999)):
        m = AutoModelForCausalLM.from_pretrained(d, load_in_low_bit="sym_int8", **kwargs)
        if cls is not None:
            assert isinstance(m.get_input_embeddings(), cls), kwargs
            if scaled:
                assert m.get_input_embeddings().embed_scale_value == 16.0
        with torch.no_grad():
            assert _cos(m(ids).logits[:, -1], ref) > floor, kwargs


def test_mixed_formats_and_rtn_names(tmp_path):
    """``mixed_fp4`` / ``mixed_fp8`` choose an integer or a float format per layer; the choice is stored with the
    checkpoint (the bytes do not tell) so ``load_low_bit`` decodes every layer as it was packed.  The per-channel
    ``*_rtn`` names of the NPU entry point are accepted on the main API as the blocked format of the same width."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.quant import qtypes as qt
    cfg = transformers.LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=500, max_position_embeddings=64,
                                   tie_word_embeddings=False)
    torch.manual_seed(0)
    src = transformers.LlamaForCausalLM(cfg)
    with torch.no_grad():
        for n, p in src.named_parameters():
            if "layers.0" in n and p.dim() > 1:
                p.copy_(torch.randn_like(p) ** 3 * 0.02)         # heavy tails: the float format wins in this layer
    d = str(tmp_path / "hf")
    src.save_pretrained(d)
    ids = torch.randint(0, 500, (1, 8))
    m = AutoModelForCausalLM.from_pretrained(d, load_in_low_bit="mixed_fp4")
    kinds = {m_.weight.qtype for m_ in m.modules() if getattr(getattr(m_, "weight", None), "quantized", False)}
    assert kinds == {qt.SYM_INT4, qt.FP4}
    low = str(tmp_path / "low")
    m.save_low_bit(low)
    again = AutoModelForCausalLM.load_low_bit(low)
    with torch.no_grad():
        assert torch.equal(again(ids).logits, m(ids).logits)
    m8 = AutoModelForCausalLM.from_pretrained(d, load_in_low_bit="mixed_fp8")
    with torch.no_grad():
        assert torch.isfinite(m8(ids).logits).all()
    with pytest.warns(UserWarning, match="per-channel NPU format"):
        rtn = AutoModelForCausalLM.from_pretrained(d, load_in_low_bit="sym_int8_rtn")
    assert rtn.config.bigdl_transformers_low_bit == "sym_int8"
