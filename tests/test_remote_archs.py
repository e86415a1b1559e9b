"""Checkpoints of remote-code families (ChatGLM2/3, Baichuan-7B / Baichuan2, InternLM, InternLM2, Qwen v1, MiniCPM,
Aquila) load into the natively implemented architecture they are equivalent to.  Each test writes a checkpoint in
the family's own tensor naming / layout (built here, independently of the loader, from a random native model) and
checks that loading it reproduces the native model's logits, plain and quantized."""
import json
import math

import torch


def _save(tmp_path, config: dict, state: dict):
    from safetensors.torch import save_file
    d = tmp_path / config["model_type"]
    d.mkdir()
    (d / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in state.items()}, str(d / "model.safetensors"))
    return str(d)


def _check(path, native, atol=1e-5):
    from ipex_llm.transformers import AutoModelForCausalLM
    ids = torch.randint(0, native.config.vocab_size, (2, 12))
    with torch.no_grad():
        ref = native(ids).logits
    m = AutoModelForCausalLM.from_pretrained(path)
    with torch.no_grad():
        out = m(ids).logits
    assert torch.allclose(out, ref, atol=atol), (out - ref).abs().max()
    q = AutoModelForCausalLM.from_pretrained(path, load_in_low_bit="sym_int8")
    with torch.no_grad():
        lq = q(ids).logits[:, -1]
    cos = torch.nn.functional.cosine_similarity(lq.float(), ref[:, -1].float(), dim=-1)
    assert cos.min() > 0.99, cos
    return m


def _native(cfg):
    import transformers
    torch.manual_seed(0)
    return transformers.AutoModelForCausalLM.from_config(cfg).eval()


def test_chatglm_checkpoint_loads_as_glm(tmp_path):
    from transformers import GlmConfig
    nh, ng, hd, H, I, L = 4, 2, 32, 128, 256, 2
    native = _native(GlmConfig(vocab_size=1000, hidden_size=H, intermediate_size=I, num_hidden_layers=L,
                               num_attention_heads=nh, num_key_value_heads=ng, head_dim=hd, attention_bias=True,
                               partial_rotary_factor=0.5, rms_norm_eps=1e-5, max_position_embeddings=256,
                               tie_word_embeddings=False, pad_token_id=0))
    sd = native.state_dict()
    st = {"transformer.embedding.word_embeddings.weight": sd["model.embed_tokens.weight"],
          "transformer.encoder.final_layernorm.weight": sd["model.norm.weight"],
          "transformer.output_layer.weight": sd["lm_head.weight"],
          "transformer.rotary_pos_emb.inv_freq": torch.ones(8)}
    for i in range(L):
        p, r = f"model.layers.{i}.", f"transformer.encoder.layers.{i}."
        for suffix in ("weight", "bias"):
            st[r + "self_attention.query_key_value." + suffix] = torch.cat(
                [sd[p + f"self_attn.{n}_proj.{suffix}"] for n in "qkv"], dim=0)
        st[r + "self_attention.dense.weight"] = sd[p + "self_attn.o_proj.weight"]
        st[r + "mlp.dense_h_to_4h.weight"] = sd[p + "mlp.gate_up_proj.weight"]
        st[r + "mlp.dense_4h_to_h.weight"] = sd[p + "mlp.down_proj.weight"]
        st[r + "input_layernorm.weight"] = sd[p + "input_layernorm.weight"]
        st[r + "post_attention_layernorm.weight"] = sd[p + "post_attention_layernorm.weight"]
    cfg = {"model_type": "chatglm", "num_layers": L, "hidden_size": H, "ffn_hidden_size": I, "kv_channels": hd,
           "num_attention_heads": nh, "multi_query_attention": True, "multi_query_group_num": ng,
           "padded_vocab_size": 1000, "layernorm_epsilon": 1e-5, "add_qkv_bias": True, "seq_length": 256,
           "rmsnorm": True, "torch_dtype": "float32"}
    m = _check(_save(tmp_path, cfg, st), native)
    assert m.config.model_type == "glm" and m.config.ipex_remote_model_type == "chatglm"


def _llama_cfg(**kw):
    from transformers import LlamaConfig
    base = dict(vocab_size=1000, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=4, max_position_embeddings=256, tie_word_embeddings=False, rms_norm_eps=1e-6)
    base.update(kw)
    return LlamaConfig(**base)


def test_baichuan2_checkpoint_loads_as_llama(tmp_path):
    native = _native(_llama_cfg(vocab_size=125696, hidden_size=64, intermediate_size=128))
    sd = dict(native.state_dict())
    # Baichuan2's NormHead stores unnormalised rows and normalises them at inference time
    raw_head = sd["lm_head.weight"] * (1.0 + torch.rand(sd["lm_head.weight"].shape[0], 1))
    native.lm_head.weight.data = torch.nn.functional.normalize(raw_head)
    st = {}
    for k, v in sd.items():
        if ".self_attn.q_proj." in k:
            st[k.replace("q_proj", "W_pack")] = torch.cat([sd[k], sd[k.replace("q_proj", "k_proj")],
                                                           sd[k.replace("q_proj", "v_proj")]], dim=0)
        elif ".self_attn.k_proj." in k or ".self_attn.v_proj." in k:
            continue
        elif k == "lm_head.weight":
            st[k] = raw_head
        else:
            st[k] = v
    cfg = {"model_type": "baichuan", "vocab_size": 125696, "hidden_size": 64, "intermediate_size": 128,
           "num_hidden_layers": 2, "num_attention_heads": 4, "rms_norm_eps": 1e-6, "model_max_length": 256,
           "max_position_embeddings": 256, "torch_dtype": "float32"}
    _check(_save(tmp_path, cfg, st), native, atol=1e-4)


def test_baichuan_13b_checkpoint_runs_with_linear_attention_biases(tmp_path):
    """Baichuan-13B / Baichuan2-13B (reference models/baichuan.py:403-447): no rotary positions, every head adds
    slope_h * key position to its scores.  Compared with a plain restatement of that architecture."""
    import math
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.models.decoder import alibi_slopes
    assert torch.allclose(alibi_slopes(8), torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    s12 = alibi_slopes(12)                               # 8 of the 8-head series, then every other one of the 16-head series
    assert torch.allclose(s12[:8], alibi_slopes(8)) and torch.allclose(s12[8:], alibi_slopes(16)[0::2][:4])
    H, nh, L, V, I = 96, 6, 2, 500, 192
    hd = H // nh
    native = _native(_llama_cfg(vocab_size=V, hidden_size=H, intermediate_size=I, num_attention_heads=nh,
                                num_key_value_heads=nh))
    sd = dict(native.state_dict())
    st = {}
    for k, v in sd.items():
        if ".self_attn.q_proj." in k:
            st[k.replace("q_proj", "W_pack")] = torch.cat([sd[k], sd[k.replace("q_proj", "k_proj")],
                                                           sd[k.replace("q_proj", "v_proj")]], dim=0)
        elif ".self_attn.k_proj." not in k and ".self_attn.v_proj." not in k:
            st[k] = v
    cfg = {"model_type": "baichuan", "vocab_size": V, "hidden_size": H, "intermediate_size": I,
           "num_hidden_layers": L, "num_attention_heads": nh, "rms_norm_eps": 1e-6, "model_max_length": 256,
           "torch_dtype": "float32"}
    d = _save(tmp_path, cfg, st)

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    def plain(ids):
        x = sd["model.embed_tokens.weight"][ids]
        B, S, _ = x.shape
        slopes = alibi_slopes(nh).view(1, nh, 1, 1)
        bias = slopes * torch.arange(S).view(1, 1, 1, S) + torch.full((S, S), float("-inf")).triu(1)
        for i in range(L):
            p = f"model.layers.{i}."
            h = rms(x, sd[p + "input_layernorm.weight"])
            q, k, v = [(h @ sd[p + f"self_attn.{n}_proj.weight"].t()).view(B, S, nh, hd).transpose(1, 2) for n in "qkv"]
            a = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(hd) + bias, -1) @ v
            x = x + a.transpose(1, 2).reshape(B, S, H) @ sd[p + "self_attn.o_proj.weight"].t()
            h = rms(x, sd[p + "post_attention_layernorm.weight"])
            g = torch.nn.functional.silu(h @ sd[p + "mlp.gate_proj.weight"].t()) * (h @ sd[p + "mlp.up_proj.weight"].t())
            x = x + g @ sd[p + "mlp.down_proj.weight"].t()
        return rms(x, sd["model.norm.weight"]) @ sd["lm_head.weight"].t()

    m = AutoModelForCausalLM.from_pretrained(d, load_in_low_bit="bf16", torch_dtype=torch.float32)
    assert m.config.ipex_alibi is True
    ids = torch.randint(0, V, (2, 17))
    with torch.no_grad():
        got, want = m(ids).logits.float(), plain(ids)
    got = got[:, -1] if got.shape[1] == 1 else got[:, -1]
    assert torch.nn.functional.cosine_similarity(got.flatten(), want[:, -1].flatten(), dim=0) > 0.999
    plain_load = AutoModelForCausalLM.from_pretrained(d)             # no conversion asked for: biases all the same
    with torch.no_grad():
        assert torch.allclose(plain_load(ids).logits, want, atol=1e-4)
    # incremental decoding adds the same biases as a full pass
    out = m.generate(ids[:1], max_new_tokens=5, do_sample=False)
    with torch.no_grad():
        again = m(out[:, :-1]).logits[:, -1].argmax(-1)
    assert torch.equal(again, out[:, -1])


def test_internlm_and_aquila_checkpoints_load_as_llama(tmp_path):
    native = _native(_llama_cfg(attention_bias=True))
    cfg = {"model_type": "internlm", "vocab_size": 1000, "hidden_size": 128, "intermediate_size": 256,
           "num_hidden_layers": 2, "num_attention_heads": 4, "bias": True, "max_position_embeddings": 256,
           "torch_dtype": "float32"}
    _check(_save(tmp_path, cfg, dict(native.state_dict())), native)
    native = _native(_llama_cfg())
    cfg = {"model_type": "aquila", "vocab_size": 1000, "hidden_size": 128, "intermediate_size": 256,
           "num_hidden_layers": 2, "num_attention_heads": 4, "max_position_embeddings": 256,
           "torch_dtype": "float32"}
    _check(_save(tmp_path, cfg, dict(native.state_dict())), native)


def test_internlm2_checkpoint_loads_as_llama(tmp_path):
    nh, nkv, hd, L = 4, 2, 32, 2
    groups = nh // nkv
    native = _native(_llama_cfg(num_key_value_heads=nkv))
    sd = native.state_dict()
    st = {"model.tok_embeddings.weight": sd["model.embed_tokens.weight"], "model.norm.weight": sd["model.norm.weight"],
          "output.weight": sd["lm_head.weight"]}
    for i in range(L):
        p = f"model.layers.{i}."
        q = sd[p + "self_attn.q_proj.weight"].view(nkv, groups, hd, -1)
        k = sd[p + "self_attn.k_proj.weight"].view(nkv, 1, hd, -1)
        v = sd[p + "self_attn.v_proj.weight"].view(nkv, 1, hd, -1)
        st[p + "attention.wqkv.weight"] = torch.cat([q, k, v], dim=1).reshape((nh + 2 * nkv) * hd, -1)
        st[p + "attention.wo.weight"] = sd[p + "self_attn.o_proj.weight"]
        st[p + "feed_forward.w1.weight"] = sd[p + "mlp.gate_proj.weight"]
        st[p + "feed_forward.w3.weight"] = sd[p + "mlp.up_proj.weight"]
        st[p + "feed_forward.w2.weight"] = sd[p + "mlp.down_proj.weight"]
        st[p + "attention_norm.weight"] = sd[p + "input_layernorm.weight"]
        st[p + "ffn_norm.weight"] = sd[p + "post_attention_layernorm.weight"]
    cfg = {"model_type": "internlm2", "vocab_size": 1000, "hidden_size": 128, "intermediate_size": 256,
           "num_hidden_layers": L, "num_attention_heads": nh, "num_key_value_heads": nkv, "bias": False,
           "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "torch_dtype": "float32"}
    _check(_save(tmp_path, cfg, st), native)


def test_qwen_v1_checkpoint_loads_as_qwen2(tmp_path):
    from transformers import Qwen2Config
    H, I, L = 128, 256, 2
    native = _native(Qwen2Config(vocab_size=1000, hidden_size=H, intermediate_size=I, num_hidden_layers=L,
                                 num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=256,
                                 tie_word_embeddings=False, rms_norm_eps=1e-6))
    sd = native.state_dict()
    st = {"transformer.wte.weight": sd["model.embed_tokens.weight"], "transformer.ln_f.weight": sd["model.norm.weight"],
          "lm_head.weight": sd["lm_head.weight"]}
    for i in range(L):
        p, r = f"model.layers.{i}.", f"transformer.h.{i}."
        for suffix in ("weight", "bias"):
            st[r + "attn.c_attn." + suffix] = torch.cat([sd[p + f"self_attn.{n}_proj.{suffix}"] for n in "qkv"], dim=0)
        st[r + "attn.c_proj.weight"] = sd[p + "self_attn.o_proj.weight"]
        st[r + "mlp.w1.weight"] = sd[p + "mlp.up_proj.weight"]          # a1 * silu(a2): w2 is the gate
        st[r + "mlp.w2.weight"] = sd[p + "mlp.gate_proj.weight"]
        st[r + "mlp.c_proj.weight"] = sd[p + "mlp.down_proj.weight"]
        st[r + "ln_1.weight"] = sd[p + "input_layernorm.weight"]
        st[r + "ln_2.weight"] = sd[p + "post_attention_layernorm.weight"]
    cfg = {"model_type": "qwen", "vocab_size": 1000, "hidden_size": H, "intermediate_size": 2 * I,
           "num_hidden_layers": L, "num_attention_heads": 4, "kv_channels": 32, "layer_norm_epsilon": 1e-6,
           "rotary_emb_base": 10000, "seq_length": 256, "no_bias": True, "torch_dtype": "float32"}
    _check(_save(tmp_path, cfg, st), native)


def test_minicpm_checkpoint_loads_as_granite(tmp_path):
    from transformers import GraniteConfig
    H, L, nh = 128, 2, 4
    scale_emb, scale_depth, dim_model_base = 12.0, 1.4, 64
    native = _native(GraniteConfig(vocab_size=1000, hidden_size=H, intermediate_size=256, num_hidden_layers=L,
                                   num_attention_heads=nh, num_key_value_heads=nh, max_position_embeddings=256,
                                   rms_norm_eps=1e-5, embedding_multiplier=scale_emb,
                                   residual_multiplier=scale_depth / math.sqrt(L), logits_scaling=H / dim_model_base,
                                   attention_multiplier=1.0 / math.sqrt(H // nh), tie_word_embeddings=False))
    native.lm_head.weight.data = native.model.embed_tokens.weight.data.clone()     # tied output layer
    st = {k: v for k, v in native.state_dict().items() if k != "lm_head.weight"}
    cfg = {"model_type": "minicpm", "vocab_size": 1000, "hidden_size": H, "intermediate_size": 256,
           "num_hidden_layers": L, "num_attention_heads": nh, "num_key_value_heads": nh, "rms_norm_eps": 1e-5,
           "scale_emb": scale_emb, "scale_depth": scale_depth, "dim_model_base": dim_model_base,
           "max_position_embeddings": 256, "torch_dtype": "float32"}
    _check(_save(tmp_path, cfg, st), native)


def test_minicpm3_checkpoint_loads_as_dense_deepseek_v2(tmp_path):
    """MiniCPM3 (reference models/minicpm3.py:116-230): latent attention with half-split rotary on the rope block,
    LongRoPE factors, and the embedding / residual / logit multipliers.  The checkpoint is random; the expected logits
    come from a plain restatement of that architecture, written independently of the mapping."""
    from ipex_llm.transformers import AutoModelForCausalLM
    torch.manual_seed(0)
    V, H, I, L, nh = 300, 64, 128, 2, 4
    nope, rope_d, qr, kvr = 16, 8, 24, 16
    vd = H // nh
    qk = nope + rope_d
    scale_emb, scale_depth, dmb, eps, theta, orig = 12.0, 1.4, 16, 1e-5, 10000.0, 32
    short = [1.0 + 0.1 * i for i in range(rope_d // 2)]
    long = [2.0 + 0.5 * i for i in range(rope_d // 2)]
    st = {"model.embed_tokens.weight": torch.randn(V, H) * 0.1, "model.norm.weight": 1 + 0.1 * torch.randn(H)}
    for i in range(L):
        p = f"model.layers.{i}."
        st.update({p + "input_layernorm.weight": 1 + 0.1 * torch.randn(H),
                   p + "post_attention_layernorm.weight": 1 + 0.1 * torch.randn(H),
                   p + "self_attn.q_a_proj.weight": torch.randn(qr, H) * 0.1,
                   p + "self_attn.q_a_layernorm.weight": 1 + 0.1 * torch.randn(qr),
                   p + "self_attn.q_b_proj.weight": torch.randn(nh * qk, qr) * 0.2,
                   p + "self_attn.kv_a_proj_with_mqa.weight": torch.randn(kvr + rope_d, H) * 0.1,
                   p + "self_attn.kv_a_layernorm.weight": 1 + 0.1 * torch.randn(kvr),
                   p + "self_attn.kv_b_proj.weight": torch.randn(nh * (nope + vd), kvr) * 0.2,
                   p + "self_attn.o_proj.weight": torch.randn(H, nh * vd) * 0.1,
                   p + "mlp.gate_proj.weight": torch.randn(I, H) * 0.1, p + "mlp.up_proj.weight": torch.randn(I, H) * 0.1,
                   p + "mlp.down_proj.weight": torch.randn(H, I) * 0.1})
    cfg = {"model_type": "minicpm3", "vocab_size": V, "hidden_size": H, "intermediate_size": I, "num_hidden_layers": L,
           "num_attention_heads": nh, "num_key_value_heads": nh, "q_lora_rank": qr, "kv_lora_rank": kvr,
           "qk_nope_head_dim": nope, "qk_rope_head_dim": rope_d, "rms_norm_eps": eps, "scale_emb": scale_emb,
           "scale_depth": scale_depth, "dim_model_base": dmb, "max_position_embeddings": 128, "rope_theta": theta,
           "rope_scaling": {"type": "longrope", "short_factor": short, "long_factor": long,
                            "original_max_position_embeddings": orig}, "torch_dtype": "float32"}
    d = _save(tmp_path, cfg, st)

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def rot_half(x):
        a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat((-b, a), dim=-1)

    def plain(ids):
        B, S = ids.shape
        ext = torch.tensor(long if S > orig else short)
        inv = 1.0 / (ext * theta ** (torch.arange(0, rope_d, 2).float() / rope_d))
        ang = torch.outer(torch.arange(S).float(), inv)
        mscale = math.sqrt(1 + math.log(128 / orig) / math.log(orig))
        cos, sin = torch.cat((ang, ang), -1).cos() * mscale, torch.cat((ang, ang), -1).sin() * mscale
        x = st["model.embed_tokens.weight"][ids] * scale_emb
        causal = torch.full((S, S), float("-inf")).triu(1)
        for i in range(L):
            p = f"model.layers.{i}."
            h = rms(x, st[p + "input_layernorm.weight"])
            q = rms(h @ st[p + "self_attn.q_a_proj.weight"].t(), st[p + "self_attn.q_a_layernorm.weight"])
            q = (q @ st[p + "self_attn.q_b_proj.weight"].t()).view(B, S, nh, qk).transpose(1, 2)
            q_nope, q_pe = q.split([nope, rope_d], -1)
            ckv = h @ st[p + "self_attn.kv_a_proj_with_mqa.weight"].t()
            ckv, k_pe = ckv.split([kvr, rope_d], -1)
            k_pe = k_pe.view(B, S, 1, rope_d).transpose(1, 2)
            kv = (rms(ckv, st[p + "self_attn.kv_a_layernorm.weight"]) @ st[p + "self_attn.kv_b_proj.weight"].t())
            kv = kv.view(B, S, nh, nope + vd).transpose(1, 2)
            k_nope, v = kv.split([nope, vd], -1)
            q_pe = q_pe * cos + rot_half(q_pe) * sin
            k_pe = k_pe * cos + rot_half(k_pe) * sin
            qf = torch.cat((q_nope, q_pe), -1)
            kf = torch.cat((k_nope, k_pe.expand(B, nh, S, rope_d)), -1)
            a = torch.softmax(qf @ kf.transpose(-1, -2) / math.sqrt(qk) + causal, -1) @ v
            a = a.transpose(1, 2).reshape(B, S, nh * vd) @ st[p + "self_attn.o_proj.weight"].t()
            x = x + a * (scale_depth / math.sqrt(L))
            h = rms(x, st[p + "post_attention_layernorm.weight"])
            m = torch.nn.functional.silu(h @ st[p + "mlp.gate_proj.weight"].t()) * (h @ st[p + "mlp.up_proj.weight"].t())
            x = x + (m @ st[p + "mlp.down_proj.weight"].t()) * (scale_depth / math.sqrt(L))
        x = rms(x, st["model.norm.weight"])
        return (x / (H / dmb)) @ st["model.embed_tokens.weight"].t()           # tied output layer

    m = AutoModelForCausalLM.from_pretrained(d)
    assert m.config.model_type == "deepseek_v2" and m.config.ipex_remote_model_type == "minicpm3"
    for n in (12, 40):                                   # below and above the LongRoPE switch point
        ids = torch.randint(0, V, (2, n))
        with torch.no_grad():
            got, want = m(ids).logits, plain(ids)
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (n, (got - want).abs().max())
    q8 = AutoModelForCausalLM.from_pretrained(d, load_in_low_bit="sym_int8")
    ids = torch.randint(0, V, (2, 12))
    with torch.no_grad():
        lq = q8(ids).logits[:, -1]
    assert torch.nn.functional.cosine_similarity(lq.float(), plain(ids)[:, -1], dim=-1).min() > 0.99
    # generation across the switch point rebuilds the cache with the long factors (as for Phi-3)
    ids = torch.randint(0, V, (1, 29))
    out = q8.generate(ids, max_new_tokens=8, do_sample=False)
    cur = ids
    with torch.no_grad():
        for _ in range(8):
            cur = torch.cat([cur, q8(cur).logits[:, -1].argmax(-1, keepdim=True)], 1)
    assert torch.equal(out, cur)


def test_uncovered_variants_fall_through():
    from ipex_llm_b200.transformers.remote_archs import REMOTE_ARCHS
    assert REMOTE_ARCHS["chatglm"]({"model_type": "chatglm", "position_encoding_2d": True}) is None      # ChatGLM-6B v1
