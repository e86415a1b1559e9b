"""GGUF import: write a tiny llama-shaped file (f32 / f16 / q8_0 / q4_0 tensors), read it back, compare with the
source model."""
import numpy as np
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
