"""Families without a dedicated forward file: low-bit linears (Conv1D included) + fused LayerNorm registration."""
import pytest
import torch


def _configs():
    import transformers as tf
    return {
        "gpt_neox": tf.GPTNeoXConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                     num_attention_heads=4, vocab_size=500, max_position_embeddings=128),
        "bloom": tf.BloomConfig(hidden_size=128, n_layer=2, n_head=4, vocab_size=500),
        "falcon": tf.FalconConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=500),
        "mpt": tf.MptConfig(d_model=128, n_layers=2, n_heads=4, vocab_size=500, max_seq_len=128),
        "phi": tf.PhiConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                            vocab_size=500),
        "opt": tf.OPTConfig(hidden_size=128, ffn_dim=256, num_hidden_layers=2, num_attention_heads=4, vocab_size=500,
                            word_embed_proj_dim=128, max_position_embeddings=128),
        "gpt2": tf.GPT2Config(n_embd=128, n_layer=2, n_head=4, vocab_size=500, n_positions=128),
        "gpt_bigcode": tf.GPTBigCodeConfig(n_embd=128, n_layer=2, n_head=4, vocab_size=500, n_positions=128),
    }


@pytest.mark.parametrize("name", ["gpt_neox", "bloom", "falcon", "mpt", "phi", "opt", "gpt2", "gpt_bigcode"])
def test_generic_family_converts_and_matches(name):
    import transformers as tf
    from ipex_llm import optimize_model
    from ipex_llm_b200.models.registry import FAMILIES
    from ipex_llm_b200.ops.linear import LowBitLinear
    torch.manual_seed(0)
    model = tf.AutoModelForCausalLM.from_config(_configs()[name]).eval()
    ids = torch.randint(0, 500, (2, 16))
    with torch.no_grad():
        ref = model(ids).logits[:, -1].float()
    q = optimize_model(model, low_bit="sym_int8")
    n_low = sum(1 for m in q.modules() if isinstance(m, LowBitLinear))
    assert n_low >= 9, n_low            # every projection of both blocks + lm_head, GPT-2's Conv1D included
    assert name in FAMILIES
    with torch.no_grad():
        out = q(ids).logits[:, -1].float()
    cos = torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0).item()
    assert cos > 0.999, cos
    toks = q.generate(ids, max_new_tokens=4, do_sample=False)
    assert toks.shape == (2, 20)
