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


def _interface_models():
    import transformers as tf
    return {
        "bert": lambda: tf.BertModel(tf.BertConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                                   intermediate_size=256, vocab_size=500)),
        "whisper": lambda: tf.WhisperForConditionalGeneration(tf.WhisperConfig(
            d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4, decoder_attention_heads=4,
            encoder_ffn_dim=256, decoder_ffn_dim=256, vocab_size=500, num_mel_bins=16, max_source_positions=32,
            max_target_positions=64, pad_token_id=0, bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)),
        "deepseek_v3": lambda: tf.DeepseekV3ForCausalLM(tf.DeepseekV3Config(
            hidden_size=128, intermediate_size=256, moe_intermediate_size=128, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=4, n_routed_experts=4, n_shared_experts=1,
            num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, kv_lora_rank=32, q_lora_rank=64,
            qk_rope_head_dim=16, qk_nope_head_dim=32, v_head_dim=32, vocab_size=500, max_position_embeddings=128)),
        "qwen2_vl_text": lambda: tf.AutoModelForCausalLM.from_config(tf.Qwen2Config(
            hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, vocab_size=500)),
    }


@pytest.mark.parametrize("name", ["bert", "whisper", "deepseek_v3"])
def test_attention_interface_serves_families_without_their_own_forward(name, monkeypatch):
    """Encoders, encoder-decoders with cross-attention and MLA attention reach the package's SDPA through the
    transformers attention-interface registry (no per-family forward), and the converted model matches the original."""
    import copy
    from ipex_llm import optimize_model
    from ipex_llm_b200.models import common
    torch.manual_seed(0)
    model = _interface_models()[name]().eval()
    calls = {"n": 0, "non_causal": 0}
    real = common.scaled_dot_product_attention

    def counting(*a, **k):
        calls["n"] += 1
        if not k.get("is_causal", False):
            calls["non_causal"] += 1
        return real(*a, **k)

    monkeypatch.setattr(common, "scaled_dot_product_attention", counting)
    if name == "bert":
        kw = dict(input_ids=torch.randint(0, 500, (2, 12)))
        pick = lambda o: o.last_hidden_state
    elif name == "whisper":
        kw = dict(input_features=torch.randn(2, 16, 64), decoder_input_ids=torch.randint(3, 500, (2, 6)))
        pick = lambda o: o.logits
    else:
        kw = dict(input_ids=torch.randint(0, 500, (2, 12)))
        pick = lambda o: o.logits[:, -1]          # the converted lm_head scores only the last position of a prompt
    with torch.no_grad():
        ref = pick(model(**kw)).float()
    q = optimize_model(copy.deepcopy(model), low_bit="sym_int8")
    with torch.no_grad():
        out = pick(q(**kw)).float()
    assert calls["n"] > 0, "the attention interface was not used"
    if name in ("bert", "whisper"):
        assert calls["non_causal"] > 0          # bidirectional / cross attention must not be made causal
    cos = torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0).item()
    assert cos > 0.995, (name, cos)


AUTO_CASES = ["AutoModel", "AutoModelForMaskedLM", "AutoModelForSequenceClassification",
              "AutoModelForTokenClassification", "AutoModelForQuestionAnswering", "AutoModelForNextSentencePrediction",
              "AutoModelForMultipleChoice", "AutoModelForSeq2SeqLM", "AutoModelForSpeechSeq2Seq"]


@pytest.mark.parametrize("auto", AUTO_CASES)
def test_every_auto_class_converts_saves_and_reloads(auto, tmp_path):
    """The Auto classes of the reference's API (model.py:788-830) beyond causal LM, on tiny BERT / T5 / Whisper
    models: low-bit conversion keeps the outputs, ``save_low_bit`` / ``load_low_bit`` reproduce them bit for bit.
    Covers a masked-LM decoder (every position of its output is used, so it is not treated as a generative head),
    BERT's position-id buffers (in no checkpoint), T5's tied output layer and its feed-forward, which casts
    activations to the weight's dtype."""
    import transformers
    import ipex_llm.transformers as IT
    from ipex_llm_b200.ops.linear import LowBitLinear
    bert = transformers.BertConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                   vocab_size=500, max_position_embeddings=64)
    t5 = transformers.T5Config(d_model=128, d_ff=256, d_kv=32, num_layers=2, num_heads=4, vocab_size=500,
                               decoder_start_token_id=0)
    wh = transformers.WhisperConfig(d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                                    decoder_attention_heads=4, encoder_ffn_dim=256, decoder_ffn_dim=256,
                                    num_mel_bins=16, max_source_positions=50, max_target_positions=64, vocab_size=500,
                                    decoder_start_token_id=1, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    ids = torch.randint(0, 500, (2, 12))
    table = {
        "AutoModel": ("BertModel", bert, dict(input_ids=ids), "last_hidden_state"),
        "AutoModelForMaskedLM": ("BertForMaskedLM", bert, dict(input_ids=ids), "logits"),
        "AutoModelForSequenceClassification": ("BertForSequenceClassification", bert, dict(input_ids=ids), "logits"),
        "AutoModelForTokenClassification": ("BertForTokenClassification", bert, dict(input_ids=ids), "logits"),
        "AutoModelForQuestionAnswering": ("BertForQuestionAnswering", bert, dict(input_ids=ids), "start_logits"),
        "AutoModelForNextSentencePrediction": ("BertForNextSentencePrediction", bert, dict(input_ids=ids), "logits"),
        "AutoModelForMultipleChoice": ("BertForMultipleChoice", bert, dict(input_ids=ids.view(1, 2, 12)), "logits"),
        "AutoModelForSeq2SeqLM": ("T5ForConditionalGeneration", t5,
                                  dict(input_ids=ids, decoder_input_ids=ids[:, :5]), "logits"),
        "AutoModelForSpeechSeq2Seq": ("WhisperForConditionalGeneration", wh,
                                      dict(input_features=torch.randn(2, 16, 100), decoder_input_ids=ids[:, :5]),
                                      "logits"),
    }
    hf_name, cfg, inputs, field = table[auto]
    torch.manual_seed(0)
    src = getattr(transformers, hf_name)(cfg).eval()
    d0, d1 = str(tmp_path / "hf"), str(tmp_path / "low")
    src.save_pretrained(d0)
    cls = getattr(IT, auto)
    low = cls.from_pretrained(d0, load_in_low_bit="sym_int8")
    assert sum(isinstance(x, LowBitLinear) for x in low.modules()) >= 12
    with torch.no_grad():
        a, ref = getattr(low(**inputs), field), getattr(src(**inputs), field)
    assert a.shape == ref.shape
    assert torch.nn.functional.cosine_similarity(a.flatten().float(), ref.flatten().float(), dim=0) > 0.999
    low.save_low_bit(d1)
    again = cls.load_low_bit(d1)
    with torch.no_grad():
        assert torch.equal(getattr(again(**inputs), field), a)


@pytest.mark.parametrize("kind", ["t5", "bart", "whisper"])
def test_encoder_decoder_generation_through_the_package_generate(kind, tmp_path):
    """``generate`` of encoder-decoder models goes through the package's wrapper to transformers' own loop (Whisper's
    override tests for the presence of keywords, so only what the caller gave may be forwarded); greedy tokens equal
    those of the unconverted model."""
    import transformers
    import ipex_llm.transformers as IT
    ids = torch.randint(3, 500, (2, 12))
    if kind == "t5":
        cfg = transformers.T5Config(d_model=128, d_ff=256, d_kv=32, num_layers=2, num_heads=4, vocab_size=500,
                                    decoder_start_token_id=0, eos_token_id=1, pad_token_id=0)
        hf, auto, inputs = "T5ForConditionalGeneration", "AutoModelForSeq2SeqLM", dict(input_ids=ids)
    elif kind == "bart":
        cfg = transformers.BartConfig(d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                                      decoder_attention_heads=4, encoder_ffn_dim=256, decoder_ffn_dim=256,
                                      vocab_size=500, max_position_embeddings=64, pad_token_id=1, bos_token_id=0,
                                      eos_token_id=2, decoder_start_token_id=2)
        hf, auto, inputs = "BartForConditionalGeneration", "AutoModelForSeq2SeqLM", dict(input_ids=ids)
    else:
        cfg = transformers.WhisperConfig(d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                                         decoder_attention_heads=4, encoder_ffn_dim=256, decoder_ffn_dim=256,
                                         num_mel_bins=16, max_source_positions=50, max_target_positions=64,
                                         vocab_size=500, decoder_start_token_id=1, pad_token_id=0, bos_token_id=1,
                                         eos_token_id=2)
        hf, auto = "WhisperForConditionalGeneration", "AutoModelForSpeechSeq2Seq"
        inputs = dict(input_features=torch.randn(2, 16, 100))
    torch.manual_seed(0)
    src = getattr(transformers, hf)(cfg).eval()
    src.generation_config.max_length = 64
    d = str(tmp_path / "hf")
    src.save_pretrained(d)
    low = getattr(IT, auto).from_pretrained(d, load_in_low_bit="bf16", torch_dtype=torch.float32)
    ref = src.generate(**inputs, max_new_tokens=8, do_sample=False, num_beams=1)
    out = low.generate(**inputs, max_new_tokens=8, do_sample=False, num_beams=1)
    assert out.shape == ref.shape and torch.equal(out, ref)
