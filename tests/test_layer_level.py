"""Layer-level numerics the way the reference checks them (python/llm/test/inference_gpu/
test_transformers_api_attention.py:37-183, _mlp.py, _RMSNorm.py): capture the input of one layer's attention / MLP /
norm in the unoptimized model with a forward pre-hook, feed it to the same layer of the optimized model, compare."""
import copy

import pytest
import torch


def _tiny():
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256, tie_word_embeddings=False)
    m = LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
    return m


@pytest.mark.parametrize("layer_attr,bound", [("self_attn", 5e-2), ("mlp", 5e-2), ("input_layernorm", 1e-4)])
def test_layer_output_matches_unoptimized(layer_attr, bound):
    from ipex_llm import optimize_model
    ref = _tiny()
    opt = optimize_model(copy.deepcopy(ref), low_bit="sym_int8")
    ids = torch.randint(0, 1000, (1, 24))
    captured = {}

    def pre_hook(module, args, kwargs):
        captured["args"], captured["kwargs"] = args, kwargs

    def post_hook(module, args, kwargs, output):
        captured["out"] = output[0] if isinstance(output, tuple) else output

    layer = getattr(ref.model.layers[-1], layer_attr)
    h1 = layer.register_forward_pre_hook(pre_hook, with_kwargs=True)
    h2 = layer.register_forward_hook(post_hook, with_kwargs=True)
    with torch.no_grad():
        ref(ids)
    h1.remove()
    h2.remove()
    opt_layer = getattr(opt.model.layers[-1], layer_attr)
    kwargs = dict(captured["kwargs"])
    kwargs.pop("past_key_values", None)
    kwargs.pop("past_key_value", None)
    with torch.no_grad():
        out = opt_layer(*captured["args"], **kwargs)
    out = out[0] if isinstance(out, tuple) else out
    diff = (out.float() - captured["out"].float()).abs().max().item()
    assert diff <= bound * max(1.0, captured["out"].abs().max().item()), (layer_attr, diff)


def test_whisper_tiny_converts():
    """optimize_model on an encoder-decoder speech model (reference test_optimize_model_api.py:23-40)."""
    from transformers import WhisperConfig, WhisperForConditionalGeneration
    from ipex_llm import optimize_model
    from ipex_llm.transformers.low_bit_linear import LowBitLinear
    torch.manual_seed(0)
    cfg = WhisperConfig(d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                        decoder_attention_heads=4, encoder_ffn_dim=256, decoder_ffn_dim=256, vocab_size=600,
                        num_mel_bins=16, max_source_positions=50, max_target_positions=32,
                        decoder_start_token_id=1, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    model = WhisperForConditionalGeneration(cfg).eval()
    feats = torch.randn(1, 16, 100)
    dec = torch.tensor([[1, 5, 7]])
    with torch.no_grad():
        ref = model(input_features=feats, decoder_input_ids=dec).logits
    opt = optimize_model(model, low_bit="sym_int8")
    assert sum(isinstance(m, LowBitLinear) for m in opt.modules()) >= 16
    with torch.no_grad():
        out = opt(input_features=feats, decoder_input_ids=dec).logits
    cos = torch.nn.functional.cosine_similarity(out.flatten().float(), ref.flatten(), dim=0).item()
    assert cos > 0.99, cos


def test_left_padding_masks_are_recognised():
    """The dispatcher of the prompt attention reduces a 4-D mask to "first real token per row" when (and only when)
    the mask is exactly a left-padding mask, causal or not, with or without a sliding window."""
    import torch
    from ipex_llm_b200.ops.cuda_ops import left_pad_mask_bounds
    S = 40
    qi, ki = torch.arange(S).view(1, S, 1), torch.arange(S).view(1, 1, S)
    lo = torch.tensor([0, 7, 25])
    for causal, window in ((True, 0), (True, 9), (False, 0)):
        ok = (ki >= lo.view(-1, 1, 1)).expand(3, S, S)
        if causal:
            ok = ok & (ki <= qi)
        if window:
            ok = ok & (ki > qi - window)
        ok = ok.clone()
        ok[1, :7] = True                           # rows of padding queries may hold anything
        for mask in (ok.unsqueeze(1), torch.zeros(3, 1, S, S).masked_fill(~ok.unsqueeze(1), float("-inf"))):
            found = left_pad_mask_bounds(mask, S, window)
            assert found is not None and found[0].tolist() == lo.tolist() and found[1] == causal
    holed = (ki <= qi).expand(1, S, S).clone()
    holed[0, 30, 10] = False
    assert left_pad_mask_bounds(holed.unsqueeze(1), S) is None


def test_mask_recognition_is_exact_for_every_fill_value_and_rejects_biases():
    """An additive mask may mark hidden keys with -inf, its dtype's minimum, another dtype's minimum or the -10000 of
    older models: all are recognised with the same bounds.  Masks that carry a bias (ALiBi) and masks that differ from
    a left-padding mask in one element are refused, so they take the generic path instead of the wrong kernel mode."""
    import random
    from ipex_llm_b200.ops.cuda_ops import left_pad_mask_bounds
    S = 24
    qi, ki = torch.arange(S).view(1, S, 1), torch.arange(S).view(1, 1, S)
    lo = torch.tensor([0, 9])
    ok = ((ki >= lo.view(-1, 1, 1)) & (ki <= qi))
    for fill in (float("-inf"), torch.finfo(torch.float32).min, float(torch.finfo(torch.float16).min), -10000.0):
        mask = torch.zeros(2, 1, S, S).masked_fill(~ok.unsqueeze(1), fill)
        found = left_pad_mask_bounds(mask, S)
        assert found is not None and found[0].tolist() == [0, 9] and found[1] is True, fill
    alibi = torch.zeros(2, 1, S, S).masked_fill(~ok.unsqueeze(1), float("-inf")) - 0.01 * (qi - ki).clamp_min(0).float()
    assert left_pad_mask_bounds(alibi, S) is None
    rnd = random.Random(0)
    for _ in range(200):                               # one flipped element: refused, or the flip sits in a padding row
        b, r, c = rnd.randrange(2), rnd.randrange(S), rnd.randrange(S)
        m = ok.clone()
        m[b, r, c] = ~m[b, r, c]
        found = left_pad_mask_bounds(m.unsqueeze(1), S)
        if found is not None:
            got = (ki >= found[0].view(-1, 1, 1).long())
            if found[1]:
                got = got & (ki <= qi)
            real = qi >= found[0].view(-1, 1, 1).long()
            assert bool(((got == m) | ~real).all()), (b, r, c)
