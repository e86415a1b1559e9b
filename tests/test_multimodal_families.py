"""Vision- and audio-language families (reference models/qwen2_vl.py, internvl.py, janus.py, mllama.py, chatglm4v.py,
whisper.py and the multimodal branches of convert.py:1303-2040): tiny random models go through ``optimize_model``;
the converted model must reproduce the fp32 one on text-only input, on input with an image / audio clip, and decode
incrementally through the package's caches."""
import copy

import pytest
import torch
import transformers as T

TXT = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           vocab_size=1000, max_position_embeddings=256)
MROPE = {"rope_type": "default", "mrope_section": [4, 6, 6], "rope_theta": 10000.0}
IMG, PATCH = 998, 3 * 2 * 14 * 14


def _qwen2_vl():
    cfg = T.Qwen2VLConfig(
        text_config=dict(TXT, rope_parameters=MROPE),
        vision_config=dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, patch_size=14, spatial_merge_size=2,
                           temporal_patch_size=2, in_channels=3, mlp_ratio=2),
        image_token_id=IMG, video_token_id=999, vision_start_token_id=997, vision_end_token_id=996)
    return cfg, T.Qwen2VLForConditionalGeneration


def _qwen2_5_vl():
    cfg = T.Qwen2_5_VLConfig(
        text_config=dict(TXT, rope_parameters=MROPE),
        vision_config=dict(depth=2, hidden_size=64, out_hidden_size=128, intermediate_size=128, num_heads=4,
                           patch_size=14, spatial_merge_size=2, temporal_patch_size=2, in_channels=3,
                           fullatt_block_indexes=[1], window_size=56),
        image_token_id=IMG, video_token_id=999, vision_start_token_id=997, vision_end_token_id=996)
    return cfg, T.Qwen2_5_VLForConditionalGeneration


def _glm4v():
    cfg = T.Glm4vConfig(
        text_config=dict(TXT, rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3],
                                               "rope_theta": 10000.0, "partial_rotary_factor": 0.5}),
        vision_config=dict(depth=2, hidden_size=64, out_hidden_size=128, intermediate_size=128, num_heads=4,
                           patch_size=14, spatial_merge_size=2, temporal_patch_size=2, image_size=56),
        image_token_id=IMG, video_token_id=999)
    return cfg, T.Glm4vForConditionalGeneration


def _internvl():
    cfg = T.InternVLConfig(
        text_config=dict(TXT, model_type="qwen2"),
        vision_config=dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                           image_size=[28, 28], patch_size=[14, 14]), image_token_id=IMG)
    return cfg, T.InternVLForConditionalGeneration


def _janus():
    cfg = T.JanusConfig(
        text_config=dict(TXT, model_type="llama"),
        vision_config=dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                           image_size=28, patch_size=14, projection_dim=128, depth=1),
        vq_config=dict(embed_dim=8, num_embeddings=64, base_channels=32, channel_multiplier=[1, 1], num_res_blocks=1,
                       projection_dim=128, image_token_embed_dim=32, num_patches=4, latent_channels=8),
        image_token_id=IMG)
    return cfg, T.JanusForConditionalGeneration


def _mllama():
    cfg = T.MllamaConfig(
        text_config=dict(TXT, cross_attention_layers=[1], pad_token_id=0,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0}),
        vision_config=dict(hidden_size=64, num_hidden_layers=2, num_global_layers=1, attention_heads=4,
                           intermediate_size=128, image_size=28, patch_size=14, vision_output_dim=128,
                           intermediate_layers_indices=[0], max_num_tiles=1, supported_aspect_ratios=[[1, 1]]),
        image_token_index=IMG)
    return cfg, T.MllamaForConditionalGeneration


def _qwen2_audio():
    cfg = T.Qwen2AudioConfig(
        text_config=dict(TXT, model_type="qwen2"),
        audio_config=dict(d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128,
                          num_mel_bins=16, max_source_positions=50), audio_token_index=IMG)
    return cfg, T.Qwen2AudioForConditionalGeneration


def _media_inputs(name):
    """Model inputs with one image (or one audio clip) spliced into a random prompt; None when the family is only
    exercised on text here."""
    ids = torch.randint(0, 900, (1, 20))
    if name in ("qwen2_vl", "qwen2_5_vl", "glm4v"):
        ids[0, 3:7] = IMG                                           # 4 x 4 patches, merged 2 x 2 -> 4 tokens
        kw = dict(input_ids=ids, pixel_values=torch.randn(16, PATCH), image_grid_thw=torch.tensor([[1, 4, 4]]))
        if name != "qwen2_5_vl":
            mm = torch.zeros_like(ids)
            mm[0, 3:7] = 1
            kw["mm_token_type_ids"] = mm
        return kw
    if name == "internvl":
        ids[0, 3:4] = IMG
        return dict(input_ids=ids, pixel_values=torch.randn(1, 3, 28, 28))
    if name == "mllama":
        return dict(input_ids=ids, pixel_values=torch.randn(1, 1, 1, 3, 28, 28), aspect_ratio_ids=torch.tensor([[1]]),
                    aspect_ratio_mask=torch.ones(1, 1, 1, dtype=torch.long),
                    cross_attention_mask=torch.ones(1, 20, 1, 1, dtype=torch.long))
    if name == "qwen2_audio":
        ids = torch.randint(0, 900, (1, 40))
        ids[0, 3:28] = IMG                                          # 100 mel frames -> 25 audio tokens
        return dict(input_ids=ids, input_features=torch.randn(1, 16, 100),
                    feature_attention_mask=torch.ones(1, 100, dtype=torch.long),
                    attention_mask=torch.ones(1, 40, dtype=torch.long))
    return None


CASES = {"qwen2_vl": _qwen2_vl, "qwen2_5_vl": _qwen2_5_vl, "glm4v": _glm4v, "internvl": _internvl, "janus": _janus,
         "mllama": _mllama, "qwen2_audio": _qwen2_audio}


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().float(), b.flatten().float(), dim=0).item()


@pytest.mark.parametrize("name", list(CASES))
def test_multimodal_family_converts_and_matches(name):
    from ipex_llm import optimize_model
    from ipex_llm_b200.ops.linear import LowBitLinear
    try:
        cfg, cls = CASES[name]()
    except (TypeError, ValueError, AttributeError) as e:               # a transformers release with another config
        pytest.skip(f"{name}: tiny config not accepted by this transformers ({e})")
    torch.manual_seed(0)
    base = cls(cfg).eval()
    low = optimize_model(copy.deepcopy(base), low_bit="sym_int8")
    assert sum(isinstance(m, LowBitLinear) for m in low.modules()) >= 20       # towers and language model alike
    ids = torch.randint(0, 900, (2, 20))
    with torch.no_grad():
        assert _cos(low(input_ids=ids).logits[:, -1], base(input_ids=ids).logits[:, -1]) > 0.999
    out = low.generate(input_ids=ids, max_new_tokens=4, do_sample=False)
    with torch.no_grad():
        full = low(input_ids=out[:, :-1]).logits[:, -1].argmax(-1)
    assert torch.equal(full, out[:, -1])
    media = _media_inputs(name)
    if media is not None:
        with torch.no_grad():
            assert _cos(low(**media).logits[:, -1], base(**media).logits[:, -1]) > 0.999
    # the packed model reloads into a shell built without allocating weights and answers the same, bit for bit
    # (vision rotary tables and the like are rebuilt, they are in no checkpoint)
    import tempfile
    from ipex_llm.optimize import load_low_bit, low_memory_init
    with tempfile.TemporaryDirectory() as d:
        low.save_low_bit(d)
        with low_memory_init():
            shell = cls(cfg)
        again = load_low_bit(shell, d)
    with torch.no_grad():
        assert torch.equal(again(input_ids=ids).logits, low(input_ids=ids).logits)
        if media is not None:
            assert torch.equal(again(**media).logits, low(**media).logits)

