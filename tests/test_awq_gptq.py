"""Pre-quantized checkpoints: write tiny AWQ (AutoAWQ gemm layout) and GPTQ (AutoGPTQ v1 layout) checkpoints of a
random Llama, load them through ``from_pretrained(load_in_4bit=True)`` and compare with the dequantized source."""
import json
import os

import pytest
import torch

GROUP = 64


def _tiny():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=320, max_position_embeddings=128, tie_word_embeddings=False)
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
    return cfg, m


def _quant_params(w):
    """asymmetric 4-bit per (group of 64 inputs, output): returns codes [in, out], scales, zeros [in/g, out]."""
    wt = w.float().t().contiguous()                        # [in, out]
    g = wt.view(-1, GROUP, wt.shape[1])
    mx, mn = g.max(dim=1).values, g.min(dim=1).values
    scales = ((mx - mn).clamp(min=1e-5) / 15).half().float()
    zeros = torch.clamp(torch.round(-mn / scales), 0, 15)
    s = scales.repeat_interleave(GROUP, dim=0)
    z = zeros.repeat_interleave(GROUP, dim=0)
    codes = torch.clamp(torch.round(wt / s + z), 0, 15)
    deq = ((codes - z) * s).t().contiguous()               # [out, in]
    return codes.to(torch.int32), scales, zeros.to(torch.int32), deq


def _write(tmp, cfg, model, method):
    from ipex_llm_b200.transformers.awq.linear import AWQ_ORDER
    sd = {}
    ref = {k: v.clone() for k, v in model.state_dict().items()}
    for name, mod in model.named_modules():
        if isinstance(mod, torch.nn.Linear) and "layers." in name:
            codes, scales, zeros, deq = _quant_params(mod.weight.data)
            ref[name + ".weight"] = deq
            if method == "awq":
                qw = torch.zeros((codes.shape[0], codes.shape[1] // 8), dtype=torch.int32)
                qz = torch.zeros((zeros.shape[0], zeros.shape[1] // 8), dtype=torch.int32)
                for j, pos in enumerate(AWQ_ORDER):
                    qw |= codes[:, j::8] << (4 * pos)
                    qz |= zeros[:, j::8] << (4 * pos)
            else:
                qw = torch.zeros((codes.shape[0] // 8, codes.shape[1]), dtype=torch.int32)
                for j in range(8):
                    qw |= codes[j::8, :] << (4 * j)
                zm1 = zeros - 1                                # AutoGPTQ v1 stores zero - 1
                qz = torch.zeros((zeros.shape[0], zeros.shape[1] // 8), dtype=torch.int32)
                for j in range(8):
                    qz |= (zm1[:, j::8] & 0xF) << (4 * j)
                sd[name + ".g_idx"] = (torch.arange(codes.shape[0]) // GROUP).to(torch.int32)
            sd[name + ".qweight"], sd[name + ".qzeros"], sd[name + ".scales"] = qw, qz, scales.half()
        elif isinstance(mod, (torch.nn.Linear, torch.nn.Embedding)) or name.endswith("norm"):
            for pn, p in mod.named_parameters(recurse=False):
                sd[f"{name}.{pn}"] = p.data.clone()
    for k, v in model.state_dict().items():
        if "norm" in k:
            sd[k] = v.clone()
    os.makedirs(tmp, exist_ok=True)
    torch.save(sd, os.path.join(tmp, "pytorch_model.bin"))
    c = cfg.to_dict()
    if method == "awq":
        c["quantization_config"] = {"quant_method": "awq", "bits": 4, "group_size": GROUP, "version": "gemm",
                                    "zero_point": True, "backend": "autoawq"}
    else:
        c["quantization_config"] = {"quant_method": "gptq", "bits": 4, "group_size": GROUP, "desc_act": False,
                                    "sym": False}
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(c, f)
    return ref


@pytest.mark.parametrize("method", ["awq", "gptq"])
def test_load_prequantized_checkpoint(tmp_path, method):
    from transformers import LlamaForCausalLM
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.ops.linear import LowBitLinear
    cfg, src = _tiny()
    ref_sd = _write(str(tmp_path / method), cfg, src, method)
    ref = LlamaForCausalLM(cfg).eval()
    ref.load_state_dict(ref_sd)
    model = AutoModelForCausalLM.from_pretrained(str(tmp_path / method), load_in_4bit=True, torch_dtype=torch.float32,
                                                 optimize_model=False)
    lows = [m for m in model.modules() if isinstance(m, LowBitLinear)]
    assert len(lows) >= 14
    ids = torch.randint(0, 320, (2, 9))
    with torch.no_grad():
        a = ref(ids).logits.float()
        b = model(ids).logits.float()
    # codes are repacked bit-exactly; scales / mins pass through fp16, lm_head is quantized by the loader
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.99, cos
