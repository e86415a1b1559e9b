"""QLoRA stack on CPU: adapter injection, backward through the frozen low-bit base, fused optimizer restatement,
adapter save / load, trainer checkpoint + resume."""
import copy
import os

import torch


def _tiny(qtype="nf4"):
    from transformers import LlamaConfig
    from ipex_llm.transformers import AutoModelForCausalLM
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=256, max_position_embeddings=128, tie_word_embeddings=False)
    torch.manual_seed(0)
    return AutoModelForCausalLM.from_config(cfg, load_in_low_bit=qtype, torch_dtype=torch.float32,
                                            modules_to_not_convert=["lm_head"], optimize_model=False, device="cpu")


def _dataset(n=64, seq=16, vocab=256):
    g = torch.Generator().manual_seed(1)
    data = []
    for _ in range(n):
        start = int(torch.randint(0, vocab - seq - 1, (1,), generator=g))
        ids = list(range(start, start + seq))          # learnable: next token = current + 1
        data.append({"input_ids": ids, "labels": ids})
    return data


def test_lora_injection_and_backward():
    from ipex_llm.transformers.qlora import (LoraConfig, LoraLowBitLinear, get_peft_model,
                                             prepare_model_for_kbit_training)
    model = prepare_model_for_kbit_training(_tiny(), use_gradient_checkpointing=False)
    cfg = LoraConfig(r=4, lora_alpha=8, lora_dropout=0.0, target_modules=["q_proj", "v_proj", "down_proj"],
                     training_mode="qlora")
    pm = get_peft_model(model, cfg)
    loras = [m for m in pm.modules() if isinstance(m, LoraLowBitLinear)]
    assert len(loras) == 2 * 3
    t, a = pm.get_nb_trainable_parameters()
    assert 0 < t < a
    assert all(("lora_" in n) == p.requires_grad for n, p in pm.named_parameters())
    ids = torch.randint(0, 256, (2, 12))
    out = pm(input_ids=ids, labels=ids)
    out.loss.backward()
    for m in loras:
        gB = m.lora_B["default"].weight.grad
        assert gB is not None and torch.isfinite(gB).all()
    # lora_B starts at zero, so A receives no gradient yet but B does
    assert any(m.lora_B["default"].weight.grad.abs().sum() > 0 for m in loras)


def test_qalora_pools_adapter_input():
    from ipex_llm.transformers.qlora import LoraConfig, LoraLowBitLinear, get_peft_model
    pm = get_peft_model(_tiny("sym_int4"), LoraConfig(r=2, target_modules=["q_proj"], training_mode="qalora"))
    m = next(x for x in pm.modules() if isinstance(x, LoraLowBitLinear))
    assert m.lora_A["default"].weight.shape == (2, 64 // 64)
    y = pm(input_ids=torch.randint(0, 256, (1, 5))).logits
    assert torch.isfinite(y).all()


def test_fused_optimizer_host_path_matches_torch_adamw():
    from ipex_llm_b200.parallel.dp import FusedLoraAdamW
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(7, 5)), torch.nn.Parameter(torch.randn(11))]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    opt = FusedLoraAdamW(ps, lr=1e-2, weight_decay=0.1)
    ropt = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.1)
    for step in range(5):
        for p, r in zip(ps, ref):
            g = torch.randn_like(p)
            p.grad.copy_(g)
            r.grad = g.clone()
        opt.step()
        ropt.step()
        opt.zero_grad()
    for p, r in zip(ps, ref):
        assert torch.allclose(p, r, atol=1e-6)


def test_trainer_learns_saves_and_resumes(tmp_path):
    from ipex_llm.transformers.qlora import (LoraConfig, PeftModel, TrainingArguments, get_peft_model,
                                             prepare_model_for_kbit_training)
    from ipex_llm_b200.train import Trainer

    def build():
        m = prepare_model_for_kbit_training(_tiny(), use_gradient_checkpointing=False)
        torch.manual_seed(3)
        return get_peft_model(m, LoraConfig(r=8, lora_alpha=16, target_modules=["q_proj", "k_proj", "v_proj",
                                                                                 "o_proj", "up_proj", "down_proj"]))
    data = _dataset(n=8)      # one batch, seen every step: the adapters can memorise it
    args = TrainingArguments(output_dir=str(tmp_path / "run"), per_device_train_batch_size=8, max_steps=12,
                             learning_rate=2e-2, logging_steps=1, save_steps=6, bf16=False, max_grad_norm=1.0,
                             optim="fused_lora_adamw", lr_scheduler_type="constant")
    pm = build()
    tr = Trainer(pm, args, train_dataset=data)
    tr.train()
    losses = [r["loss"] for r in tr.state.log_history]
    assert losses[-1] < losses[0] - 0.15, losses
    assert os.path.exists(tmp_path / "run" / "checkpoint-6" / "adapter_model.bin")
    final = {k: v.clone() for k, v in pm.state_dict().items() if "lora_" in k}

    # resume from step 6 and land on the same weights
    pm2 = build()
    tr2 = Trainer(pm2, copy.deepcopy(args), train_dataset=data)
    tr2.train(resume_from_checkpoint=str(tmp_path / "run" / "checkpoint-6"))
    assert tr2.state.global_step == 12
    for k, v in pm2.state_dict().items():
        if "lora_" in k:
            assert torch.allclose(v, final[k], atol=1e-5), k

    # adapter round trip onto a fresh base
    pm.save_pretrained(str(tmp_path / "adapter"))
    pm3 = PeftModel.from_pretrained(_tiny(), str(tmp_path / "adapter"))
    ids = torch.randint(0, 256, (1, 9))
    pm.eval()
    with torch.no_grad():
        assert torch.allclose(pm(input_ids=ids).logits, pm3(input_ids=ids).logits, atol=1e-5)


def test_relora_merge_and_lisa_switching(tmp_path):
    from ipex_llm.transformers.lisa import DynamicLayerActivationCallback
    from ipex_llm.transformers.qlora import (LoraConfig, TrainingArguments, get_peft_model,
                                             prepare_model_for_kbit_training)
    from ipex_llm.transformers.relora import ReLoRATrainer, find_lora_modules, lora_delta_weight, merge_and_requantize
    m = prepare_model_for_kbit_training(_tiny("sym_int8"), use_gradient_checkpointing=False)
    pm = get_peft_model(m, LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "down_proj"],
                                      training_mode="relora"))
    mods = find_lora_modules(pm)
    assert len(mods) == 4
    name, layer = next(iter(mods.items()))
    with torch.no_grad():
        layer.lora_B["default"].weight.normal_(0, 0.05)
    before = layer.base_layer.weight.dequantize(torch.float32).clone()
    delta = lora_delta_weight(layer)
    x = torch.randn(3, layer.in_features)
    y_before = layer(x)
    merge_and_requantize(pm, reinit=True)
    after = layer.base_layer.weight.dequantize(torch.float32)
    # merged weight = old + delta up to int8 re-quantization error; adapter restarted at zero
    assert (after - (before + delta)).abs().max() < 0.02 * (before + delta).abs().max()
    assert float(layer.lora_B["default"].weight.abs().sum()) == 0.0
    assert torch.allclose(layer(x), y_before, atol=0.05 * float(y_before.abs().max()))

    data = _dataset(n=8)
    args = TrainingArguments(output_dir=str(tmp_path / "relora"), per_device_train_batch_size=8, max_steps=7,
                             learning_rate=1e-2, logging_steps=1, bf16=False, lr_scheduler_type="constant")
    tr = ReLoRATrainer(pm, args, train_dataset=data, relora_steps=3, relora_warmup_steps=2)
    tr.train()
    assert tr.relora.num_restarts == 2
    lrs = [r["lr"] for r in tr.state.log_history]
    assert lrs[3] < lrs[2] and lrs[4] > lrs[3]          # re-warm-up after the restart at step 3

    # LISA: layer subsets switch on the interval, only float parameters are unfrozen
    base = _tiny("sym_int4")
    cb = DynamicLayerActivationCallback(n_layers=1, interval_steps=2, model=base, seed=1)

    class S:
        global_step = 0
    seen = set()
    for step in range(6):
        S.global_step = step
        cb.on_step_begin(None, S, None)
        seen.add(tuple(cb.active_layers_indices))
        act = [i for i, l in enumerate(cb.layers) if any(p.requires_grad for p in l.parameters())]
        assert act == list(cb.active_layers_indices)
        assert not any(p.requires_grad for l in cb.layers for p in l.parameters() if hasattr(p, "qtype"))
    assert len(seen) >= 1


def test_paged_adamw_matches_torch_adamw_cpu():
    from ipex_llm_b200.parallel.dp import PagedAdamW
    torch.manual_seed(0)
    ws = [torch.randn(37, 5), torch.randn(130)]
    a = [torch.nn.Parameter(w.clone()) for w in ws]
    b = [torch.nn.Parameter(w.clone()) for w in ws]
    oa = PagedAdamW(a, lr=1e-2, weight_decay=0.01, page_elems=64)
    ob = torch.optim.AdamW(b, lr=1e-2, weight_decay=0.01)
    for step in range(4):
        for pa, pb in zip(a, b):
            g = torch.randn_like(pa)
            pa.grad, pb.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    for pa, pb in zip(a, b):
        assert torch.allclose(pa, pb, atol=1e-6, rtol=1e-5)
