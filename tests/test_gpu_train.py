"""Training-side GPU checks: fused flat AdamW kernel, QLoRA forward/backward through the packed base."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_adamw_kernel_matches_torch(dtype):
    from ipex_llm_b200.ops import cuda_ops
    from ipex_llm_b200.parallel.dp import FusedLoraAdamW
    torch.manual_seed(0)
    shapes = [(8, 4096), (4096, 8), (5, 3)]
    ps = [torch.nn.Parameter((torch.randn(s, device="cuda") * 0.1).to(dtype)) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().float().clone()) for p in ps]
    opt = FusedLoraAdamW(ps, lr=1e-2, weight_decay=0.05)
    ropt = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.05)
    for _ in range(5):
        for p, r in zip(ps, ref):
            g = (torch.randn_like(p.float()) * 0.3).to(dtype)
            p.grad.copy_(g)
            r.grad = g.float()
        opt.step()
        ropt.step()
        opt.zero_grad()
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(ps[0].device)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for p, r in zip(ps, ref):
        assert (p.float() - r).abs().max().item() < tol


def test_qlora_forward_backward_gpu():
    from transformers import LlamaConfig
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm.transformers.qlora import LoraConfig, get_peft_model, prepare_model_for_kbit_training
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256, tie_word_embeddings=False)
    model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="nf4", torch_dtype=torch.bfloat16, device="cuda",
                                             modules_to_not_convert=["lm_head"], optimize_model=False)
    model = prepare_model_for_kbit_training(model, use_gradient_checkpointing=False)
    pm = get_peft_model(model, LoraConfig(r=8, lora_alpha=16, target_modules=["q_proj", "v_proj", "up_proj"]))
    for m in pm.modules():
        if hasattr(m, "lora_A"):
            m.lora_A.to(torch.bfloat16)
            m.lora_B.to(torch.bfloat16)
    ids = torch.randint(0, 1000, (4, 64), device="cuda")
    pm.train()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = pm(input_ids=ids, labels=ids).loss
    loss.backward()
    assert torch.isfinite(loss)
    grads = [p.grad for n, p in pm.named_parameters() if "lora_B" in n]
    assert len(grads) == 6 and all(g is not None and torch.isfinite(g).all() for g in grads)
    assert any(float(g.abs().sum()) > 0 for g in grads)


def test_paged_adamw_double_buffered_matches_torch_adamw():
    """Moments in pinned host pages, two device buffers, copy stream + events: same numbers as torch.optim.AdamW."""
    from ipex_llm_b200.parallel.dp import PagedAdamW
    torch.manual_seed(0)
    ws = [torch.randn(300, 70, device="cuda"), torch.randn(5000, device="cuda"), torch.randn(8, 64, device="cuda")]
    a = [torch.nn.Parameter(w.clone()) for w in ws]
    b = [torch.nn.Parameter(w.clone()) for w in ws]
    oa = PagedAdamW(a, lr=1e-2, weight_decay=0.01, page_elems=4096)      # several pages per tensor
    ob = torch.optim.AdamW(b, lr=1e-2, weight_decay=0.01)
    for step in range(5):
        for pa, pb in zip(a, b):
            g = torch.randn_like(pa)
            pa.grad, pb.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    for pa, pb in zip(a, b):
        assert torch.allclose(pa, pb, atol=1e-5, rtol=1e-4)
    hm, hv = oa._host[a[0]]
    assert hm.is_pinned() and float(hm.abs().sum()) > 0 and float(hv.sum()) > 0
