"""Pipeline parallelism across model families on gloo stages: greedy tokens equal those of the unpartitioned low-bit
model.  The families were chosen for what their causal-LM wrapper does to the logits (Cohere scales them, Granite
divides them, Gemma-2 soft-caps them: none of it may touch the hidden states that travel between stages), for MoE
blocks and latent attention, and for caches of both kinds.  Prints ``rank N: ok``."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist
import transformers

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

MLA = dict(kv_lora_rank=32, q_lora_rank=48, qk_nope_head_dim=16, qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=4,
           num_experts_per_tok=2, moe_intermediate_size=64, n_shared_experts=1, first_k_dense_replace=1,
           num_key_value_heads=4, n_group=2, topk_group=1)
FAMILIES = {
    "cohere": ("CohereConfig", dict(pad_token_id=0, logit_scale=0.0625)),
    "granite": ("GraniteConfig", dict(logits_scaling=8.0, residual_multiplier=0.5, embedding_multiplier=3.0)),
    "gemma2": ("Gemma2Config", dict(head_dim=32, sliding_window=16, query_pre_attn_scalar=32,
                                    final_logit_softcapping=2.0)),
    "mixtral": ("MixtralConfig", dict(num_local_experts=4, num_experts_per_tok=2)),
    "deepseek_v3": ("DeepseekV3Config", MLA),
    "phi3": ("Phi3Config", dict(pad_token_id=0)),
}


def main():
    from ipex_llm.transformers import AutoModelForCausalLM, init_pipeline_parallel
    init_pipeline_parallel()
    rank, world = dist.get_rank(), dist.get_world_size()
    ids = torch.randint(0, 900, (3, 17), generator=torch.Generator().manual_seed(0))
    for fam, (cls_name, extra) in FAMILIES.items():
        kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
                  num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256)
        kw.update(extra)
        torch.manual_seed(0)
        src = transformers.AutoModelForCausalLM.from_config(getattr(transformers, cls_name)(**kw)).eval()
        box = [tempfile.mkdtemp() if rank == 0 else None]
        dist.broadcast_object_list(box, 0)
        if rank == 0:
            src.save_pretrained(box[0])
        dist.barrier()
        whole = AutoModelForCausalLM.from_pretrained(box[0], load_in_low_bit="sym_int8", torch_dtype=torch.float32)
        ref = whole.generate(ids, max_new_tokens=6, do_sample=False)
        del whole
        staged = AutoModelForCausalLM.from_pretrained(box[0], load_in_low_bit="sym_int8", torch_dtype=torch.float32,
                                                      pipeline_parallel_stages=world)
        out = staged.generate(ids, max_new_tokens=6, do_sample=False)
        assert out.shape == ref.shape and torch.equal(out, ref), (fam, out[:, 17:].tolist(), ref[:, 17:].tolist())
        dist.barrier()
    # a model laid out as `transformer.h` is refused with a message, not with an attribute error
    cfg = transformers.GPTJConfig(n_embd=128, n_layer=2, n_head=4, rotary_dim=16, vocab_size=1000)
    box = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(box, 0)
    if rank == 0:
        transformers.AutoModelForCausalLM.from_config(cfg).save_pretrained(box[0])
    dist.barrier()
    try:
        AutoModelForCausalLM.from_pretrained(box[0], load_in_low_bit="sym_int8", pipeline_parallel_stages=world)
        raise AssertionError("a transformer.h model was accepted")
    except RuntimeError as e:
        assert "laid out differently" in str(e), e
    print(f"rank {rank}: ok", flush=True)


if __name__ == "__main__":
    main()
