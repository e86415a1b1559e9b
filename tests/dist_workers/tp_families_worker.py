"""Tensor parallelism across model families on gloo ranks: the sharded low-bit model gives the logits of the whole one.
Covers fused qkv / gate_up matrices (Phi-3, GLM), expert banks whose partial sums are all-reduced at the bank's output
(Mixtral through the package's MoE block, Phi-MoE through its own), a shared expert beside the bank (Qwen2-MoE), and
attention modules that stay replicated (latent attention, whole-vector q / k norms, configured head counts,
head-interleaved qkv).  Prints ``rank N: ok``."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist
import transformers

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

MLA = dict(kv_lora_rank=32, q_lora_rank=48, qk_nope_head_dim=16, qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=4,
           num_experts_per_tok=2, moe_intermediate_size=64, n_shared_experts=1, first_k_dense_replace=1,
           num_key_value_heads=4, n_group=2, topk_group=1)
FAMILIES = {
    "phi3": ("Phi3Config", dict(pad_token_id=0), 0.8),
    "glm": ("GlmConfig", dict(head_dim=32, pad_token_id=0), 0.8),
    "mixtral": ("MixtralConfig", dict(num_local_experts=4, num_experts_per_tok=2), 0.7),
    "qwen2_moe": ("Qwen2MoeConfig", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                                         shared_expert_intermediate_size=128), 0.7),
    "phimoe": ("PhimoeConfig", dict(num_local_experts=4, num_experts_per_tok=2), 0.7),
    "deepseek_v3": ("DeepseekV3Config", MLA, 0.9),
    "olmo2": ("Olmo2Config", dict(pad_token_id=0), 0.9),
    "stablelm": ("StableLmConfig", dict(), 0.9),
    "falcon": ("FalconConfig", dict(), 0.9),
}


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.parallel.tp import TPGroup
    tp = TPGroup(rank=rank, world_size=world)
    ids = torch.randint(0, 900, (2, 16), generator=torch.Generator().manual_seed(0))
    for fam, (cls_name, extra, max_fraction) in FAMILIES.items():
        kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
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
        shard = AutoModelForCausalLM.from_pretrained(box[0], load_in_low_bit="sym_int8", torch_dtype=torch.float32,
                                                     tp_group=tp)
        with torch.no_grad():
            a, b = whole(ids).logits[:, -1].float(), shard(ids).logits[:, -1].float()
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
        assert cos > 0.9999, (fam, cos)
        frac = sum(p.numel() for p in shard.parameters()) / sum(p.numel() for p in whole.parameters())
        assert frac < max_fraction, (fam, frac)                 # the rank really holds less than the whole model
        out = shard.generate(ids, max_new_tokens=4, do_sample=False)
        ref = whole.generate(ids, max_new_tokens=4, do_sample=False)
        assert torch.equal(out, ref), fam
        dist.barrier()
    print(f"rank {rank}: ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
