"""Self-speculative decoding on synthetic data: half-precision target + sym_int4 draft of the same weights.

    python -m ipex_llm_b200.utils.bench_speculative [--model llama2-7b] [--prompt 1024] [--new-tokens 128]

Random-init weights of the named architecture (so the draft is the int4 quantization of the target, as with a real
checkpoint), batch 1, greedy, ``max_step_draft`` 8.  Reports end-to-end tokens/s (host timed around ``generate`` with
a device synchronise on both sides, second of two runs), the number of drafted / accepted tokens and the plain
low-bit decode speed of the same model for comparison.  With random weights the logits are nearly flat, so the
acceptance rate here is a lower bound on what a trained checkpoint gives.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

ARCH = {
    "llama2-7b": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=32, vocab_size=32000, max_position_embeddings=4096),
    "tiny": dict(hidden_size=512, intermediate_size=1408, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=4, vocab_size=32000, max_position_embeddings=2048),
}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama2-7b", choices=list(ARCH))
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--max-step-draft", type=int, default=8)
    a = ap.parse_args(argv)
    from transformers import LlamaConfig
    from ..transformers import AutoModelForCausalLM
    cfg = LlamaConfig(tie_word_embeddings=False, **ARCH[a.model])
    model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="fp16", device="cuda", torch_dtype=torch.float16,
                                             speculative=True, seed=0)
    ids = torch.randint(0, cfg.vocab_size, (1, a.prompt), generator=torch.Generator().manual_seed(3)).cuda()
    res = {}
    for run in range(2):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = model.generate(ids, max_new_tokens=a.new_tokens, do_sample=False, max_step_draft=a.max_step_draft)
        torch.cuda.synchronize()
        res = {"seconds": time.perf_counter() - t0, "new_tokens": int(out.shape[1] - ids.shape[1])}
    line = {"metric": "self-speculative decoding", "model": a.model, "prompt": a.prompt,
            "new_tokens": res["new_tokens"], "e2e_tokens_per_s": round(res["new_tokens"] / res["seconds"], 2),
            "e2e_seconds": round(res["seconds"], 4), "n_drafted": int(getattr(model, "n_drafted", 0)),
            "n_matched": int(getattr(model, "n_matched", 0)), "max_step_draft": a.max_step_draft,
            "target": "fp16", "draft": "sym_int4"}
    if line["n_drafted"]:
        line["accept_rate"] = round(line["n_matched"] / line["n_drafted"], 4)
    print(json.dumps(line))


if __name__ == "__main__":
    main()
