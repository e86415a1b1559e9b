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


def _snap_target_to_draft(target, draft):
    from ..ops import cuda_ops
    from ..ops.linear import LowBitLinear
    mods = dict(target.named_modules())
    for name, mod in draft.named_modules():
        if isinstance(mod, LowBitLinear) and name in mods and hasattr(mods[name], "weight"):
            w = mod.weight
            deq = cuda_ops.dequantize_device(w.data, tuple(int(v) for v in w._shape), w.qtype, torch.float16)
            mods[name].weight.data.copy_(deq)


def run(argv=None, timed=None):
    """Run the benchmark and return the result dictionary."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama2-7b", choices=list(ARCH))
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--max-step-draft", type=int, default=8)
    ap.add_argument("--snap", action="store_true",
                    help="give the target the draft's dequantized weights: draft and target then agree, which shows "
                         "the speed at (near) full acceptance instead of the near-zero acceptance of random weights")
    ap.add_argument("--th-stop-draft", type=float, default=None,
                    help="fixed confidence threshold of the draft's early stop (0 = always draft max-step-draft "
                         "tokens); default: the library's adaptive threshold")
    a = ap.parse_args(argv)
    spec_kw = {"max_step_draft": a.max_step_draft}
    if a.th_stop_draft is not None:
        spec_kw.update(th_stop_draft=a.th_stop_draft, auto_th_stop_draft=False)
    from transformers import LlamaConfig
    from ..transformers import AutoModelForCausalLM
    cfg = LlamaConfig(tie_word_embeddings=False, **ARCH[a.model])
    model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="fp16", device="cuda", torch_dtype=torch.float16,
                                             speculative=True, seed=0)
    if a.snap:
        _snap_target_to_draft(model, model.draft_model)
    ids = torch.randint(0, cfg.vocab_size, (1, a.prompt), generator=torch.Generator().manual_seed(3)).cuda()
    res = {}
    for run in range(2):
        torch.cuda.synchronize()
        if timed and run == 1:
            timed[0]()                       # clock sampling covers the measured (second) pass only
        t0 = time.perf_counter()
        out = model.generate(ids, max_new_tokens=a.new_tokens, do_sample=False, **spec_kw)
        torch.cuda.synchronize()
        res = {"seconds": time.perf_counter() - t0, "new_tokens": int(out.shape[1] - ids.shape[1])}
        if timed and run == 1:
            timed[1]()
    line = {"metric": "self-speculative decoding", "model": a.model, "prompt": a.prompt,
            "new_tokens": res["new_tokens"], "e2e_tokens_per_s": round(res["new_tokens"] / res["seconds"], 2),
            "e2e_seconds": round(res["seconds"], 4), "n_drafted": int(getattr(model, "n_drafted", 0)),
            "n_matched": int(getattr(model, "n_matched", 0)), "max_step_draft": a.max_step_draft,
            "target": "fp16 with the draft's dequantized weights" if a.snap else "fp16", "draft": "sym_int4",
            "first_token_ms": round(1e3 * float(getattr(model, "first_token_time", 0.0)), 2),
            "decode_tokens_per_s": round((res["new_tokens"] - 1) /
                                         max(1e-9, float(getattr(model, "e2e_time_without_first", 0.0))), 2),
            "draft_ms_total": round(1e3 * sum(getattr(model, "draft_time", [])), 2),
            "verify_ms_total": round(1e3 * sum(getattr(model, "verify_time", [])), 2),
            "iterations": len(getattr(model, "verify_time", []))}
    if line["n_drafted"]:
        line["accept_rate"] = round(line["n_matched"] / line["n_drafted"], 4)
    # the target alone (plain half-precision decode through its graph engine) for the speed-up ratio
    draft, model.draft_model = model.draft_model, None
    try:
        for run in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = model.generate(ids, max_new_tokens=a.new_tokens, do_sample=False)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        line["target_alone_e2e_tokens_per_s"] = round(int(out.shape[1] - ids.shape[1]) / dt, 2)
        line["speedup_vs_target_alone"] = round(line["e2e_tokens_per_s"] / line["target_alone_e2e_tokens_per_s"], 3)
    finally:
        model.draft_model = draft
    line["value"], line["unit"] = line["e2e_tokens_per_s"], "tokens/s"
    line["ms_per_step"] = round(1e3 * res["seconds"] / max(1, res["new_tokens"]), 4)
    return line


def main(argv=None):
    print(json.dumps(run(argv)))


if __name__ == "__main__":
    main()
