"""python examples/generate.py --repo-id-or-model-path <dir> [--low-bit sym_int4] [--save <dir>] --prompt "..." """
import argparse
import time

import torch
from transformers import AutoTokenizer

from ipex_llm.transformers import AutoModelForCausalLM

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id-or-model-path", required=True)
    ap.add_argument("--low-bit", default="sym_int4")
    ap.add_argument("--load-low-bit", action="store_true", help="the path is a save_low_bit directory")
    ap.add_argument("--save", default=None, help="write the quantized model here")
    ap.add_argument("--prompt", default="What is AI?")
    ap.add_argument("--n-predict", type=int, default=64)
    a = ap.parse_args()
    if a.load_low_bit:
        model = AutoModelForCausalLM.load_low_bit(a.repo_id_or_model_path, trust_remote_code=True)
    else:
        model = AutoModelForCausalLM.from_pretrained(a.repo_id_or_model_path, load_in_low_bit=a.low_bit,
                                                     optimize_model=True, trust_remote_code=True, use_cache=True)
    if a.save:
        model.save_low_bit(a.save)
    model = model.to("cuda" if torch.cuda.is_available() else "cpu")
    tok = AutoTokenizer.from_pretrained(a.repo_id_or_model_path, trust_remote_code=True)
    ids = tok(a.prompt, return_tensors="pt")["input_ids"].to(next(model.parameters()).device)
    with torch.inference_mode():
        model.generate(ids, max_new_tokens=8)                    # warm-up (graph capture)
        t0 = time.perf_counter()
        out = model.generate(ids, max_new_tokens=a.n_predict)
        dt = time.perf_counter() - t0
    print(tok.decode(out[0], skip_special_tokens=True))
    print(f"Inference time: {dt:.3f} s; first token {getattr(model, 'first_token_time', 0) * 1e3:.1f} ms, "
          f"next tokens {getattr(model, 'rest_cost_mean', 0) * 1e3:.2f} ms")
