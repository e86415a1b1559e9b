"""Long prompts on one GPU: fp8 (e5m2) KV cache, SnapKV compression of the prompt's KV, low-memory mode.
Reference: python/llm/example/GPU/Long-Context/llama2-32k/generate.py

    IPEX_LLM_QUANTIZE_KV_CACHE=1 IPEX_LLM_COMPRESS_KV_CACHE=1 IPEX_LLM_LOW_MEM=1 \
        python examples/long_context.py --repo-id-or-model-path <dir> --prompt-file long.txt
"""
import argparse
import time

import torch
from transformers import AutoTokenizer

from ipex_llm.transformers import AutoModelForCausalLM

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id-or-model-path", required=True)
    ap.add_argument("--prompt-file", required=True)
    ap.add_argument("--n-predict", type=int, default=128)
    ap.add_argument("--low-bit", default="sym_int4")
    a = ap.parse_args()
    tok = AutoTokenizer.from_pretrained(a.repo_id_or_model_path, trust_remote_code=True)
    model = AutoModelForCausalLM.from_pretrained(a.repo_id_or_model_path, load_in_low_bit=a.low_bit,
                                                 torch_dtype=torch.float16, trust_remote_code=True).half().to("cuda")
    with open(a.prompt_file) as f:
        ids = tok(f.read(), return_tensors="pt").input_ids.to("cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = model.generate(ids, max_new_tokens=a.n_predict, do_sample=False)
    torch.cuda.synchronize()
    print(f"prompt {ids.shape[1]} tokens, {out.shape[1] - ids.shape[1]} new tokens in {time.perf_counter() - t0:.2f} s, "
          f"first token {getattr(model, 'first_token_time', 0.0) * 1e3:.1f} ms, "
          f"peak memory {torch.cuda.max_memory_allocated() / 2 ** 30:.1f} GiB")
    print(tok.decode(out[0, ids.shape[1]:], skip_special_tokens=True))
