"""python examples/speculative.py --repo-id-or-model-path <dir> --prompt "..."   (fp16 target + sym_int4 draft)"""
import argparse

import torch
from transformers import AutoTokenizer

from ipex_llm.transformers import AutoModelForCausalLM

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id-or-model-path", required=True)
    ap.add_argument("--prompt", default="Tell me a long story.")
    ap.add_argument("--n-predict", type=int, default=128)
    a = ap.parse_args()
    model = AutoModelForCausalLM.from_pretrained(a.repo_id_or_model_path, load_in_low_bit="fp16", speculative=True,
                                                 torch_dtype=torch.float16, trust_remote_code=True).to("cuda")
    tok = AutoTokenizer.from_pretrained(a.repo_id_or_model_path)
    ids = tok(a.prompt, return_tensors="pt")["input_ids"].cuda()
    out = model.generate(ids, max_new_tokens=a.n_predict, th_stop_draft=0.6, do_sample=False)
    print(tok.decode(out[0], skip_special_tokens=True))
    print(f"drafted {model.n_drafted}, accepted {model.n_matched}")
