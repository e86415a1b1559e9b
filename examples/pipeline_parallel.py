"""torchrun --nproc-per-node N --master-addr 127.0.0.1 examples/pipeline_parallel.py --repo-id-or-model-path <dir>"""
import argparse

import torch
import torch.distributed as dist
from transformers import AutoTokenizer

from ipex_llm.transformers import AutoModelForCausalLM, init_pipeline_parallel

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id-or-model-path", required=True)
    ap.add_argument("--low-bit", default="sym_int4")
    ap.add_argument("--prompt", default="Once upon a time")
    ap.add_argument("--n-predict", type=int, default=64)
    a = ap.parse_args()
    init_pipeline_parallel()
    model = AutoModelForCausalLM.from_pretrained(a.repo_id_or_model_path, load_in_low_bit=a.low_bit,
                                                 torch_dtype=torch.float16,
                                                 pipeline_parallel_stages=dist.get_world_size())
    tok = AutoTokenizer.from_pretrained(a.repo_id_or_model_path)
    ids = tok(a.prompt, return_tensors="pt")["input_ids"]
    out = model.generate(ids, max_new_tokens=a.n_predict)
    if dist.get_rank() == 0:
        print(tok.decode(out[0], skip_special_tokens=True))
        print(f"first token {model.first_token_time * 1e3:.1f} ms, next {model.rest_cost_mean * 1e3:.2f} ms")
