"""torchrun --nproc-per-node N --master-addr 127.0.0.1 examples/tensor_parallel.py --repo-id-or-model-path <dir>"""
import argparse
import os

import torch
import torch.distributed as dist
from transformers import AutoTokenizer

from ipex_llm.transformers import AutoModelForCausalLM
from ipex_llm_b200.parallel.tp import TPGroup

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id-or-model-path", required=True)
    ap.add_argument("--low-bit", default="fp8_e4m3")
    ap.add_argument("--prompt", default="Once upon a time")
    ap.add_argument("--n-predict", type=int, default=64)
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    model = AutoModelForCausalLM.from_pretrained(a.repo_id_or_model_path, load_in_low_bit=a.low_bit,
                                                 torch_dtype=torch.bfloat16, tp_group=TPGroup()).to(f"cuda:{local}")
    tok = AutoTokenizer.from_pretrained(a.repo_id_or_model_path)
    ids = tok(a.prompt, return_tensors="pt")["input_ids"].cuda()
    out = model.generate(ids, max_new_tokens=a.n_predict, do_sample=False)
    if dist.get_rank() == 0:
        print(tok.decode(out[0], skip_special_tokens=True))
    dist.destroy_process_group()
