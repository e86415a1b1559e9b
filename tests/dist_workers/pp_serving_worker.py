"""Pipeline-parallel serving on gloo ranks: every rank builds a ``PPModelWorker`` over its stage; rank 0 submits two
prompts of different lengths, the other rank follows the batches rank 0 announces; the generated text equals what the
unpartitioned model generates for each prompt alone.  Prints ``rank N: ok``."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    model_dir = sys.argv[1]
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.serving.model_worker import SamplingParams
    from ipex_llm_b200.serving.pp_worker import PPModelWorker
    worker = PPModelWorker(model_dir, low_bit="sym_int8", max_num_seqs=4, torch_dtype=torch.float32)
    rank = dist.get_rank()
    if rank != 0:
        worker._serve_forever()                      # returns when rank 0 announces the stop
        print(f"rank {rank}: ok", flush=True)
        return
    whole = AutoModelForCausalLM.from_pretrained(model_dir, load_in_low_bit="sym_int8", torch_dtype=torch.float32)
    tok = worker.tokenizer
    prompts = ["w1 w2 w3 w4 w5 w6 w7", "w9 w8"]
    want = []
    for p in prompts:
        ids = tok(p, return_tensors="pt")["input_ids"]
        out = whole.generate(ids, max_new_tokens=6, do_sample=False)
        want.append(tok.decode(out[0, ids.shape[1]:], skip_special_tokens=True))
    reqs = [worker.submit_blocking(p, SamplingParams(max_new_tokens=6)) for p in prompts]
    worker.start()
    deadline = time.time() + 120
    while not all(r.finished for r in reqs) and time.time() < deadline:
        time.sleep(0.05)
    worker.shutdown()
    assert all(r.finished for r in reqs), "requests did not finish"
    for r, w in zip(reqs, want):
        assert r.text.strip() == w.strip(), (r.text, w)
    print(f"rank {rank}: ok", flush=True)


if __name__ == "__main__":
    main()
