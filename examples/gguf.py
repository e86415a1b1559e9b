"""Load a ``.gguf`` file straight into a low-bit model (llama, mistral, mixtral, qwen2, qwen3, gemma, gemma2, phi3,
baichuan, yuan, bloom, falcon and mpt files; f32 / f16 / bf16 / q4_0 ... q8_0 / k-quant / i-quant tensors; sentencepiece
and byte-level BPE vocabularies) and generate.  Reference: python/llm/example/GPU/HuggingFace/Advanced-Quantizations/GGUF/generate.py

    python examples/gguf.py --model model.gguf --prompt "What is AI?" --n-predict 32
"""
import argparse

import torch

from ipex_llm.transformers import AutoModelForCausalLM

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt", default="What is AI?")
    ap.add_argument("--n-predict", type=int, default=32)
    ap.add_argument("--low-bit", default="sym_int4")
    a = ap.parse_args()
    model, tokenizer = AutoModelForCausalLM.from_gguf(a.model, low_bit=a.low_bit)
    if torch.cuda.is_available():
        model = model.half().to("cuda")
    if tokenizer is None:
        raise SystemExit("the file carries no sentencepiece vocabulary; pass token ids to model.generate directly")
    ids = tokenizer(a.prompt, return_tensors="pt")["input_ids"].to(next(model.parameters()).device)
    out = model.generate(ids, max_new_tokens=a.n_predict, do_sample=False)
    print(tokenizer.decode(out[0], skip_special_tokens=True))
