"""Very-low-bit and mixed formats: ``gguf_iq2_xxs`` / ``gguf_iq2_xs`` / ``gguf_iq1_s`` with a llama.cpp importance
matrix, ``q2_k``, and the ``gguf_q4k_m`` / ``gguf_q4k_s`` presets.  Reference:
python/llm/example/GPU/HuggingFace/Advanced-Quantizations (imatrix flow of python/llm/src/ipex_llm/transformers/model.py:325-341)

    python examples/low_bit_formats.py --model <hf dir> --low-bit gguf_iq2_xxs --imatrix imatrix.dat

The code-book formats need the importance matrix; their search runs on the GPU when the weights are already there
(pass --quantize-on-gpu), which takes seconds where the CPU takes minutes.
"""
import argparse

import torch

from ipex_llm.transformers import AutoModelForCausalLM

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--low-bit", default="gguf_iq2_xxs")
    ap.add_argument("--imatrix", default=None, help="llama.cpp imatrix file (required for gguf_iq2_* / gguf_iq1_*)")
    ap.add_argument("--save", default=None, help="directory for save_low_bit")
    ap.add_argument("--prompt", default="What is AI?")
    ap.add_argument("--n-predict", type=int, default=32)
    a = ap.parse_args()
    kw = {"imatrix": a.imatrix} if a.imatrix else {}
    model = AutoModelForCausalLM.from_pretrained(a.model, load_in_low_bit=a.low_bit, torch_dtype=torch.float16, **kw)
    kinds = {}
    for m in model.modules():
        w = getattr(m, "weight", None)
        if getattr(w, "quantized", False):
            kinds[w.qtype] = kinds.get(w.qtype, 0) + 1
    from ipex_llm_b200.quant.qtypes import qtype_name
    print("packed layers per format:", {qtype_name(k): v for k, v in kinds.items()})
    if a.save:
        model.save_low_bit(a.save)
    if torch.cuda.is_available():
        model = model.to("cuda")
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(a.model)
    ids = tok(a.prompt, return_tensors="pt")["input_ids"].to(next(model.parameters()).device)
    print(tok.decode(model.generate(ids, max_new_tokens=a.n_predict, do_sample=False)[0], skip_special_tokens=True))
