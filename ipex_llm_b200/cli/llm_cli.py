"""``llm-cli``: one-shot completion, ``llm-chat``: interactive chat, both on a low-bit checkpoint.

    python -m ipex_llm_b200.cli.llm_cli -m <model dir or low-bit dir> -p "Once upon a time" -n 64 [-t sym_int4]
    python -m ipex_llm_b200.cli.llm_cli --chat -m <model dir>

The reference ships shell wrappers around per-family native binaries (``llm-cli -x llama -m model.bin -p ...``,
python/llm/src/ipex_llm/cli/llm-cli:1-98); here the same flags drive the transformers-style API and ``-x`` is accepted
for compatibility (the architecture is read from the checkpoint).
"""
from __future__ import annotations

import argparse
import os
import sys
import time


def _load(path: str, low_bit: str, device: str):
    import torch
    from transformers import AutoTokenizer
    from ..transformers import AutoModel, AutoModelForCausalLM
    cfg = os.path.join(path, "config.json")
    saved = False
    if os.path.exists(cfg):
        import json
        with open(cfg) as f:
            saved = "bigdl_transformers_low_bit" in json.load(f)
    if path.endswith(".gguf"):
        model, tok = AutoModelForCausalLM.from_gguf(path, low_bit=low_bit)
    else:
        tok = AutoTokenizer.from_pretrained(path, trust_remote_code=True)
        loader = (lambda c: c.load_low_bit(path, trust_remote_code=True)) if saved else \
            (lambda c: c.from_pretrained(path, load_in_low_bit=low_bit, trust_remote_code=True))
        try:
            model = loader(AutoModelForCausalLM)
        except Exception:  # noqa: BLE001
            model = loader(AutoModel)
    if device == "auto":
        device = "cuda" if torch.cuda.is_available() else "cpu"
    return model.eval().to(device), tok


def build_parser():
    p = argparse.ArgumentParser(prog="llm-cli", description=__doc__.split("\n")[0])
    p.add_argument("-m", "--model", required=True, help="checkpoint directory, low-bit directory or .gguf file")
    p.add_argument("-x", "--model_family", default=None, help="accepted for compatibility; read from the checkpoint")
    p.add_argument("-t", "--low-bit", default="sym_int4")
    p.add_argument("-p", "--prompt", default=None)
    p.add_argument("-n", "--n_predict", type=int, default=128)
    p.add_argument("--temp", type=float, default=0.0)
    p.add_argument("--top_p", type=float, default=1.0)
    p.add_argument("--device", default="auto")
    p.add_argument("--chat", action="store_true", help="interactive chat (llm-chat)")
    return p


def _generate(model, tok, prompt, n, temp, top_p, stream=True):
    import torch
    from transformers import TextStreamer
    dev = next(model.parameters()).device
    ids = tok(prompt, return_tensors="pt")["input_ids"].to(dev)
    kw = dict(max_new_tokens=n, do_sample=temp > 0)
    if temp > 0:
        kw.update(temperature=temp, top_p=top_p)
    streamer = TextStreamer(tok, skip_prompt=True, skip_special_tokens=True) if stream else None
    t0 = time.perf_counter()
    with torch.no_grad():
        out = model.generate(ids, streamer=streamer, **kw)
    dt = time.perf_counter() - t0
    new = out.shape[1] - ids.shape[1]
    return tok.decode(out[0][ids.shape[1]:], skip_special_tokens=True), new, dt


def main(argv=None):
    a = build_parser().parse_args(argv)
    model, tok = _load(a.model, a.low_bit, a.device)
    if not a.chat:
        prompt = a.prompt if a.prompt is not None else sys.stdin.read()
        _, new, dt = _generate(model, tok, prompt, a.n_predict, a.temp, a.top_p)
        print(f"\n[{new} tokens, {dt:.2f} s, {new / max(dt, 1e-9):.1f} tokens/s]", file=sys.stderr)
        return 0
    history = []
    print("Interactive chat; empty line or Ctrl-D to quit.")
    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        if not line.strip():
            break
        history.append({"role": "user", "content": line})
        if getattr(tok, "chat_template", None):
            prompt = tok.apply_chat_template(history, tokenize=False, add_generation_prompt=True)
        else:
            prompt = "".join(f"{m['role']}: {m['content']}\n" for m in history) + "assistant:"
        text, _, _ = _generate(model, tok, prompt, a.n_predict, a.temp, a.top_p)
        history.append({"role": "assistant", "content": text})
    return 0


def chat_main(argv=None):
    return main((argv if argv is not None else sys.argv[1:]) + ["--chat"])


def quantize_main(argv=None):
    """``ipex-quantize in.gguf out.gguf q4_k [--keep substr] [--output-type q6_k]``: hands over to the native
    executable (built on first use), the counterpart of the reference's ``quantize-<family>`` binaries."""
    import os
    import sys
    from ..native.build import build_tools
    exe = build_tools()
    os.execv(exe, [exe, *(sys.argv[1:] if argv is None else argv)])


if __name__ == "__main__":
    sys.exit(main())
