"""Sliding-window perplexity of a low-bit model: ``python -m ipex_llm_b200.benchmark.perplexity --model_path ...``.

Counterpart of python/llm/dev/benchmark/perplexity/ppl.py (class ``BigDLPPL``: ``perplexity_hf`` runs the text
through the model in windows and accumulates the shifted cross-entropy) and ``run_wikitext.py`` (strided windows
over one long token stream, the first ``seq_len - stride`` targets of every window after the first are masked).
The accuracy table of the reference's README (Wikitext perplexity per low-bit format) is produced this way.
"""
from __future__ import annotations

import argparse
import math

import torch


class BigDLPPL:
    def __init__(self, model_path=None, device="cuda", model=None, **model_kwargs):
        if model is None:
            from ..transformers import AutoModelForCausalLM
            model_kwargs.setdefault("trust_remote_code", True)
            model = AutoModelForCausalLM.from_pretrained(model_path, **model_kwargs)
            if device != "cpu":
                model = model.half().to(device)
        self.model = model.eval()
        self.device = next(model.parameters()).device

    @torch.no_grad()
    def nll(self, input_ids: torch.Tensor, target_from: int = 0):
        """Summed negative log-likelihood (fp32) of tokens ``target_from + 1 ..`` given their prefixes, and the
        number of scored tokens."""
        ids = input_ids.to(self.device)
        if ids.dim() == 1:
            ids = ids.unsqueeze(0)
        import os
        prev = os.environ.get("IPEX_LLM_LAST_LM_HEAD")
        os.environ["IPEX_LLM_LAST_LM_HEAD"] = "0"          # every position's logits are needed
        try:
            out = self.model(ids)
        finally:
            if prev is None:
                os.environ.pop("IPEX_LLM_LAST_LM_HEAD", None)
            else:
                os.environ["IPEX_LLM_LAST_LM_HEAD"] = prev
        logits = out.logits
        if logits.shape[1] != ids.shape[1]:
            raise RuntimeError("the model returned logits for the last position only; perplexity needs all of them")
        logp = torch.log_softmax(logits[:, :-1].float(), dim=-1)
        tgt = ids[:, 1:]
        tok = logp.gather(-1, tgt.unsqueeze(-1)).squeeze(-1)
        tok = tok[:, target_from:]
        return float(-tok.sum()), int(tok.numel())

    def perplexity_hf(self, token_stream: torch.Tensor, seq_len: int = 512, stride: int = None) -> float:
        """Perplexity of one long token stream ``[N]`` with windows of ``seq_len`` advanced by ``stride``."""
        stride = stride or seq_len
        n = token_stream.numel()
        total, count, prev_end = 0.0, 0, 0
        for begin in range(0, max(1, n - 1), stride):
            end = min(begin + seq_len, n)
            new = end - prev_end                       # tokens not scored by an earlier window
            window = token_stream[begin:end]
            if window.numel() < 2:
                break
            skip = max(0, window.numel() - 1 - new) if begin > 0 else 0
            s, c = self.nll(window, target_from=skip)
            total, count, prev_end = total + s, count + c, end
            if end == n:
                break
        return math.exp(total / max(1, count))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", required=True)
    ap.add_argument("--low_bit", default="sym_int4")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--text_file", default=None, help="plain text; default: random tokens (sanity run)")
    ap.add_argument("--seq_len", type=int, default=512)
    ap.add_argument("--stride", type=int, default=None)
    a = ap.parse_args(argv)
    ppl = BigDLPPL(a.model_path, a.device, load_in_low_bit=a.low_bit)
    if a.text_file:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
        with open(a.text_file) as f:
            ids = tok(f.read(), return_tensors="pt").input_ids[0]
    else:
        ids = torch.randint(0, ppl.model.config.vocab_size, (4 * a.seq_len,))
    print({"low_bit": a.low_bit, "tokens": int(ids.numel()), "seq_len": a.seq_len,
           "perplexity": round(ppl.perplexity_hf(ids, a.seq_len, a.stride), 4)})


if __name__ == "__main__":
    main()
