"""llama-cpp-python style classes (``Llama(model_path)(prompt, max_tokens=...) -> completion dict``).

The reference binds one native C library per family through ctypes
(python/llm/src/ipex_llm/ggml/model/{llama,bloom,gptneox,starcoder,chatglm}/, ~7000 lines) and exposes
``Llama`` / ``Bloom`` / ``Gptneox`` / ``Starcoder`` / ``ChatGLM`` plus ``ipex_llm.models``.  This package has one
runtime for every architecture, so the classes share one implementation: ``model_path`` may be a Hugging Face
checkpoint directory, a ``save_low_bit`` directory (what ``llm_convert`` writes) or a ``.gguf`` file.
"""
from __future__ import annotations

import os
import time
import uuid
from typing import Iterator, List, Optional, Union

from .generation import GenerationMixin


class GenericModel(GenerationMixin):
    family = "llama"

    def __init__(self, model_path: str, n_ctx: int = 512, n_threads: int = -1, seed: int = -1, n_batch: int = 512,
                 embedding: bool = False, verbose: bool = True, low_bit: str = "sym_int4", device: str = "auto",
                 **kwargs):
        import torch
        from ...cli.llm_cli import _load
        self.model_path, self.n_ctx, self.embedding = model_path, n_ctx, embedding
        if n_threads and n_threads > 0:
            torch.set_num_threads(n_threads)
        if seed is not None and seed >= 0:
            torch.manual_seed(seed)
        self.model, self.tokenizer = _load(model_path, low_bit, device)

    # ---- tokens ---------------------------------------------------------------------------------------
    def tokenize(self, text: Union[str, bytes], add_bos: bool = True) -> List[int]:
        if isinstance(text, bytes):
            text = text.decode("utf-8", errors="ignore")
        return list(self.tokenizer.encode(text, add_special_tokens=add_bos))

    def detokenize(self, tokens: List[int]) -> bytes:
        return self.tokenizer.decode(tokens, skip_special_tokens=True).encode("utf-8")

    # ---- completion -----------------------------------------------------------------------------------
    def _gen_kwargs(self, max_tokens, temperature, top_p, top_k, repeat_penalty):
        kw = dict(max_new_tokens=max_tokens, do_sample=temperature is not None and temperature > 0)
        if kw["do_sample"]:
            kw.update(temperature=temperature, top_p=top_p)
            if top_k and top_k > 0:
                kw["top_k"] = top_k
        if repeat_penalty and repeat_penalty != 1.0:
            kw["repetition_penalty"] = repeat_penalty
        return kw

    def create_completion(self, prompt: str, max_tokens: int = 128, temperature: float = 0.0, top_p: float = 0.95,
                          top_k: int = 40, stop: Optional[List[str]] = None, echo: bool = False,
                          repeat_penalty: float = 1.0, stream: bool = False, **kwargs):
        import torch
        dev = next(self.model.parameters()).device
        ids = self.tokenizer(prompt, return_tensors="pt")["input_ids"].to(dev)
        kw = self._gen_kwargs(max_tokens, temperature, top_p, top_k, repeat_penalty)
        cid, created = f"cmpl-{uuid.uuid4()}", int(time.time())

        def pack(text, finish):
            return {"id": cid, "object": "text_completion", "created": created, "model": self.model_path,
                    "choices": [{"text": text, "index": 0, "logprobs": None, "finish_reason": finish}]}

        def cut(text):
            for s in stop or []:
                i = text.find(s)
                if i >= 0:
                    return text[:i], True
            return text, False

        if stream:
            def it() -> Iterator[dict]:
                from threading import Thread
                from transformers import TextIteratorStreamer
                st = TextIteratorStreamer(self.tokenizer, skip_prompt=True, skip_special_tokens=True)
                th = Thread(target=lambda: self.model.generate(ids, streamer=st, **kw), daemon=True)
                th.start()
                acc = ""
                for piece in st:
                    acc += piece
                    txt, hit = cut(acc)
                    if hit:
                        yield pack(txt[len(acc) - len(piece):], "stop")
                        break
                    yield pack(piece, None)
                th.join()
                yield pack("", "length")
            return it()
        with torch.no_grad():
            out = self.model.generate(ids, **kw)
        new = out[0][ids.shape[1]:]
        text, hit = cut(self.tokenizer.decode(new, skip_special_tokens=True))
        res = pack((prompt if echo else "") + text, "stop" if hit or len(new) < max_tokens else "length")
        res["usage"] = {"prompt_tokens": int(ids.shape[1]), "completion_tokens": int(len(new)),
                        "total_tokens": int(ids.shape[1] + len(new))}
        return res

    def __call__(self, prompt: str, **kwargs):
        return self.create_completion(prompt, **kwargs)

    def _generate_ids(self, tokens: List[int], max_tokens, temp, top_p, top_k, repeat_penalty) -> List[int]:
        import torch
        dev = next(self.model.parameters()).device
        ids = torch.tensor([tokens], device=dev)
        with torch.no_grad():
            out = self.model.generate(ids, **self._gen_kwargs(max_tokens, temp, top_p, top_k, repeat_penalty))
        return out[0][len(tokens):].tolist()

    def _generate(self, tokens: List[int], top_k: int = 40, top_p: float = 0.95, temp: float = 0.0,
                  repeat_penalty: float = 1.0, max_tokens: int = 128, **kwargs) -> Iterator[int]:
        """Generator over the new tokens of one prompt (the llama-cpp form of ``generate``)."""
        yield from self._generate_ids(tokens, max_tokens, temp, top_p, top_k, repeat_penalty)

    def embed(self, text: str) -> List[float]:
        import torch
        dev = next(self.model.parameters()).device
        ids = self.tokenizer(text, return_tensors="pt")["input_ids"].to(dev)
        with torch.no_grad():
            out = self.model(input_ids=ids, output_hidden_states=True)
        return out.hidden_states[-1][0].float().mean(dim=0).cpu().tolist()

    def create_embedding(self, input: Union[str, List[str]]):
        texts = [input] if isinstance(input, str) else list(input)
        data = [{"object": "embedding", "embedding": self.embed(t), "index": i} for i, t in enumerate(texts)]
        return {"object": "list", "data": data, "model": self.model_path}


class Llama(GenericModel):
    family = "llama"


class Bloom(GenericModel):
    family = "bloom"


class Gptneox(GenericModel):
    family = "gptneox"


class Starcoder(GenericModel):
    family = "starcoder"


class ChatGLM(GenericModel):
    family = "chatglm"
