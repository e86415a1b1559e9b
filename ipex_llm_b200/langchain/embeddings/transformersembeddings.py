"""``TransformersEmbeddings``: sentence embeddings from a low-bit model's last hidden state, mean pooled
(reference: python/llm/src/ipex_llm/langchain/embeddings/transformersembeddings.py:56-180)."""
from __future__ import annotations

from typing import List, Optional

DEFAULT_MODEL_NAME = "gpt2"


class TransformersEmbeddings:
    def __init__(self, model=None, tokenizer=None, model_id: str = DEFAULT_MODEL_NAME, model_kwargs: Optional[dict] = None,
                 encode_kwargs: Optional[dict] = None):
        self.model, self.tokenizer, self.model_id = model, tokenizer, model_id
        self.model_kwargs, self.encode_kwargs = model_kwargs, dict(encode_kwargs or {})

    @classmethod
    def from_model_id(cls, model_id: str, model_kwargs: Optional[dict] = None, device_map: str = "cuda", **kwargs):
        import torch
        from transformers import AutoTokenizer
        from ...transformers import AutoModel
        kw = dict(model_kwargs or {})
        tok = AutoTokenizer.from_pretrained(model_id)
        model = AutoModel.from_pretrained(model_id, load_in_4bit=True, **kw)
        if device_map in ("cuda", "xpu", "gpu") and torch.cuda.is_available():
            model = model.to("cuda")
        return cls(model=model, tokenizer=tok, model_id=model_id, model_kwargs=kw, **kwargs)

    def embed(self, text: str, **kwargs) -> List[float]:
        import torch
        dev = next(self.model.parameters()).device
        enc = self.tokenizer(text, return_tensors="pt", **{**self.encode_kwargs, **kwargs})
        ids = enc["input_ids"].to(dev)
        with torch.no_grad():
            out = self.model(input_ids=ids, output_hidden_states=True)
        hidden = out.hidden_states[-1] if getattr(out, "hidden_states", None) is not None else out.last_hidden_state
        return hidden[0].float().mean(dim=0).cpu().tolist()

    def embed_documents(self, texts: List[str], **kwargs) -> List[List[float]]:
        return [self.embed(t.replace("\n", " "), **kwargs) for t in texts]

    def embed_query(self, text: str, **kwargs) -> List[float]:
        return self.embed(text.replace("\n", " "), **kwargs)


class TransformersBgeEmbeddings(TransformersEmbeddings):
    """BGE-style sentence vector: the first token's last hidden state, L2-normalised (reference
    transformersembeddings.py:188-195)."""

    def embed(self, text: str, **kwargs) -> List[float]:
        import torch
        dev = next(self.model.parameters()).device
        enc = self.tokenizer(text, return_tensors="pt", **{**self.encode_kwargs, **kwargs})
        with torch.no_grad():
            out = self.model(input_ids=enc["input_ids"].to(dev), output_hidden_states=True)
        hidden = out.hidden_states[-1] if getattr(out, "hidden_states", None) is not None else out.last_hidden_state
        return torch.nn.functional.normalize(hidden[:, 0].float(), p=2, dim=1)[0].cpu().tolist()
