"""``python -m ipex_llm.serving.fastchat.model_worker``: FastChat's generic model worker command line on this package.

Counterpart of python/llm/src/ipex_llm/serving/fastchat/model_worker.py:75-506 (FastChat's ``ModelWorker`` with the
model loaded through the ipex-llm adapters, ``generate_stream_gate`` / ``generate_gate`` / ``get_embeddings``, heart
beats, the worker semaphore).  The worker itself is ``BigDLLLMWorker``: this module adds FastChat's argument names
(``--model-path`` with the ``bigdl`` / ``bigdl-lowbit`` path convention of the adapters, ``--device``,
``--load-in-low-bit``, ``--conv-template``, ``--embed-in-truncate``) and builds the same FastAPI application.
"""
from __future__ import annotations

import argparse
import uuid

from ..model_worker import ModelWorker as _BatchingWorker
from .bigdl_llm_model import load_model
from .ipex_llm_worker import BigDLLLMWorker, create_app  # noqa: F401


def heart_beat_worker(obj):
    """Body of the heart-beat thread (kept under FastChat's name)."""
    obj._heart_beat_loop()


class ModelWorker(BigDLLLMWorker):
    """FastChat-style worker: the model is loaded by the adapter that claims ``model_path``."""

    def __init__(self, controller_addr, worker_addr, worker_id, model_path, model_names=None,
                 limit_worker_concurrency: int = 5, no_register: bool = False, device: str = "cuda",
                 load_in_low_bit: str = None, conv_template: str = None, stream_interval: int = 2,
                 embed_in_truncate: bool = False, worker=None, **kwargs):
        self.conv_template, self.embed_in_truncate = conv_template, embed_in_truncate
        if worker is None:
            model, tok = load_model(model_path, device=device, load_in_low_bit=load_in_low_bit)
            worker = _BatchingWorker(model=model, tokenizer=tok, max_num_seqs=limit_worker_concurrency)
        super().__init__(controller_addr, worker_addr, worker_id, model_path, model_names, limit_worker_concurrency,
                         load_in_low_bit or "sym_int4", device, no_register, worker=worker,
                         stream_interval=stream_interval)

    def get_conv_template(self):
        conv = super().get_conv_template()
        if self.conv_template:
            conv["conv"]["name"] = self.conv_template
        return conv


def main(argv=None):
    import uvicorn
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="localhost")
    ap.add_argument("--port", type=int, default=21002)
    ap.add_argument("--worker-address", default="http://localhost:21002")
    ap.add_argument("--controller-address", default="http://localhost:21001")
    ap.add_argument("--model-path", required=True)
    ap.add_argument("--device", default="cuda", choices=["cpu", "cuda", "xpu"])
    ap.add_argument("--load-in-low-bit", default=None)
    ap.add_argument("--model-names", type=lambda s: s.split(","))
    ap.add_argument("--conv-template", default=None)
    ap.add_argument("--embed-in-truncate", action="store_true")
    ap.add_argument("--limit-worker-concurrency", type=int, default=5)
    ap.add_argument("--stream-interval", type=int, default=2)
    ap.add_argument("--no-register", action="store_true")
    a = ap.parse_args(argv)
    w = ModelWorker(a.controller_address, a.worker_address, str(uuid.uuid4())[:8], a.model_path, a.model_names,
                    a.limit_worker_concurrency, a.no_register, a.device, a.load_in_low_bit, a.conv_template,
                    a.stream_interval, a.embed_in_truncate)
    uvicorn.run(create_app(w), host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
