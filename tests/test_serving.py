"""HTTP serving on CPU: tiny random Llama + a word-level tokenizer built in the test, FastAPI TestClient."""
import json

import pytest
import torch


@pytest.fixture(scope="module")
def worker():
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import LlamaConfig, PreTrainedTokenizerFast
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.serving import ModelWorker
    words = ["<pad>", "<s>", "</s>", "<unk>"] + [f"w{i}" for i in range(60)]
    tk = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.Whitespace()
    tok = PreTrainedTokenizerFast(tokenizer_object=tk, pad_token="<pad>", bos_token="<s>", eos_token="</s>",
                                  unk_token="<unk>", padding_side="left")
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=64, max_position_embeddings=256, tie_word_embeddings=False,
                      eos_token_id=2, pad_token_id=0, bos_token_id=1)
    model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="sym_int8", torch_dtype=torch.float32, device="cpu")
    w = ModelWorker(model=model.eval(), tokenizer=tok, max_num_seqs=4)
    yield w
    w.shutdown()


def test_pipeline_token_emitter():
    """The first stage's per-step streamer: deltas per request, stop strings held back and cut, eos, token limits."""
    from ipex_llm_b200.serving.model_worker import SamplingParams
    from ipex_llm_b200.serving.pp_worker import _TokenEmitter

    class Tok:
        eos_token_id = 2

        def decode(self, ids, **kw):
            return "".join(chr(ord("a") + (i % 26)) for i in ids)

    class Req:
        def __init__(self, max_new_tokens, stop):
            self.params = SamplingParams(max_new_tokens=max_new_tokens, stop=stop)
            self.pieces = []

        def emit(self, s):
            self.pieces.append(s)

    reqs = [Req(10, []), Req(3, []), Req(10, ["hi"]), Req(10, [])]
    em = _TokenEmitter(Tok(), reqs)
    em.put(torch.zeros(4, 5, dtype=torch.long))                 # prompt
    # per step: request 0 spells "defg...", 1 is cut by its limit, 2 runs into the stop string "hi", 3 ends with eos
    steps = [[3, 3, 6, 3], [4, 4, 7, 2], [5, 5, 8, 9], [6, 6, 9, 9], [7, 7, 10, 9]]
    for s in steps:
        em.put(torch.tensor(s))
    em.end()
    assert "".join(reqs[0].pieces) == "defgh" and len(reqs[0].pieces) == 5      # one delta per token
    assert "".join(reqs[1].pieces) == "def"                                      # max_new_tokens = 3
    assert "".join(reqs[2].pieces) == "g" and em.done[2]                         # "h" held back, then "hi" cut
    assert "".join(reqs[3].pieces) == "d" and em.done[3]                         # eos at the second step
    assert em.sent[0] == 5 and em.prefix[2] == "g"


def test_batch_streamer_incremental_text():
    from ipex_llm.transformers.streamer import BatchTextIteratorStreamer

    class Tok:
        def decode(self, ids, **kw):
            return " ".join(f"w{i}" for i in ids)
    s = BatchTextIteratorStreamer(2, Tok(), skip_prompt=True)
    s.put(torch.tensor([[1, 2], [3, 4]]))          # prompt: skipped
    s.put(torch.tensor([5, 6]))
    s.put(torch.tensor([7, 8]))
    s.end()
    chunks = list(s)
    assert "".join(c[0] for c in chunks) == "w5 w7" and "".join(c[1] for c in chunks) == "w6 w8"


def test_generate_and_openai_endpoints(worker):
    from fastapi.testclient import TestClient
    from ipex_llm_b200.serving import FastApp
    with TestClient(FastApp(worker, served_model_name="tiny").app) as c:
        assert c.get("/health").text == "OK"
        assert c.get("/v1/models").json()["data"][0]["id"] == "tiny"
        r = c.post("/generate", json={"inputs": "w1 w2 w3", "parameters": {"max_new_tokens": 6}}).json()
        assert r["generated_tokens"] <= 6 and r["prompt_tokens"] == 3 and isinstance(r["generated_text"], str)
        ref = worker.submit_blocking("w1 w2 w3", __import__("ipex_llm_b200.serving", fromlist=["SamplingParams"])
                                     .SamplingParams(max_new_tokens=6))
        assert ref.text == r["generated_text"]          # batching / streaming does not change greedy output
        r = c.post("/v1/completions", json={"model": "tiny", "prompt": ["w4 w5", "w6 w7 w8 w9"], "max_tokens": 5,
                                            "temperature": 1.0}).json()
        assert len(r["choices"]) == 2 and r["usage"]["prompt_tokens"] == 6
        r = c.post("/v1/chat/completions", json={"model": "tiny", "max_tokens": 4, "messages": [
            {"role": "user", "content": "w1 w2"}]}).json()
        assert r["choices"][0]["message"]["role"] == "assistant" and r["usage"]["completion_tokens"] <= 4
        m = c.get("/metrics").text
        assert "ipex_llm_requests_total" in m


def test_streaming_endpoints(worker):
    from fastapi.testclient import TestClient
    from ipex_llm_b200.serving import FastApp
    with TestClient(FastApp(worker, served_model_name="tiny").app) as c:
        full = c.post("/generate", json={"inputs": "w9 w8", "parameters": {"max_new_tokens": 8}}).json()
        with c.stream("POST", "/generate_stream", json={"inputs": "w9 w8", "parameters": {"max_new_tokens": 8}}) as r:
            events = [json.loads(l[6:]) for l in r.iter_lines() if l.startswith("data: ")]
        assert "".join(e["token"]["text"] for e in events) == full["generated_text"]
        assert events[-1]["finish_reason"] in ("length", "stop")
        with c.stream("POST", "/v1/chat/completions", json={"model": "tiny", "stream": True, "max_tokens": 5,
                                                            "messages": [{"role": "user", "content": "w3"}]}) as r:
            lines = [l[6:] for l in r.iter_lines() if l.startswith("data: ")]
        assert lines[-1] == "[DONE]"
        chunks = [json.loads(l) for l in lines[:-1]]
        assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
        assert chunks[-1]["choices"][0]["finish_reason"] in ("stop", "length")


def test_stop_string_truncates(worker):
    from ipex_llm_b200.serving import SamplingParams
    base = worker.submit_blocking("w1 w2", SamplingParams(max_new_tokens=10))
    words = base.text.split()
    if len(words) >= 3:
        stop = words[2]
        cut = worker.submit_blocking("w1 w2", SamplingParams(max_new_tokens=10, stop=[stop]))
        assert stop not in cut.text and base.text.startswith(cut.text)
        assert cut.finish_reason == "stop"


def test_fastchat_protocol_worker(worker):
    from fastapi.testclient import TestClient
    from ipex_llm_b200.serving.fastchat.ipex_llm_worker import BigDLLLMWorker, create_app
    w = BigDLLLMWorker(None, "http://localhost:21002", "w0", "tiny", worker=worker, no_register=True,
                       stream_interval=1)
    with TestClient(create_app(w)) as c:
        st = c.post("/worker_get_status").json()
        assert st["model_names"] == ["tiny"]
        assert c.post("/count_token", json={"prompt": "w1 w2 w3"}).json()["count"] == 3
        r = c.post("/worker_generate", json={"prompt": "w1 w2", "max_new_tokens": 5, "temperature": 0.0,
                                             "echo": False}).json()
        assert r["error_code"] == 0 and r["usage"]["completion_tokens"] <= 5
        with c.stream("POST", "/worker_generate_stream", json={"prompt": "w1 w2", "max_new_tokens": 5,
                                                              "temperature": 0.0, "echo": False}) as resp:
            chunks = [json.loads(x) for x in resp.read().split(b"\0") if x]
        assert chunks[-1]["text"] == r["text"] and chunks[-1]["finish_reason"] in ("length", "stop")


def test_fastchat_embeddings_adapters_and_generic_worker(worker, tmp_path):
    """``/worker_get_embeddings``; the ``bigdl`` / ``bigdl-lowbit`` path adapters (reference
    serving/fastchat/bigdl_llm_model.py); the generic ``model_worker.ModelWorker`` on an adapter-loaded model."""
    from fastapi.testclient import TestClient
    from ipex_llm_b200.serving.fastchat import bigdl_llm_model as adapters
    from ipex_llm_b200.serving.fastchat.model_worker import ModelWorker, create_app
    w = ModelWorker(None, "http://localhost:21002", "w0", "tiny", worker=worker, no_register=True,
                    conv_template="vicuna_v1.1")
    with TestClient(create_app(w)) as c:
        r = c.post("/worker_get_embeddings", json={"input": ["w1 w2 w3", "w4"]}).json()
        assert len(r["embedding"]) == 2 and r["token_num"] == 4
        n0 = sum(x * x for x in r["embedding"][0]) ** 0.5
        assert abs(n0 - 1.0) < 1e-4
        assert c.post("/worker_get_conv_template").json()["conv"]["name"] == "vicuna_v1.1"
    assert isinstance(adapters.get_model_adapter("/models/bigdl-7b"), adapters.BigDLLLMAdapter)
    assert isinstance(adapters.get_model_adapter("/models/BigDL-LowBit-7b"), adapters.BigDLLMLOWBITAdapter)
    assert adapters.get_model_adapter("/models/vicuna") is None
    assert adapters.patch_fastchat() in (True, False)            # FastChat is optional
    # both adapters load the same tiny checkpoint to the same logits
    import torch
    src = str(tmp_path / "bigdl-tiny")
    worker.model.save_low_bit(str(tmp_path / "bigdl-lowbit-tiny"))
    worker.tokenizer.save_pretrained(str(tmp_path / "bigdl-lowbit-tiny"))
    m_low, tok = adapters.load_model(str(tmp_path / "bigdl-lowbit-tiny"), device="cpu")
    ids = torch.tensor([[5, 6, 7]])
    with torch.no_grad():
        assert torch.equal(m_low(ids).logits, worker.model(ids).logits)
    assert tok.decode([5]) == worker.tokenizer.decode([5]) and src


def test_audio_transcription_endpoint(monkeypatch):
    """multipart upload of a WAV file -> decoded, resampled to 16 kHz, handed to the worker's speech model."""
    import io
    import wave

    import numpy as np
    from fastapi.testclient import TestClient
    from ipex_llm_b200.serving.api_server import FastApp
    from ipex_llm_b200.serving.audio import decode_wav, parse_multipart, resample

    rate = 8000
    t = np.arange(rate // 2) / rate
    pcm = (np.sin(2 * np.pi * 440 * t) * 20000).astype("<i2")
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(rate)
        w.writeframes(pcm.tobytes())
    wav = buf.getvalue()
    x, r = decode_wav(wav)
    assert r == rate and abs(float(np.abs(x).max()) - 20000 / 32768) < 1e-3
    assert len(resample(x, r)) == len(x) * 2

    seen = {}

    class Worker:
        model_name = "fake-whisper"
        tokenizer = None
        stats = {"requests": 0, "batches": 0, "generated_tokens": 0, "first_token_s": [], "next_token_s": []}

        def transcribe(self, samples, language=None):
            seen["n"], seen["language"] = len(samples), language
            return "hello world"

    client = TestClient(FastApp(Worker()).app)
    boundary = "----ipexllmtest"
    body = (f"--{boundary}\r\nContent-Disposition: form-data; name=\"language\"\r\n\r\nen\r\n"
            f"--{boundary}\r\nContent-Disposition: form-data; name=\"file\"; filename=\"a.wav\"\r\n"
            f"Content-Type: audio/wav\r\n\r\n").encode() + wav + f"\r\n--{boundary}--\r\n".encode()
    form = parse_multipart(body, f"multipart/form-data; boundary={boundary}")
    assert form["language"] == "en" and form["file"][0] == "a.wav" and form["file"][1] == wav
    resp = client.post("/v1/audio/transcriptions", content=body,
                       headers={"content-type": f"multipart/form-data; boundary={boundary}"})
    assert resp.status_code == 200 and resp.json() == {"text": "hello world"}
    assert seen == {"n": len(x) * 2, "language": "en"}
    bad = client.post("/v1/audio/transcriptions", content=b"x", headers={"content-type": "text/plain"})
    assert bad.status_code == 400


def test_tgi_api_server_relays_fastchat_worker_stream():
    """``TGIApp`` turns a FastChat worker's NUL-delimited cumulative-text stream into TGI ``/generate`` and
    ``/generate_stream`` responses (worker looked up through a controller; the transport is a double)."""
    import json as _json
    from starlette.testclient import TestClient
    from ipex_llm_b200.serving.fastchat.tgi_api_server import TGIApp

    class _Transport:
        def __init__(self):
            self.posts = []

        async def post_json(self, url, payload):
            self.posts.append((url, payload))
            if url.endswith("/list_models"):
                return {"models": ["tiny"]}
            return {"address": "http://worker:1"}

        async def post_stream(self, url, payload):
            self.posts.append((url, payload))
            chunks = [{"text": "Hel", "error_code": 0}, {"text": "Hello", "error_code": 0},
                      {"text": "Hello!", "error_code": 0, "finish_reason": "stop",
                       "usage": {"completion_tokens": 3}}]
            raw = b"".join(_json.dumps(c).encode() + b"\0" for c in chunks)
            yield raw[:20]                      # chunks split across reads
            yield raw[20:]

    tr = _Transport()
    client = TestClient(TGIApp(controller_address="http://ctl", transport=tr).app)
    r = client.post("/generate", json={"inputs": "Hi", "parameters": {"max_new_tokens": 5, "details": True,
                                                                      "do_sample": False, "stop": ["\n"]}})
    assert r.status_code == 200
    body = r.json()
    assert body["generated_text"] == "Hello!" and body["details"]["finish_reason"] == "stop"
    assert body["details"]["generated_tokens"] == 3
    url, payload = [p for p in tr.posts if p[0].endswith("/worker_generate_stream")][0]
    assert url == "http://worker:1/worker_generate_stream"
    assert payload["prompt"] == "Hi" and payload["max_new_tokens"] == 5 and payload["temperature"] == 0.0
    assert payload["stop"] == ["\n"] and payload["model"] == ""
    with client.stream("POST", "/generate_stream", json={"inputs": "Hi"}) as s:
        events = [_json.loads(line[6:]) for line in s.iter_lines() if line.startswith("data: ")]
    assert [e["token"]["text"] for e in events] == ["Hel", "lo", "!"]
    assert events[-1]["generated_text"] == "Hello!" and events[-1]["details"]["finish_reason"] == "stop"
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"


def test_fastchat_vllm_worker_streams_engine_outputs():
    """``VLLMWorker`` maps FastChat parameters to vLLM sampling arguments and streams the engine's cumulative outputs
    as NUL-delimited chunks (an async double stands in for the vLLM engine)."""
    import json as _json
    from starlette.testclient import TestClient
    from ipex_llm_b200.serving.fastchat.vllm_worker import VLLMWorker, create_app

    class _Out:
        def __init__(self, text, ids, finished):
            self.outputs = [type("O", (), {"text": text, "token_ids": ids, "cumulative_logprob": -1.0,
                                           "finish_reason": "stop" if finished else None})()]
            self.prompt_token_ids = [1, 2, 3]
            self.finished = finished

    class _Engine:
        def __init__(self):
            self.calls = []

        async def generate(self, prompt, sampling, request_id):
            self.calls.append((prompt, sampling, request_id))
            yield _Out(" a", [5], False)
            yield _Out(" a b", [5, 6], True)

    eng = _Engine()
    w = VLLMWorker(None, "http://w", "id0", "/models/tiny", engine=eng)
    kw = VLLMWorker.sampling_kwargs({"temperature": 0.0, "top_p": 0.3, "max_new_tokens": 9, "stop": "###"})
    assert kw["temperature"] == 0.0 and kw["top_p"] == 1.0 and kw["max_tokens"] == 9 and kw["stop"] == ["###"]
    client = TestClient(create_app(w))
    r = client.post("/worker_generate", json={"prompt": "x", "max_new_tokens": 4, "echo": False})
    body = r.json()
    assert body["text"] == " a b" and body["finish_reason"] == "stop"
    assert body["usage"] == {"prompt_tokens": 3, "completion_tokens": 2, "total_tokens": 5}
    with client.stream("POST", "/worker_generate_stream", json={"prompt": "x", "echo": True}) as s:
        raw = b"".join(s.iter_bytes())
    chunks = [_json.loads(c) for c in raw.split(b"\0") if c]
    assert [c["text"] for c in chunks] == ["x a", "x a b"] and chunks[0]["finish_reason"] is None
    assert client.post("/worker_get_status").json()["model_names"] == ["tiny"]
    assert eng.calls[0][0] == "x"
