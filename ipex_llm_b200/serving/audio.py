"""Audio helpers of the transcription endpoint: multipart form parsing, WAV decoding, resampling — standard library
and numpy only (no ``python-multipart``, ``librosa`` or ``soundfile`` at run time).

The reference's endpoint saves the upload and loads it with ``librosa`` at 16 kHz
(python/llm/src/ipex_llm/serving/fastapi/api_server.py:403-425, model_worker.py:100-118).
"""
from __future__ import annotations

import io
import wave
from email.parser import BytesParser
from email.policy import default as _policy
from typing import Dict, Tuple

import numpy as np


def parse_multipart(body: bytes, content_type: str) -> Dict[str, object]:
    """``{field: str}`` for text fields and ``{field: (filename, bytes)}`` for files of a multipart/form-data body."""
    head = f"Content-Type: {content_type}\r\nMIME-Version: 1.0\r\n\r\n".encode()
    msg = BytesParser(policy=_policy).parsebytes(head + body)
    out: Dict[str, object] = {}
    if not msg.is_multipart():
        return out
    for part in msg.iter_parts():
        name = part.get_param("name", header="content-disposition")
        if name is None:
            continue
        fname = part.get_filename()
        data = part.get_payload(decode=True) or b""
        out[name] = (fname, data) if fname is not None else data.decode("utf-8", "replace").strip()
    return out


def decode_wav(data: bytes) -> Tuple[np.ndarray, int]:
    """Mono float32 samples in [-1, 1] and the sampling rate of a PCM WAV file (8 / 16 / 32-bit integer)."""
    with wave.open(io.BytesIO(data), "rb") as w:
        rate, ch, width, n = w.getframerate(), w.getnchannels(), w.getsampwidth(), w.getnframes()
        raw = w.readframes(n)
    if width == 2:
        x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
    elif width == 4:
        x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
    elif width == 1:
        x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    else:
        raise ValueError(f"unsupported WAV sample width {width}")
    if ch > 1:
        x = x.reshape(-1, ch).mean(axis=1)
    return x, rate


def resample(x: np.ndarray, rate: int, target: int = 16000) -> np.ndarray:
    """Linear-interpolation resampling (speech models take 16 kHz)."""
    if rate == target or len(x) == 0:
        return x.astype(np.float32)
    n = max(1, int(round(len(x) * target / rate)))
    pos = np.linspace(0, len(x) - 1, n)
    return np.interp(pos, np.arange(len(x)), x).astype(np.float32)
