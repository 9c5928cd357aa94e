"""Synthetic request sets for the serving benchmark
(vllm_omni/benchmarks/data_modules/random_multi_modal_dataset.py): random text of a given
length with optional random image / audio / video attachments, reproducible from a seed."""
from __future__ import annotations

import base64
import io
import random
import struct
from dataclasses import dataclass, field


@dataclass
class BenchRequest:
    prompt: str
    prompt_len: int
    max_tokens: int
    content: list = field(default_factory=list)       # OpenAI chat content parts (text + media)
    modalities: list | None = None


_WORDS = ("the of and to in is that it for as with on be at by this from or an are not have they "
          "image sound voice picture describe explain answer scene color music speech motion").split()


def _png_b64(rng: random.Random, w: int, h: int) -> str:
    try:
        from PIL import Image
        img = Image.new("RGB", (w, h), (rng.randrange(256), rng.randrange(256), rng.randrange(256)))
        buf = io.BytesIO()
        img.save(buf, format="PNG")
        return base64.b64encode(buf.getvalue()).decode()
    except Exception:  # noqa: BLE001  (no Pillow: a 1x1 PNG)
        return ("iVBORw0KGgoAAAANSUhEUgAAAAEAAAABCAYAAAAfFcSJAAAADUlEQVR42mP8z8BQDwAEhQGAhKmMIQAAAABJRU5ErkJggg==")


def _wav_b64(rng: random.Random, seconds: float, rate: int = 16000) -> str:
    n = int(seconds * rate)
    data = b"".join(struct.pack("<h", rng.randrange(-2000, 2000)) for _ in range(n))
    hdr = b"RIFF" + struct.pack("<I", 36 + len(data)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, rate, rate * 2, 2, 16)
    return base64.b64encode(hdr + b"data" + struct.pack("<I", len(data)) + data).decode()


def random_multimodal_requests(n: int, input_len: int = 64, output_len: int = 32, images: int = 0, audios: int = 0,
                               image_size=(64, 64), audio_seconds: float = 1.0, seed: int = 0,
                               modalities=None) -> list[BenchRequest]:
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        text = " ".join(rng.choice(_WORDS) for _ in range(input_len))
        content = [{"type": "text", "text": text}]
        for _ in range(images):
            content.append({"type": "image_url", "image_url": {"url": "data:image/png;base64," + _png_b64(rng, *image_size)}})
        for _ in range(audios):
            content.append({"type": "input_audio", "input_audio": {"data": _wav_b64(rng, audio_seconds), "format": "wav"}})
        out.append(BenchRequest(text, input_len, output_len, content, modalities))
    return out
