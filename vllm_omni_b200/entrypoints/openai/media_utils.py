"""Image / audio / video (de)serialisation helpers for the HTTP layer
(vllm_omni/entrypoints/openai/{image_api_utils,audio_utils_mixin,video_api_utils}.py)."""
from __future__ import annotations

import base64
import io
import struct

import numpy as np
import torch


def parse_size(size: str | None, default=(1024, 1024)) -> tuple[int, int]:
    """'WxH' -> (width, height); raises ValueError on malformed or non-positive sizes."""
    if not size:
        return default
    parts = size.lower().replace("*", "x").split("x")
    if len(parts) != 2:
        raise ValueError(f"size must look like 1024x1024, got {size!r}")
    try:
        w, h = int(parts[0]), int(parts[1])
    except ValueError as e:
        raise ValueError(f"size must look like 1024x1024, got {size!r}") from e
    if w <= 0 or h <= 0:
        raise ValueError("size must be positive")
    return w, h


def encode_image_base64(img, fmt: str = "PNG") -> str:
    buf = io.BytesIO()
    img.save(buf, format=fmt)
    return base64.b64encode(buf.getvalue()).decode()


def decode_image_base64(data: str):
    from PIL import Image
    if data.startswith("data:"):
        data = data.split(",", 1)[1]
    return Image.open(io.BytesIO(base64.b64decode(data))).convert("RGB")


def wav_bytes(audio, sample_rate: int = 24000) -> bytes:
    """float waveform in [-1, 1] -> 16-bit PCM WAV container."""
    a = audio.detach().float().cpu().numpy() if isinstance(audio, torch.Tensor) else np.asarray(audio, dtype=np.float32)
    a = a.reshape(-1)
    pcm = (np.clip(a, -1.0, 1.0) * 32767.0).astype("<i2").tobytes()
    hdr = b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, sample_rate,
                                                                                 sample_rate * 2, 2, 16)
    return hdr + b"data" + struct.pack("<I", len(pcm)) + pcm


def pcm_bytes(audio) -> bytes:
    a = audio.detach().float().cpu().numpy() if isinstance(audio, torch.Tensor) else np.asarray(audio, dtype=np.float32)
    return (np.clip(a.reshape(-1), -1.0, 1.0) * 32767.0).astype("<i2").tobytes()


AUDIO_MEDIA_TYPES = {"wav": "audio/wav", "pcm": "audio/pcm", "flac": "audio/flac", "mp3": "audio/mpeg",
                     "aac": "audio/aac", "opus": "audio/ogg"}


def encode_audio(audio, sample_rate: int, fmt: str = "wav", speed: float = 1.0) -> tuple[bytes, str]:
    """wav and pcm are encoded here; compressed formats need an encoder library that this
    image does not ship, so they are refused with a clear message."""
    if speed and abs(speed - 1.0) > 1e-6:
        a = audio if isinstance(audio, torch.Tensor) else torch.as_tensor(np.asarray(audio))
        n = max(1, int(round(a.numel() / speed)))
        audio = torch.nn.functional.interpolate(a.reshape(1, 1, -1).float(), size=n, mode="linear",
                                                align_corners=False).reshape(-1)
    if fmt == "wav":
        return wav_bytes(audio, sample_rate), AUDIO_MEDIA_TYPES["wav"]
    if fmt == "pcm":
        return pcm_bytes(audio), AUDIO_MEDIA_TYPES["pcm"]
    raise ValueError(f"response_format {fmt!r} needs an audio encoder that is not installed; use wav or pcm")


def frames_to_gif_bytes(frames: np.ndarray, fps: int = 16) -> bytes:
    """[T, H, W, 3] uint8 -> animated GIF (PIL only; mp4 needs imageio/ffmpeg, absent here)."""
    from PIL import Image
    imgs = [Image.fromarray(f) for f in frames]
    buf = io.BytesIO()
    imgs[0].save(buf, format="GIF", save_all=True, append_images=imgs[1:], duration=int(1000 / max(fps, 1)), loop=0)
    return buf.getvalue()
