"""Multimodal request inputs for the omni thinker: raw images, audio clips and video frames from a chat
request become the tensors the thinker's towers take, and the message text gets one placeholder group
per item at the position the item had in the message.

The reference leaves this to vLLM's multimodal processor around the HF ``Qwen3OmniMoeProcessor``
(vllm_omni/model_executor/models/qwen3_omni/qwen3_omni_moe_thinker.py, the ``*MultiModalProcessor`` /
``*ProcessingInfo`` classes); here it is a few plain functions:

* image: "smart resize" (both sides rounded to a multiple of patch x merge, area kept inside
  [min_pixels, max_pixels], aspect ratio kept), bicubic, scaled to [-1, 1] -> ``[1, 3, H, W]``;
* video: the same per frame, frames sub-sampled to ``max_frames`` -> ``[T, 3, H, W]``;
* audio: mono, resampled to 16 kHz, Whisper log-mel with 128 bins, 100 frames per second -> ``[128, T]``.

The thinker expands each single placeholder token to the length of the item's features
(``Qwen3OmniMoeThinker.preprocess_request``), so the text carries ONE pad token per item, wrapped in the
start / end markers of the chat template.
"""
from __future__ import annotations

import base64
import io
import math
import wave

import numpy as np
import torch

PLACEHOLDER = {
    "image": "<|vision_start|><|image_pad|><|vision_end|>",
    "video": "<|vision_start|><|video_pad|><|vision_end|>",
    "audio": "<|audio_start|><|audio_pad|><|audio_end|>",
}
PLACEHOLDER_QWEN25 = {      # the Qwen2.5-Omni chat template's spelling
    "image": "<|vision_bos|><|IMAGE|><|vision_eos|>",
    "video": "<|vision_bos|><|VIDEO|><|vision_eos|>",
    "audio": "<|audio_bos|><|AUDIO|><|audio_eos|>",
}
AUDIO_RATE = 16000


def placeholders_for(style: str | None) -> dict:
    return PLACEHOLDER_QWEN25 if style == "qwen2_5_omni" else PLACEHOLDER


def smart_resize(height: int, width: int, factor: int = 32, min_pixels: int = 56 * 56, max_pixels: int = 1280 * 28 * 28) -> tuple[int, int]:
    """Target (height, width): multiples of ``factor``, area within [min_pixels, max_pixels], aspect ratio kept
    as closely as the rounding allows."""
    if min(height, width) <= 0:
        raise ValueError("empty image")
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200:1")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def image_to_pixels(image, factor: int = 32, min_pixels: int = 56 * 56, max_pixels: int = 1280 * 28 * 28) -> torch.Tensor:
    """PIL image / uint8 HWC array / float CHW tensor in [0, 1] -> [1, 3, H, W] in [-1, 1]."""
    from PIL import Image
    if isinstance(image, torch.Tensor):
        arr = (image.detach().float().clamp(0, 1) * 255).round().to(torch.uint8)
        arr = arr.permute(1, 2, 0).cpu().numpy() if arr.dim() == 3 and arr.shape[0] in (1, 3) else arr.cpu().numpy()
        image = Image.fromarray(arr.squeeze(-1) if arr.ndim == 3 and arr.shape[-1] == 1 else arr)
    elif isinstance(image, np.ndarray):
        image = Image.fromarray(image.astype(np.uint8))
    image = image.convert("RGB")
    h, w = smart_resize(image.height, image.width, factor, min_pixels, max_pixels)
    if (h, w) != (image.height, image.width):
        image = image.resize((w, h), Image.BICUBIC)
    x = torch.from_numpy(np.asarray(image, dtype=np.float32).copy()).permute(2, 0, 1) / 127.5 - 1.0
    return x[None].contiguous()


def video_to_pixels(frames, factor: int = 32, max_frames: int = 32, max_pixels: int = 768 * 28 * 28) -> torch.Tensor:
    """A list of frames (PIL / arrays / tensors) -> [T, 3, H, W]: evenly sub-sampled to ``max_frames``, all frames at
    the size chosen for the first one."""
    frames = list(frames)
    if not frames:
        raise ValueError("video without frames")
    if len(frames) > max_frames:
        idx = np.linspace(0, len(frames) - 1, max_frames).round().astype(int)
        frames = [frames[i] for i in idx]
    first = image_to_pixels(frames[0], factor, factor * factor, max_pixels)
    H, W = first.shape[-2:]
    out = [first]
    for f in frames[1:]:
        p = image_to_pixels(f, factor, factor * factor, max_pixels)
        if p.shape[-2:] != (H, W):
            p = torch.nn.functional.interpolate(p, size=(H, W), mode="bilinear", align_corners=False)
        out.append(p)
    return torch.cat(out, 0)


def decode_audio_bytes(blob: bytes) -> tuple[torch.Tensor, int]:
    """A RIFF/WAVE file (8 / 16 / 32-bit PCM) -> (mono float waveform in [-1, 1], sample rate).  Other containers
    need codec libraries this image does not have and are refused with a message."""
    if blob[:4] != b"RIFF" or blob[8:12] != b"WAVE":
        raise ValueError("audio input must be a WAV file (PCM); mp3 / ogg / flac decoding is not available")
    with wave.open(io.BytesIO(blob), "rb") as f:
        rate, n, width, ch = f.getframerate(), f.getnframes(), f.getsampwidth(), f.getnchannels()
        raw = f.readframes(n)
    if width == 2:
        x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
    elif width == 4:
        x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
    elif width == 1:
        x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    else:
        raise ValueError(f"unsupported WAV sample width {width}")
    x = x.reshape(-1, ch).mean(1) if ch > 1 else x
    return torch.from_numpy(np.ascontiguousarray(x)), int(rate)


def decode_data_url(data: str) -> bytes:
    """``data:<mime>;base64,<payload>`` or bare base64 -> bytes."""
    if data.startswith("data:"):
        data = data.split(",", 1)[1]
    return base64.b64decode(data)


def audio_to_mel(wave_: torch.Tensor, rate: int, n_mels: int = 128, max_seconds: float = 600.0) -> torch.Tensor:
    """Mono waveform -> [n_mels, frames] Whisper log-mel at 100 frames per second of 16 kHz audio."""
    from ..models.qwen3_tts.speaker import resample_sinc
    from ..models.qwen3_tts.tokenizer_25hz import whisper_log_mel
    w = torch.as_tensor(wave_, dtype=torch.float32).reshape(1, -1)
    if rate != AUDIO_RATE:
        w = resample_sinc(w, int(rate), AUDIO_RATE)
    w = w[0, : int(max_seconds * AUDIO_RATE)]
    if w.numel() < 400:
        w = torch.nn.functional.pad(w, (0, 400 - w.numel()))
    return whisper_log_mel(w, n_mels)


def gif_frames(blob: bytes) -> list:
    """Frames of an animated GIF / multi-frame image as RGB PIL images."""
    from PIL import Image, ImageSequence
    im = Image.open(io.BytesIO(blob))
    return [f.convert("RGB") for f in ImageSequence.Iterator(im)]


def thinker_inputs(mm: dict, vision_factor: int = 32, n_mels: int = 128, style: str | None = None) -> dict:
    """Raw items collected from a chat request ({"image": [PIL...], "audio": [(wave, rate)...], "video":
    [[frames]...]}) -> what ``Qwen3OmniMoeThinker.preprocess_request`` takes under the same keys."""
    out = {}
    if mm.get("image"):
        out["image"] = [image_to_pixels(im, vision_factor) for im in mm["image"]]
    if mm.get("video"):
        out["video"] = [video_to_pixels(v, vision_factor) for v in mm["video"]]
    if mm.get("audio"):
        out["audio"] = [audio_to_mel(w, r, n_mels) for w, r in mm["audio"]]
    return out


def processor_kwargs_for(model: str | None, stage_cfgs=None) -> dict:
    """``thinker_inputs`` keyword arguments for a served model: the vision rounding factor (patch x merge) and the
    number of mel bins, read from the checkpoint's ``config.json`` (``thinker_config.vision_config`` /
    ``audio_config``); tiny test geometries when a stage asks for them; the Qwen3-Omni values otherwise."""
    import json
    import os
    for sc in stage_cfgs or []:
        ov = (getattr(sc, "engine_args", None) or {}).get("model_overrides") or {}
        if ov.get("tiny") and (getattr(sc, "engine_args", {}) or {}).get("model_stage") == "thinker":
            from ..models.qwen3_omni.config import Qwen3OmniConfig
            c = Qwen3OmniConfig.tiny()
            return {"vision_factor": c.vision.patch_size * c.vision.spatial_merge_size, "n_mels": c.audio.num_mel_bins}
    out = {"vision_factor": 32, "n_mels": 128}
    path = os.path.join(model, "config.json") if model and os.path.isdir(model) else None
    if path and os.path.isfile(path):
        with open(path) as f:
            cfg = json.load(f)
        if "qwen2_5_omni" in str(cfg.get("model_type", "")):
            out["style"] = "qwen2_5_omni"
        th = cfg.get("thinker_config") or cfg
        v, a = th.get("vision_config") or {}, th.get("audio_config") or {}
        if v.get("patch_size"):
            out["vision_factor"] = int(v["patch_size"]) * int(v.get("spatial_merge_size", 2))
        if a.get("num_mel_bins"):
            out["n_mels"] = int(a["num_mel_bins"])
    return out
