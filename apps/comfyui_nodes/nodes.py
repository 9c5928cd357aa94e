"""HTTP client nodes: image generation, image editing, speech, omni chat.

Every node is a plain class with ComfyUI's conventions (``INPUT_TYPES``, ``RETURN_TYPES``,
``FUNCTION``, ``CATEGORY``); images cross the node boundary as float tensors [B, H, W, 3] in
[0, 1], audio as ``{"waveform": [1, 1, T], "sample_rate": int}``.  Only ``requests``, ``numpy``
and Pillow are needed on the ComfyUI side; ``torch`` is used when present (ComfyUI ships it).
"""
from __future__ import annotations

import base64
import io
import json
import wave

import numpy as np


def _to_tensor(arr: np.ndarray):
    try:
        import torch
        return torch.from_numpy(arr)
    except Exception:  # noqa: BLE001
        return arr


def _png_to_image(b64: str):
    from PIL import Image
    im = Image.open(io.BytesIO(base64.b64decode(b64))).convert("RGB")
    return np.asarray(im, dtype=np.float32)[None] / 255.0


def _image_to_png(image) -> bytes:
    from PIL import Image
    arr = np.asarray(image.cpu() if hasattr(image, "cpu") else image)
    arr = (np.clip(arr[0] if arr.ndim == 4 else arr, 0, 1) * 255).astype(np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    return buf.getvalue()


def _wav_to_audio(blob: bytes):
    with wave.open(io.BytesIO(blob), "rb") as f:
        rate, n, width, ch = f.getframerate(), f.getnframes(), f.getsampwidth(), f.getnchannels()
        raw = f.readframes(n)
    pcm = np.frombuffer(raw, dtype=np.int16 if width == 2 else np.uint8).astype(np.float32)
    pcm = pcm / (32768.0 if width == 2 else 128.0)
    return {"waveform": _to_tensor(pcm.reshape(-1, ch).T[None].copy()), "sample_rate": rate}


def _post(url, **kw):
    import requests
    r = requests.post(url, timeout=kw.pop("timeout", 1800), **kw)
    if r.status_code != 200:
        raise RuntimeError(f"{url}: HTTP {r.status_code}: {r.text[:300]}")
    return r


class OmniImageGenerate:
    CATEGORY = "omni"
    RETURN_TYPES = ("IMAGE",)
    FUNCTION = "run"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Qwen/Qwen-Image"}),
                             "prompt": ("STRING", {"multiline": True, "default": ""}),
                             "width": ("INT", {"default": 1024, "min": 64, "max": 4096, "step": 16}),
                             "height": ("INT", {"default": 1024, "min": 64, "max": 4096, "step": 16}),
                             "steps": ("INT", {"default": 50, "min": 1, "max": 200}),
                             "cfg": ("FLOAT", {"default": 4.0, "min": 0.0, "max": 20.0}),
                             "seed": ("INT", {"default": 0, "min": 0, "max": 2 ** 31 - 1})},
                "optional": {"negative_prompt": ("STRING", {"multiline": True, "default": " "}),
                             "n": ("INT", {"default": 1, "min": 1, "max": 8})}}

    def run(self, server, model, prompt, width, height, steps, cfg, seed, negative_prompt=" ", n=1):
        body = {"model": model, "prompt": prompt, "negative_prompt": negative_prompt, "size": f"{width}x{height}",
                "num_inference_steps": steps, "true_cfg_scale": cfg, "seed": seed, "n": n}
        data = _post(server.rstrip("/") + "/v1/images/generations", json=body).json()["data"]
        return (_to_tensor(np.concatenate([_png_to_image(d["b64_json"]) for d in data], 0)),)


class OmniImageEdit:
    CATEGORY = "omni"
    RETURN_TYPES = ("IMAGE",)
    FUNCTION = "run"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Qwen/Qwen-Image-Edit"}),
                             "image": ("IMAGE",), "prompt": ("STRING", {"multiline": True, "default": ""}),
                             "steps": ("INT", {"default": 40, "min": 1, "max": 200}),
                             "seed": ("INT", {"default": 0, "min": 0, "max": 2 ** 31 - 1})}}

    def run(self, server, model, image, prompt, steps, seed):
        files = {"image": ("image.png", _image_to_png(image), "image/png")}
        form = {"model": model, "prompt": prompt, "num_inference_steps": str(steps), "seed": str(seed)}
        data = _post(server.rstrip("/") + "/v1/images/edits", files=files, data=form).json()["data"]
        return (_to_tensor(_png_to_image(data[0]["b64_json"])),)


class OmniSpeech:
    CATEGORY = "omni"
    RETURN_TYPES = ("AUDIO",)
    FUNCTION = "run"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Qwen/Qwen3-TTS"}),
                             "text": ("STRING", {"multiline": True, "default": ""}),
                             "voice": ("STRING", {"default": "default"})}}

    def run(self, server, model, text, voice):
        r = _post(server.rstrip("/") + "/v1/audio/speech",
                  json={"model": model, "input": text, "voice": voice, "response_format": "wav"}, timeout=600)
        return (_wav_to_audio(r.content),)


class OmniChat:
    """Chat completion with optional image input; returns the reply text and, when the model speaks, audio."""
    CATEGORY = "omni"
    RETURN_TYPES = ("STRING", "AUDIO")
    FUNCTION = "run"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Qwen/Qwen3-Omni-30B-A3B-Instruct"}),
                             "prompt": ("STRING", {"multiline": True, "default": ""}),
                             "speak": ("BOOLEAN", {"default": True})},
                "optional": {"image": ("IMAGE",)}}

    def run(self, server, model, prompt, speak, image=None):
        content = [{"type": "text", "text": prompt}]
        if image is not None:
            b64 = base64.b64encode(_image_to_png(image)).decode()
            content.append({"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}})
        body = {"model": model, "messages": [{"role": "user", "content": content}],
                "modalities": ["text", "audio"] if speak else ["text"]}
        out = _post(server.rstrip("/") + "/v1/chat/completions", json=body, timeout=600).json()
        text, audio = "", {"waveform": _to_tensor(np.zeros((1, 1, 0), np.float32)), "sample_rate": 24000}
        for ch in out.get("choices", []):
            msg = ch.get("message") or {}
            if msg.get("content"):
                text += msg["content"] if isinstance(msg["content"], str) else json.dumps(msg["content"])
            if (msg.get("audio") or {}).get("data"):
                audio = _wav_to_audio(base64.b64decode(msg["audio"]["data"]))
        return (text, audio)


NODE_CLASS_MAPPINGS = {"OmniImageGenerate": OmniImageGenerate, "OmniImageEdit": OmniImageEdit,
                       "OmniSpeech": OmniSpeech, "OmniChat": OmniChat}
NODE_DISPLAY_NAME_MAPPINGS = {"OmniImageGenerate": "Omni: generate image", "OmniImageEdit": "Omni: edit image",
                              "OmniSpeech": "Omni: text to speech", "OmniChat": "Omni: chat (text / audio)"}
