"""HTTP client nodes: image generation, image editing, video, speech, voice cloning, omni chat with image /
audio / video inputs, and parameter nodes (per-stage sampling parameters, Qwen-TTS options) that plug into them.

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


def _audio_to_wav(audio) -> bytes:
    """ComfyUI audio ({"waveform": [B, C, T], "sample_rate"}) -> 16-bit WAV bytes of the first item."""
    w = audio["waveform"]
    arr = np.asarray(w.cpu() if hasattr(w, "cpu") else w, dtype=np.float32)
    arr = arr[0] if arr.ndim == 3 else arr
    pcm = (np.clip(arr.T, -1, 1) * 32767).astype("<i2")           # [T, C]
    buf = io.BytesIO()
    with wave.open(buf, "wb") as f:
        f.setnchannels(pcm.shape[1])
        f.setsampwidth(2)
        f.setframerate(int(audio["sample_rate"]))
        f.writeframes(pcm.tobytes())
    return buf.getvalue()


def _frames_to_gif(frames, fps: int = 8) -> bytes:
    from PIL import Image
    arr = np.asarray(frames.cpu() if hasattr(frames, "cpu") else frames)
    ims = [Image.fromarray((np.clip(a, 0, 1) * 255).astype(np.uint8)) for a in arr]
    buf = io.BytesIO()
    ims[0].save(buf, format="GIF", save_all=True, append_images=ims[1:], duration=int(1000 / fps), loop=0)
    return buf.getvalue()


def check_server(server: str, model: str):
    """ComfyUI ``VALIDATE_INPUTS`` helper: True or the message shown on the node."""
    if not isinstance(server, str) or not server.startswith(("http://", "https://")):
        return "server must be an http(s) URL such as http://127.0.0.1:8000"
    if not model:
        return "model must not be empty"
    return True


class OmniARSampling:
    """Sampling parameters of one autoregressive stage (thinker, talker)."""
    CATEGORY = "omni/params"
    RETURN_TYPES = ("SAMPLING_PARAMS",)
    FUNCTION = "get"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"max_tokens": ("INT", {"default": 512, "min": 1, "max": 32768}),
                             "temperature": ("FLOAT", {"default": 1.0, "min": 0.0, "max": 2.0, "step": 0.01}),
                             "top_p": ("FLOAT", {"default": 1.0, "min": 0.0, "max": 1.0, "step": 0.01}),
                             "top_k": ("INT", {"default": 0, "min": 0, "max": 1000}),
                             "repetition_penalty": ("FLOAT", {"default": 1.0, "min": 0.0, "max": 5.0, "step": 0.01}),
                             "seed": ("INT", {"default": -1, "min": -1, "max": 2 ** 31 - 1})}}

    def get(self, seed, top_k, **kw):
        if seed >= 0:
            kw["seed"] = seed
        if top_k > 0:
            kw["top_k"] = top_k
        return ({"type": "ar", **kw},)


class OmniDiffusionSampling:
    """Sampling parameters of a diffusion stage."""
    CATEGORY = "omni/params"
    RETURN_TYPES = ("SAMPLING_PARAMS",)
    FUNCTION = "get"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"n": ("INT", {"default": 1, "min": 1, "max": 8}),
                             "num_inference_steps": ("INT", {"default": 50, "min": 1, "max": 200}),
                             "guidance_scale": ("FLOAT", {"default": 0.0, "min": 0.0, "max": 20.0, "step": 0.1}),
                             "true_cfg_scale": ("FLOAT", {"default": 4.0, "min": 0.0, "max": 20.0, "step": 0.1}),
                             "seed": ("INT", {"default": -1, "min": -1, "max": 2 ** 31 - 1})}}

    def get(self, seed, n, **kw):
        if seed >= 0:
            kw["seed"] = seed
        return ({"type": "diffusion", "num_outputs_per_prompt": n, **kw},)


class OmniSamplingParamsList:
    """One parameter set per stage, in stage order (the server's ``sampling_params_list``)."""
    CATEGORY = "omni/params"
    RETURN_TYPES = ("SAMPLING_PARAMS",)
    FUNCTION = "get"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"stage0": ("SAMPLING_PARAMS",)},
                "optional": {"stage1": ("SAMPLING_PARAMS",), "stage2": ("SAMPLING_PARAMS",)}}

    def get(self, stage0, stage1=None, stage2=None):
        out = []
        for p in (stage0, stage1, stage2):
            if p is None:
                continue
            out += p["list"] if p.get("type") == "list" else [p]
        return ({"type": "list", "list": out},)


def _stage_params(p) -> list[dict]:
    if p is None:
        return []
    items = p["list"] if p.get("type") == "list" else [p]
    return [{k: v for k, v in it.items() if k != "type"} for it in items]


class OmniQwenTTSParams:
    CATEGORY = "omni/params"
    RETURN_TYPES = ("TTS_PARAMS",)
    FUNCTION = "get"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"task_type": (["CustomVoice", "VoiceDesign", "Base"], {"default": "CustomVoice"}),
                             "language": (["Auto", "Chinese", "English", "Japanese", "Korean"], {"default": "Auto"}),
                             "instructions": ("STRING", {"multiline": True, "default": ""}),
                             "max_new_tokens": ("INT", {"default": 2048, "min": 1, "max": 32768})}}

    def get(self, **kw):
        return ({"type": "qwen-tts", **kw},)


def _speech_body(model, text, voice, response_format, speed, tts):
    body = {"model": model, "input": text, "voice": voice, "response_format": response_format, "speed": speed}
    if tts:
        body.update({k: v for k, v in tts.items() if k != "type" and v not in ("", None)})
        if body.get("language") == "Auto":
            body.pop("language")
    return body


class OmniTTS(OmniSpeech):
    """Speech with the container, the speed and the Qwen-TTS options exposed."""

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Qwen/Qwen3-TTS-12Hz-1.7B-CustomVoice"}),
                             "text": ("STRING", {"multiline": True, "default": ""}),
                             "voice": ("STRING", {"default": "Vivian"}),
                             "response_format": (["wav", "flac", "pcm"],),
                             "speed": ("FLOAT", {"default": 1.0, "min": 0.25, "max": 4.0, "step": 0.01})},
                "optional": {"tts_params": ("TTS_PARAMS",)}}

    @classmethod
    def VALIDATE_INPUTS(cls, server, model, **_):
        return check_server(server, model)

    def run(self, server, model, text, voice, response_format="wav", speed=1.0, tts_params=None):
        body = _speech_body(model, text, voice, "wav", speed, tts_params)       # the node decodes WAV itself
        return (_wav_to_audio(_post(server.rstrip("/") + "/v1/audio/speech", json=body, timeout=600).content),)


class OmniVoiceClone(OmniSpeech):
    """Speech in the voice of a reference clip (x-vector only, or in-context with the clip's transcript)."""

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Qwen/Qwen3-TTS-12Hz-1.7B-Base"}),
                             "text": ("STRING", {"multiline": True, "default": ""}),
                             "ref_audio": ("AUDIO",),
                             "ref_text": ("STRING", {"multiline": True, "default": ""}),
                             "x_vector_only_mode": ("BOOLEAN", {"default": False}),
                             "speed": ("FLOAT", {"default": 1.0, "min": 0.25, "max": 4.0, "step": 0.01})},
                "optional": {"tts_params": ("TTS_PARAMS",)}}

    @classmethod
    def VALIDATE_INPUTS(cls, server, model, **_):
        return check_server(server, model)

    def run(self, server, model, text, ref_audio, ref_text, x_vector_only_mode, speed=1.0, tts_params=None):
        if not x_vector_only_mode and not ref_text.strip():
            raise ValueError("in-context cloning needs the reference clip's transcript (or set x_vector_only_mode)")
        body = _speech_body(model, text, None, "wav", speed, tts_params)
        body.pop("voice")
        body.update({"task_type": "Base", "ref_audio": "data:audio/wav;base64," + base64.b64encode(_audio_to_wav(ref_audio)).decode(),
                     "ref_text": ref_text, "x_vector_only_mode": bool(x_vector_only_mode)})
        return (_wav_to_audio(_post(server.rstrip("/") + "/v1/audio/speech", json=body, timeout=600).content),)


class OmniVideoGenerate:
    """``/v1/videos``: text (and optionally a first frame) to a clip, returned as an IMAGE batch of frames."""
    CATEGORY = "omni"
    RETURN_TYPES = ("IMAGE", "INT")
    RETURN_NAMES = ("frames", "fps")
    FUNCTION = "run"

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Wan-AI/Wan2.2-T2V-A14B-Diffusers"}),
                             "prompt": ("STRING", {"multiline": True, "default": ""}),
                             "width": ("INT", {"default": 832, "min": 64, "max": 2048, "step": 16}),
                             "height": ("INT", {"default": 480, "min": 64, "max": 2048, "step": 16}),
                             "num_frames": ("INT", {"default": 81, "min": 1, "max": 257}),
                             "fps": ("INT", {"default": 16, "min": 1, "max": 60}),
                             "steps": ("INT", {"default": 40, "min": 1, "max": 200}),
                             "guidance_scale": ("FLOAT", {"default": 4.0, "min": 0.0, "max": 20.0}),
                             "seed": ("INT", {"default": 0, "min": 0, "max": 2 ** 31 - 1})},
                "optional": {"negative_prompt": ("STRING", {"multiline": True, "default": ""}), "image": ("IMAGE",)}}

    @classmethod
    def VALIDATE_INPUTS(cls, server, model, **_):
        return check_server(server, model)

    def run(self, server, model, prompt, width, height, num_frames, fps, steps, guidance_scale, seed, negative_prompt="",
            image=None):
        body = {"model": model, "prompt": prompt, "size": f"{width}x{height}", "num_frames": num_frames, "fps": fps,
                "num_inference_steps": steps, "guidance_scale": guidance_scale, "seed": seed, "response_format": "frames_b64"}
        if negative_prompt:
            body["negative_prompt"] = negative_prompt
        if image is not None:
            body["image"] = base64.b64encode(_image_to_png(image)).decode()
        clip = _post(server.rstrip("/") + "/v1/videos", json=body, timeout=7200).json()["data"][0]
        return (_to_tensor(np.concatenate([_png_to_image(b) for b in clip["frames_b64"]], 0)), int(clip.get("fps") or fps))


class OmniComprehension(OmniChat):
    """Chat with any mix of image, audio and video inputs; text and / or speech out; per-stage sampling parameters."""

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"server": ("STRING", {"default": "http://127.0.0.1:8000"}),
                             "model": ("STRING", {"default": "Qwen/Qwen3-Omni-30B-A3B-Instruct"}),
                             "prompt": ("STRING", {"multiline": True, "default": ""}),
                             "output_text": ("BOOLEAN", {"default": True}),
                             "output_audio": ("BOOLEAN", {"default": True})},
                "optional": {"image": ("IMAGE",), "audio": ("AUDIO",), "video": ("IMAGE",),
                             "system_prompt": ("STRING", {"multiline": True, "default": ""}),
                             "sampling_params": ("SAMPLING_PARAMS",)}}

    @classmethod
    def VALIDATE_INPUTS(cls, server, model, output_text=True, output_audio=True, **_):
        if not (output_text or output_audio):
            return "choose text, audio or both as output"
        return check_server(server, model)

    def run(self, server, model, prompt, output_text=True, output_audio=True, image=None, audio=None, video=None,
            system_prompt="", sampling_params=None):
        content = []
        if image is not None:
            for i in range(len(image) if hasattr(image, "__len__") and getattr(image, "ndim", 4) == 4 else 1):
                b64 = base64.b64encode(_image_to_png(image[i:i + 1] if getattr(image, "ndim", 4) == 4 else image)).decode()
                content.append({"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}})
        if video is not None:          # a frame batch: sent as an animated GIF in a data URL
            content.append({"type": "video_url", "video_url": {"url": "data:image/gif;base64," + base64.b64encode(_frames_to_gif(video)).decode()}})
        if audio is not None:
            content.append({"type": "audio_url",
                            "audio_url": {"url": "data:audio/wav;base64," + base64.b64encode(_audio_to_wav(audio)).decode()}})
        content.append({"type": "text", "text": prompt})
        msgs = ([{"role": "system", "content": system_prompt}] if system_prompt.strip() else []) + [{"role": "user", "content": content}]
        body = {"model": model, "messages": msgs,
                "modalities": (["text"] if output_text else []) + (["audio"] if output_audio else [])}
        sp = _stage_params(sampling_params)
        if sp:
            body["sampling_params_list"] = sp
        out = _post(server.rstrip("/") + "/v1/chat/completions", json=body, timeout=1800).json()
        text, spoken = "", {"waveform": _to_tensor(np.zeros((1, 1, 0), np.float32)), "sample_rate": 24000}
        for ch in out.get("choices", []):
            msg = ch.get("message") or {}
            if msg.get("content"):
                text += msg["content"] if isinstance(msg["content"], str) else json.dumps(msg["content"])
            if (msg.get("audio") or {}).get("data"):
                spoken = _wav_to_audio(base64.b64decode(msg["audio"]["data"]))
        return (text, spoken)


NODE_CLASS_MAPPINGS = {"OmniImageGenerate": OmniImageGenerate, "OmniImageEdit": OmniImageEdit,
                       "OmniSpeech": OmniSpeech, "OmniChat": OmniChat, "OmniTTS": OmniTTS, "OmniVoiceClone": OmniVoiceClone,
                       "OmniVideoGenerate": OmniVideoGenerate, "OmniComprehension": OmniComprehension,
                       "OmniARSampling": OmniARSampling, "OmniDiffusionSampling": OmniDiffusionSampling,
                       "OmniSamplingParamsList": OmniSamplingParamsList, "OmniQwenTTSParams": OmniQwenTTSParams}
NODE_DISPLAY_NAME_MAPPINGS = {"OmniImageGenerate": "Omni: generate image", "OmniImageEdit": "Omni: edit image",
                              "OmniSpeech": "Omni: text to speech", "OmniChat": "Omni: chat (text / audio)",
                              "OmniTTS": "Omni: TTS (format, speed, options)", "OmniVoiceClone": "Omni: voice clone",
                              "OmniVideoGenerate": "Omni: generate video", "OmniComprehension": "Omni: multimodal chat",
                              "OmniARSampling": "Omni: AR sampling params", "OmniDiffusionSampling": "Omni: diffusion sampling params",
                              "OmniSamplingParamsList": "Omni: per-stage params list", "OmniQwenTTSParams": "Omni: Qwen-TTS params"}
