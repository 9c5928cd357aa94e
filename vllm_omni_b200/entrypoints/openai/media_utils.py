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


# ---------------------------------------------------------------------------------------------- FLAC
_CRC8 = [0] * 256
_CRC16 = [0] * 256
for _i in range(256):
    _c8, _c16 = _i, _i << 8
    for _ in range(8):
        _c8 = ((_c8 << 1) ^ 0x07) & 0xFF if _c8 & 0x80 else (_c8 << 1) & 0xFF
        _c16 = ((_c16 << 1) ^ 0x8005) & 0xFFFF if _c16 & 0x8000 else (_c16 << 1) & 0xFFFF
    _CRC8[_i], _CRC16[_i] = _c8, _c16
_FLAC_RATES = {88200: 1, 176400: 2, 192000: 3, 8000: 4, 16000: 5, 22050: 6, 24000: 7, 32000: 8, 44100: 9, 48000: 10, 96000: 11}


def _bits(value: int, n: int) -> np.ndarray:
    return np.array([(value >> (n - 1 - i)) & 1 for i in range(n)], dtype=np.uint8)


def _utf8_number(v: int) -> list:
    """The variable-length frame number of a FLAC frame header (UTF-8's byte layout, up to 36 bits)."""
    if v < 0x80:
        return [v]
    for nbytes, lead_bits in ((2, 5), (3, 4), (4, 3), (5, 2), (6, 1), (7, 0)):
        if v < (1 << (lead_bits + 6 * (nbytes - 1))):
            tail = []
            for _ in range(nbytes - 1):
                tail.append(0x80 | (v & 0x3F))
                v >>= 6
            return [((0xFF << (8 - nbytes)) & 0xFF) | v] + tail[::-1]
    raise ValueError("frame number too large")


def _rice_bits(res: np.ndarray, k: int) -> np.ndarray:
    """Rice code of signed residuals with parameter k: zig-zag, quotient in unary (zeros then a one), k-bit remainder."""
    u = np.where(res >= 0, res << 1, ((-res) << 1) - 1).astype(np.int64)
    q = u >> k
    length = q + 1 + k
    start = np.concatenate([[0], np.cumsum(length)[:-1]])
    out = np.zeros(int(length.sum()), dtype=np.uint8)
    out[start + q] = 1
    for j in range(k):
        out[start + q + 1 + j] = (u >> (k - 1 - j)) & 1
    return out


def flac_bytes(audio, sample_rate: int = 24000, block: int = 4096) -> bytes:
    """float waveform in [-1, 1], [T] or [C, T] with C <= 2 -> a 16-bit FLAC stream: fixed block size,
    per channel the best of the fixed predictors of order 0..2 with one Rice partition (lossless for the
    16-bit samples; STREAMINFO carries their MD5)."""
    import hashlib
    a = audio.detach().float().cpu().numpy() if isinstance(audio, torch.Tensor) else np.asarray(audio, dtype=np.float32)
    a = a.reshape(1, -1) if a.ndim == 1 else a
    C, T = a.shape
    if C > 2:
        raise ValueError("FLAC output supports mono or stereo")
    pcm = (np.clip(a, -1.0, 1.0) * 32767.0).astype(np.int64)
    md5 = hashlib.md5(pcm.T.astype("<i2").tobytes()).digest()
    frames, sizes = [], []
    for fi, s in enumerate(range(0, max(T, 1), block)):
        x = pcm[:, s:s + block]
        n = x.shape[1]
        if n == 0:
            break
        hdr = [0xFF, 0xF8, (7 << 4) | _FLAC_RATES.get(sample_rate, 0), ((C - 1) << 4) | (4 << 1)]
        hdr += _utf8_number(fi)
        hdr += [((n - 1) >> 8) & 0xFF, (n - 1) & 0xFF]      # 16-bit block size - 1 (block-size code 0111)
        c8 = 0
        for b in hdr:
            c8 = _CRC8[c8 ^ b]
        hdr.append(c8)
        bits = [np.unpackbits(np.array(hdr, dtype=np.uint8))]
        for ch in range(C):
            v = x[ch]
            best = None
            for order in range(min(3, n)):
                r = v[order:] if order == 0 else (v[1:] - v[:-1] if order == 1 else v[2:] - 2 * v[1:-1] + v[:-2])
                mean = float(np.abs(r).mean()) if r.size else 0.0
                k = min(14, max(0, int(np.ceil(np.log2(mean + 1e-9))) if mean > 1 else 0))
                cost = int(((np.where(r >= 0, r << 1, ((-r) << 1) - 1) >> k) + 1 + k).sum()) if r.size else 0
                if best is None or cost < best[0]:
                    best = (cost, order, k, r)
            _, order, k, r = best
            sub = [_bits((0b001000 | order) << 1, 8)]
            sub += [_bits(int(w) & 0xFFFF, 16) for w in v[:order]]
            sub += [_bits(0, 2), _bits(0, 4), _bits(k, 4), _rice_bits(r, k)]
            bits += sub
        allbits = np.concatenate(bits)
        if allbits.size % 8:
            allbits = np.concatenate([allbits, np.zeros(8 - allbits.size % 8, dtype=np.uint8)])
        body = np.packbits(allbits).tobytes()
        c16 = 0
        for b in body:
            c16 = ((c16 << 8) & 0xFFFF) ^ _CRC16[(c16 >> 8) ^ b]
        frames.append(body + struct.pack(">H", c16))
        sizes.append(len(frames[-1]))
    info = _bits(block, 16).tolist() + _bits(block, 16).tolist() + _bits(min(sizes) if sizes else 0, 24).tolist() + \
        _bits(max(sizes) if sizes else 0, 24).tolist() + _bits(sample_rate, 20).tolist() + _bits(C - 1, 3).tolist() + \
        _bits(15, 5).tolist() + _bits(T, 36).tolist()
    streaminfo = np.packbits(np.array(info, dtype=np.uint8)).tobytes() + md5
    return b"fLaC" + bytes([0x80]) + struct.pack(">I", len(streaminfo))[1:] + streaminfo + b"".join(frames)


AUDIO_MEDIA_TYPES = {"wav": "audio/wav", "pcm": "audio/pcm", "flac": "audio/flac", "mp3": "audio/mpeg",
                     "aac": "audio/aac", "opus": "audio/ogg"}


def encode_audio(audio, sample_rate: int, fmt: str = "wav", speed: float = 1.0) -> tuple[bytes, str]:
    """wav, pcm and flac are encoded here; the lossy formats (mp3, aac, opus) need an encoder library
    that this image does not ship, so they are refused with a clear message."""
    if speed and abs(speed - 1.0) > 1e-6:
        a = audio if isinstance(audio, torch.Tensor) else torch.as_tensor(np.asarray(audio))
        n = max(1, int(round(a.numel() / speed)))
        audio = torch.nn.functional.interpolate(a.reshape(1, 1, -1).float(), size=n, mode="linear",
                                                align_corners=False).reshape(-1)
    if fmt == "wav":
        return wav_bytes(audio, sample_rate), AUDIO_MEDIA_TYPES["wav"]
    if fmt == "pcm":
        return pcm_bytes(audio), AUDIO_MEDIA_TYPES["pcm"]
    if fmt == "flac":
        return flac_bytes(audio, sample_rate), AUDIO_MEDIA_TYPES["flac"]
    raise ValueError(f"response_format {fmt!r} needs an audio encoder that is not installed; use wav, pcm or flac")


def frames_to_gif_bytes(frames: np.ndarray, fps: int = 16) -> bytes:
    """[T, H, W, 3] uint8 -> animated GIF (PIL only; mp4 needs imageio/ffmpeg, absent here)."""
    from PIL import Image
    imgs = [Image.fromarray(f) for f in frames]
    buf = io.BytesIO()
    imgs[0].save(buf, format="GIF", save_all=True, append_images=imgs[1:], duration=int(1000 / max(fps, 1)), loop=0)
    return buf.getvalue()
