"""Chat-request inputs for the omni thinker: resize rule, pixel / frame / log-mel tensors, placeholders in the
message text, and the pieces end to end through the tiny thinker's ``preprocess_request``."""
import base64
import io

import numpy as np
import pytest
import torch
from PIL import Image

from vllm_omni_b200.inputs import omni_processor as op


def test_smart_resize_rounds_bounds_and_keeps_ratio():
    assert op.smart_resize(480, 640, 32) == (480, 640)
    assert op.smart_resize(481, 655, 32) == (480, 640)
    h, w = op.smart_resize(4000, 6000, 32, max_pixels=1280 * 28 * 28)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 1280 * 28 * 28 and abs(h / w - 4000 / 6000) < 0.03
    h, w = op.smart_resize(10, 20, 32, min_pixels=56 * 56)
    assert h % 32 == 0 and w % 32 == 0 and h * w >= 56 * 56
    with pytest.raises(ValueError):
        op.smart_resize(2, 1000, 32)


def test_image_video_audio_tensors():
    im = Image.fromarray((np.random.RandomState(0).rand(70, 100, 3) * 255).astype(np.uint8))
    px = op.image_to_pixels(im, 32)
    assert px.shape == (1, 3, 64, 96) and -1.0 <= float(px.min()) and float(px.max()) <= 1.0
    same = op.image_to_pixels(Image.fromarray(np.full((64, 96, 3), 255, np.uint8)), 32)
    assert torch.allclose(same, torch.ones_like(same))
    vid = op.video_to_pixels([im] * 40, 32, max_frames=8)
    assert vid.shape == (8, 3, 64, 96)
    # 0.5 s of a 440 Hz tone at 24 kHz -> 16 kHz -> 50 frames of 128 bins
    t = torch.arange(12000) / 24000
    mel = op.audio_to_mel(torch.sin(2 * torch.pi * 440 * t), 24000)
    assert mel.shape == (128, 50) and torch.isfinite(mel).all()
    low, high = mel[:20].mean(), mel[100:].mean()
    assert low > high                                      # the energy sits in the low bins


def _wav_b64(x: np.ndarray, rate: int, width: int = 2) -> str:
    import wave
    buf = io.BytesIO()
    with wave.open(buf, "wb") as f:
        f.setnchannels(1)
        f.setsampwidth(width)
        f.setframerate(rate)
        f.writeframes((x * 32767).astype("<i2").tobytes())
    return base64.b64encode(buf.getvalue()).decode()


def test_wav_decode_and_refusal_of_other_containers():
    x = np.sin(np.arange(800) / 10).astype(np.float32) * 0.5
    w, r = op.decode_audio_bytes(base64.b64decode(_wav_b64(x, 16000)))
    assert r == 16000 and w.shape == (800,) and float((w - torch.from_numpy(x)).abs().max()) < 1e-4
    with pytest.raises(ValueError, match="WAV"):
        op.decode_audio_bytes(b"ID3\x04" + b"\0" * 64)


def test_chat_content_becomes_text_with_placeholders_and_raw_items():
    from vllm_omni_b200.entrypoints.openai.api_server import _flatten_content
    png = io.BytesIO()
    Image.new("RGB", (40, 24), (10, 200, 30)).save(png, format="PNG")
    gif = io.BytesIO()
    fr = [Image.new("RGB", (32, 32), (i * 40, 0, 0)) for i in range(3)]
    fr[0].save(gif, format="GIF", save_all=True, append_images=fr[1:], duration=100)
    x = np.zeros(1600, np.float32)
    content = [{"type": "text", "text": "look: "},
               {"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(png.getvalue()).decode()}},
               {"type": "text", "text": " listen: "},
               {"type": "input_audio", "input_audio": {"data": _wav_b64(x, 16000), "format": "wav"}},
               {"type": "audio_url", "audio_url": {"url": "data:audio/wav;base64," + _wav_b64(x, 8000)}},
               {"type": "video_url", "video_url": {"url": "data:image/gif;base64," + base64.b64encode(gif.getvalue()).decode()}},
               {"type": "text", "text": " what happens?"}]
    text, mm = _flatten_content(content, placeholders=True)
    assert text == ("look: " + op.PLACEHOLDER["image"] + " listen: " + op.PLACEHOLDER["audio"] * 2 + op.PLACEHOLDER["video"]
                    + " what happens?")
    assert len(mm["image"]) == 1 and len(mm["audio"]) == 2 and mm["audio"][1][1] == 8000 and len(mm["video"][0]) == 3
    plain, mm2 = _flatten_content(content)
    assert plain == "look:  listen:  what happens?" and mm2["image"][0].size == (40, 24)      # diffusion chat: no placeholders
    feats = op.thinker_inputs(mm, 32)
    assert feats["image"][0].shape == (1, 3, 64, 96) and feats["video"][0].shape == (3, 3, 32, 32)   # the small image is scaled up to the minimum area
    assert feats["audio"][0].shape == (128, 10) and feats["audio"][1].shape == (128, 20)
    with pytest.raises(ValueError, match="inline"):
        _flatten_content([{"type": "audio_url", "audio_url": {"url": "https://example.com/a.wav"}}])


def test_processed_items_feed_the_tiny_thinker():
    """One placeholder per item in the token ids is expanded to the item's feature length."""
    from vllm_omni_b200.engine.request import Request
    from vllm_omni_b200.inputs import SamplingParams
    from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
    from vllm_omni_b200.models.qwen3_omni.thinker import Qwen3OmniMoeThinker as Qwen3OmniThinker
    cfg = Qwen3OmniConfig.tiny()
    torch.manual_seed(0)
    th = Qwen3OmniThinker(cfg, torch.float32, "cpu")
    factor = cfg.vision.patch_size * cfg.vision.spatial_merge_size
    im = Image.fromarray((np.random.RandomState(1).rand(2 * factor, 3 * factor, 3) * 255).astype(np.uint8))
    t = torch.arange(8000) / 16000
    feats = op.thinker_inputs({"image": [im], "audio": [(torch.sin(2 * torch.pi * 300 * t), 16000)]}, factor, cfg.audio.num_mel_bins)
    ids = [5, cfg.image_token_id, 6, cfg.audio_token_id, 7]
    req = Request("r", ids, SamplingParams(max_tokens=1), multi_modal_data=feats)
    th.preprocess_request(req)
    H, W = feats["image"][0].shape[-2:]                        # the small image was scaled up to the minimum area
    n_img = (H // factor) * (W // factor)                      # merged grid cells
    assert req.prompt_token_ids.count(cfg.image_token_id) == n_img
    assert req.prompt_token_ids.count(cfg.audio_token_id) >= 1
    assert len(req.prompt_token_ids) == 3 + n_img + req.prompt_token_ids.count(cfg.audio_token_id)


def test_processor_settings_come_from_the_checkpoint_config(tmp_path):
    import json
    (tmp_path / "config.json").write_text(json.dumps({"thinker_config": {
        "vision_config": {"patch_size": 14, "spatial_merge_size": 2}, "audio_config": {"num_mel_bins": 80}}}))
    assert op.processor_kwargs_for(str(tmp_path)) == {"vision_factor": 28, "n_mels": 80}
    assert op.processor_kwargs_for(None) == {"vision_factor": 32, "n_mels": 128}
    tiny_stage = type("S", (), {"engine_args": {"model_stage": "thinker", "model_overrides": {"tiny": True}}})()
    assert op.processor_kwargs_for(None, [tiny_stage]) == {"vision_factor": 8, "n_mels": 16}
