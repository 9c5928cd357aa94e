"""HTTP surface with FastAPI's TestClient: schema validation with a mocked engine, and the real
tiny engines (diffusion + three-stage omni) end to end."""
import base64
import io

import pytest
import torch
from fastapi.testclient import TestClient

from vllm_omni_b200.entrypoints.openai.api_server import build_app
from vllm_omni_b200.outputs import OmniRequestOutput


class FakeDiffusionEngine:
    """Records what the server asked for and returns a 1-pixel image per requested output."""
    stage_list = []

    def __init__(self):
        self.calls = []

    async def check_health(self):
        return None

    async def generate(self, prompt, request_id=None, sampling_params_list=None, output_modalities=None):
        from PIL import Image
        sp = sampling_params_list[0]
        self.calls.append((prompt, sp))
        imgs = [Image.new("RGB", (sp.width, sp.height), (i, 0, 0)) for i in range(sp.num_outputs_per_prompt)]
        yield OmniRequestOutput.from_diffusion(request_id, imgs, prompt)


@pytest.fixture()
def fake_client():
    eng = FakeDiffusionEngine()
    return TestClient(build_app(eng, "fake", kind="diffusion")), eng


def test_image_generation_request_mapping(fake_client):
    c, eng = fake_client
    r = c.post("/v1/images/generations", json={"prompt": "a cat", "n": 2, "size": "64x32", "seed": 7,
                                                "negative_prompt": "blurry", "num_inference_steps": 9,
                                                "true_cfg_scale": 3.5})
    assert r.status_code == 200, r.text
    body = r.json()
    assert len(body["data"]) == 2 and body["size"] == "64x32"
    from PIL import Image
    im = Image.open(io.BytesIO(base64.b64decode(body["data"][1]["b64_json"])))
    assert im.size == (64, 32)
    prompt, sp = eng.calls[0]
    assert prompt == {"prompt": "a cat", "negative_prompt": "blurry"}
    assert (sp.width, sp.height, sp.seed, sp.num_inference_steps, sp.true_cfg_scale) == (64, 32, 7, 9, 3.5)


@pytest.mark.parametrize("payload,code", [({"prompt": "x", "size": "abc"}, 400), ({"prompt": "x", "size": "100x100"}, 400),
                                          ({"prompt": "x", "n": 0}, 422), ({"size": "64x64"}, 422),
                                          ({"prompt": "x", "response_format": "url"}, 400),
                                          ({"prompt": "x", "lora": {"name": "a"}}, 400)])
def test_image_generation_validation(fake_client, payload, code):
    c, _ = fake_client
    assert c.post("/v1/images/generations", json=payload).status_code == code


def test_models_health_and_chat_as_image(fake_client):
    c, eng = fake_client
    assert c.get("/health").status_code == 200
    assert c.get("/v1/models").json()["data"][0]["id"] == "fake"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a red fox"}],
                                             "extra_body": {"size": "32x32", "num_inference_steps": 3}})
    assert r.status_code == 200, r.text
    url = r.json()["choices"][0]["message"]["content"][0]["image_url"]["url"]
    assert url.startswith("data:image/png;base64,")
    assert eng.calls[-1][1].num_inference_steps == 3


def test_image_edit_multipart(fake_client):
    c, eng = fake_client
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGB", (48, 32), (9, 9, 9)).save(buf, format="PNG")
    r = c.post("/v1/images/edits", files={"image": ("a.png", buf.getvalue(), "image/png")},
               data={"prompt": "make it blue", "n": "1"})
    assert r.status_code == 200, r.text
    prompt, sp = eng.calls[-1]
    assert prompt["multi_modal_data"]["image"].size == (48, 32) and (sp.width, sp.height) == (48, 32)


def test_real_tiny_diffusion_server():
    from vllm_omni_b200.entrypoints.async_omni import AsyncOmni
    eng = AsyncOmni("TinyMMDiTPipeline", dtype="float32", device="cpu")
    try:
        with TestClient(build_app(eng, "tiny", kind="diffusion")) as c:
            r = c.post("/v1/images/generations", json={"prompt": "a boat", "size": "64x64", "num_inference_steps": 2,
                                                        "seed": 1})
            assert r.status_code == 200, r.text
            assert len(base64.b64decode(r.json()["data"][0]["b64_json"])) > 100
            assert "omni_e2e_requests 1" in c.get("/metrics").text
    finally:
        eng.close()


def test_real_tiny_omni_chat_and_speech(tmp_path):
    from test_async_omni import _engine
    eng = _engine(tmp_path)
    try:
        with TestClient(build_app(eng, "tiny-omni", kind="omni")) as c:
            r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                     "modalities": ["text", "audio"], "max_tokens": 4})
            assert r.status_code == 200, r.text
            msg = r.json()["choices"][0]["message"]
            assert r.json()["usage"]["completion_tokens"] == 4
            assert base64.b64decode(msg["audio"]["data"])[:4] == b"RIFF"
            # streaming: SSE chunks with text deltas, then [DONE]
            with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                                 "stream": True, "max_tokens": 3}) as s:
                lines = [l for l in s.iter_lines() if l.startswith("data:")]
            assert lines[-1].strip() == "data: [DONE]" and len(lines) >= 2
            r = c.post("/v1/audio/speech", json={"input": "hello there", "voice": "Vivian", "max_new_tokens": 4})
            assert r.status_code == 200 and r.content[:4] == b"RIFF"
            assert c.post("/v1/audio/speech", json={"input": "x", "voice": "nobody"}).status_code == 400
            assert c.post("/v1/audio/speech", json={"input": "x", "response_format": "mp3"}).status_code == 400
            assert "Vivian" in c.get("/v1/audio/voices").json()["voices"]
    finally:
        eng.close()


def test_chat_with_audio_and_image_parts_reaches_the_engine_as_features():
    """Audio / image parts of a chat message arrive at the engine as log-mel features and pixel tensors, and the
    prompt text carries one placeholder group per item where the item stood."""
    import io
    import wave

    import numpy as np
    from PIL import Image

    from vllm_omni_b200.inputs.omni_processor import PLACEHOLDER

    class Capture:
        tokenizer = None
        mm_processor_kwargs = {"vision_factor": 16, "n_mels": 16}

        def __init__(self):
            self.prompts = []

        async def generate(self, prompt, request_id=None, sampling_params_list=None, output_modalities=None):
            self.prompts.append(prompt)
            return
            yield   # pragma: no cover  (an async generator that yields nothing)

    buf = io.BytesIO()
    with wave.open(buf, "wb") as f:
        f.setnchannels(1)
        f.setsampwidth(2)
        f.setframerate(16000)
        f.writeframes((np.sin(np.arange(3200) / 5) * 12000).astype("<i2").tobytes())
    png = io.BytesIO()
    Image.new("RGB", (96, 64), (9, 9, 200)).save(png, format="PNG")
    eng = Capture()
    with TestClient(build_app(eng, "cap", kind="omni")) as c:
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "audio_url", "audio_url": {"url": "data:audio/wav;base64," + base64.b64encode(buf.getvalue()).decode()}},
            {"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(png.getvalue()).decode()}},
            {"type": "text", "text": "what is this?"}]}]})
        assert r.status_code == 200, r.text
        p = eng.prompts[0]
        assert PLACEHOLDER["audio"] + PLACEHOLDER["image"] + "what is this?" in p["prompt"]
        mm = p["multi_modal_data"]
        assert tuple(mm["audio"][0].shape) == (16, 20) and tuple(mm["image"][0].shape) == (1, 3, 64, 96)
        bad = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "input_audio", "input_audio": {"data": base64.b64encode(b"ID3 not a wav").decode(), "format": "mp3"}}]}]})
        assert bad.status_code == 400 and "WAV" in bad.text


def test_real_tiny_omni_chat_with_an_audio_clip(tmp_path):
    """An audio part goes all the way: decoded, turned into log-mel features, its placeholder expanded by the
    thinker to the clip's feature length (the prompt grows by more than the text alone), reply text comes back."""
    import io
    import wave

    import numpy as np
    from test_async_omni import _engine
    buf = io.BytesIO()
    with wave.open(buf, "wb") as f:
        f.setnchannels(1)
        f.setsampwidth(2)
        f.setframerate(16000)
        f.writeframes((np.sin(np.arange(6400) / 7) * 9000).astype("<i2").tobytes())
    eng = _engine(tmp_path)
    try:
        assert eng.mm_processor_kwargs == {"vision_factor": 8, "n_mels": 16}
        with TestClient(build_app(eng, "tiny-omni", kind="omni")) as c:
            plain = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
            withclip = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
                {"type": "audio_url", "audio_url": {"url": "data:audio/wav;base64," + base64.b64encode(buf.getvalue()).decode()}},
                {"type": "text", "text": "hi"}]}], "max_tokens": 3})
            assert plain.status_code == 200 and withclip.status_code == 200, withclip.text
            extra = withclip.json()["usage"]["prompt_tokens"] - plain.json()["usage"]["prompt_tokens"]
            # 0.4 s of audio = 40 mel frames -> several encoder positions, plus the start / end marker strings
            assert extra > 28 + 1, extra      # 28 bytes of start / end marker text + the expanded placeholder
    finally:
        eng.close()


def test_video_route_maps_the_request_and_returns_gif_or_frames():
    """``/v1/videos``: fields reach the sampling parameters, a base64 first frame becomes the conditioning image,
    the clip comes back as one GIF or as PNG frames."""
    import numpy as np
    from PIL import Image

    class FakeVideoEngine:
        stage_list = []

        def __init__(self):
            self.calls = []

        async def generate(self, prompt, request_id=None, sampling_params_list=None, output_modalities=None):
            sp = sampling_params_list[0]
            self.calls.append((prompt, sp))
            frames = np.zeros((sp.num_frames, sp.height, sp.width, 3), np.uint8)
            frames[:, :, :, 1] = np.arange(sp.num_frames, dtype=np.uint8)[:, None, None] * 20
            yield OmniRequestOutput.from_diffusion(request_id, [], prompt, multimodal_output={"video": frames},
                                                   final_output_type="video")

    eng = FakeVideoEngine()
    with TestClient(build_app(eng, "fake-video", kind="diffusion")) as c:
        png = io.BytesIO()
        Image.new("RGB", (32, 16), (200, 10, 10)).save(png, format="PNG")
        r = c.post("/v1/videos", json={"prompt": "a boat", "size": "32x16", "num_frames": 5, "fps": 8, "seed": 4,
                                       "num_inference_steps": 3, "guidance_scale": 2.5, "negative_prompt": "blur",
                                       "image": base64.b64encode(png.getvalue()).decode(), "response_format": "frames_b64"})
        assert r.status_code == 200, r.text
        clip = r.json()["data"][0]
        assert len(clip["frames_b64"]) == 5 and clip["fps"] == 8 and clip["format"] == "png"
        assert Image.open(io.BytesIO(base64.b64decode(clip["frames_b64"][2]))).size == (32, 16)
        prompt, sp = eng.calls[0]
        assert prompt["prompt"] == "a boat" and prompt["negative_prompt"] == "blur"
        assert prompt["multi_modal_data"]["image"].size == (32, 16)
        assert (sp.width, sp.height, sp.num_frames, sp.fps, sp.seed, sp.num_inference_steps, sp.guidance_scale) == \
            (32, 16, 5, 8, 4, 3, 2.5)
        r = c.post("/v1/videos", json={"prompt": "a boat", "size": "32x16", "num_frames": 3})
        assert r.status_code == 200 and base64.b64decode(r.json()["data"][0]["b64_json"])[:3] == b"GIF"
        assert c.post("/v1/videos", json={"prompt": "x", "size": "wide"}).status_code == 400
        assert c.post("/v1/videos", json={"prompt": "x", "num_frames": 0}).status_code == 422
