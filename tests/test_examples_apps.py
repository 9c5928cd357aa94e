"""User-facing scripts: the ComfyUI-style nodes against a fake server transport, the offline
throughput benchmark on the tiny pipeline, and that every example at least parses."""
import ast
import base64
import io
import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_examples_and_benchmarks_parse():
    files = list((ROOT / "examples").rglob("*.py")) + list((ROOT / "benchmarks").rglob("*.py")) + \
        list((ROOT / "apps").rglob("*.py"))
    assert len(files) >= 10
    for f in files:
        ast.parse(f.read_text(), filename=str(f))


def test_comfy_nodes_round_trip(monkeypatch):
    sys.path.insert(0, str(ROOT / "apps"))
    try:
        from comfyui_nodes import NODE_CLASS_MAPPINGS, nodes
    finally:
        sys.path.pop(0)
    from PIL import Image
    seen = {}

    class Resp:
        status_code = 200

        def __init__(self, payload=None, content=b""):
            self._p, self.content, self.text = payload, content, ""

        def json(self):
            return self._p

    def fake_post(url, **kw):
        seen[url.rsplit("/", 1)[-1]] = kw
        if url.endswith("videos"):
            buf = io.BytesIO()
            Image.new("RGB", (8, 4), (0, 255, 0)).save(buf, format="PNG")
            b = base64.b64encode(buf.getvalue()).decode()
            return Resp({"data": [{"frames_b64": [b, b, b], "fps": 12}]})
        if url.endswith("generations") or url.endswith("edits"):
            buf = io.BytesIO()
            Image.new("RGB", (8, 4), (255, 0, 0)).save(buf, format="PNG")
            n = (kw.get("json") or {}).get("n", 1)
            return Resp({"data": [{"b64_json": base64.b64encode(buf.getvalue()).decode()}] * n})
        import struct
        pcm = struct.pack("<4h", 0, 16384, -16384, 0)
        wav = b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, 24000, 48000, 2, 16) \
            + b"data" + struct.pack("<I", len(pcm)) + pcm
        if url.endswith("speech"):
            return Resp(content=wav)
        return Resp({"choices": [{"message": {"content": "hi", "audio": {"data": base64.b64encode(wav).decode()}}}]})

    monkeypatch.setattr(nodes, "_post", fake_post)
    img, = NODE_CLASS_MAPPINGS["OmniImageGenerate"]().run("http://s", "m", "p", 8, 4, 2, 4.0, 1, n=2)
    assert tuple(img.shape) == (2, 4, 8, 3) and float(img[0, 0, 0, 0]) == 1.0
    assert seen["generations"]["json"]["size"] == "8x4"
    out, = NODE_CLASS_MAPPINGS["OmniImageEdit"]().run("http://s", "m", img[:1], "p", 2, 0)
    assert tuple(out.shape) == (1, 4, 8, 3) and seen["edits"]["files"]["image"][2] == "image/png"
    audio, = NODE_CLASS_MAPPINGS["OmniSpeech"]().run("http://s", "m", "hello", "default")
    assert audio["sample_rate"] == 24000 and tuple(audio["waveform"].shape) == (1, 1, 4)
    assert abs(float(audio["waveform"][0, 0, 1]) - 0.5) < 1e-4
    text, audio = NODE_CLASS_MAPPINGS["OmniChat"]().run("http://s", "m", "hello", True, image=img[:1])
    assert text == "hi" and tuple(audio["waveform"].shape) == (1, 1, 4)
    assert seen["completions"]["json"]["messages"][0]["content"][1]["type"] == "image_url"
    frames, fps = NODE_CLASS_MAPPINGS["OmniVideoGenerate"]().run("http://s", "m", "p", 8, 4, 3, 12, 2, 4.0, 0, image=img[:1])
    assert tuple(frames.shape) == (3, 4, 8, 3) and fps == 12 and seen["videos"]["json"]["response_format"] == "frames_b64"
    assert "image" in seen["videos"]["json"]
    # parameter nodes feed the request bodies; cloning sends the clip inline; the chat node sends audio and video inline
    ar, = NODE_CLASS_MAPPINGS["OmniARSampling"]().get(seed=-1, top_k=0, max_tokens=64, temperature=0.7, top_p=0.9, repetition_penalty=1.0)
    dif, = NODE_CLASS_MAPPINGS["OmniDiffusionSampling"]().get(seed=3, n=2, num_inference_steps=20, guidance_scale=0.0, true_cfg_scale=4.0)
    lst, = NODE_CLASS_MAPPINGS["OmniSamplingParamsList"]().get(ar, dif)
    assert lst["list"][0]["max_tokens"] == 64 and "seed" not in lst["list"][0] and lst["list"][1]["seed"] == 3
    tts, = NODE_CLASS_MAPPINGS["OmniQwenTTSParams"]().get(task_type="VoiceDesign", language="Auto", instructions="calm", max_new_tokens=99)
    NODE_CLASS_MAPPINGS["OmniTTS"]().run("http://s", "m", "hello", "Vivian", tts_params=tts)
    body = seen["speech"]["json"]
    assert body["task_type"] == "VoiceDesign" and body["instructions"] == "calm" and "language" not in body and body["max_new_tokens"] == 99
    clip = {"waveform": audio["waveform"], "sample_rate": 24000}
    NODE_CLASS_MAPPINGS["OmniVoiceClone"]().run("http://s", "m", "hello", clip, "the transcript", False)
    body = seen["speech"]["json"]
    assert body["task_type"] == "Base" and body["ref_text"] == "the transcript" and "voice" not in body
    assert base64.b64decode(body["ref_audio"].split(",", 1)[1])[:4] == b"RIFF"
    with pytest.raises(ValueError):
        NODE_CLASS_MAPPINGS["OmniVoiceClone"]().run("http://s", "m", "hello", clip, "  ", False)
    text, _ = NODE_CLASS_MAPPINGS["OmniComprehension"]().run("http://s", "m", "what?", True, False, image=img[:1], audio=clip,
                                                             video=img, system_prompt="be brief", sampling_params=lst)
    body = seen["completions"]["json"]
    kinds = [p["type"] for p in body["messages"][1]["content"]]
    assert text == "hi" and kinds == ["image_url", "video_url", "audio_url", "text"] and body["modalities"] == ["text"]
    assert body["messages"][0]["role"] == "system" and len(body["sampling_params_list"]) == 2 and "type" not in body["sampling_params_list"][0]
    assert base64.b64decode(body["messages"][1]["content"][1]["video_url"]["url"].split(",", 1)[1])[:3] == b"GIF"
    assert NODE_CLASS_MAPPINGS["OmniComprehension"].VALIDATE_INPUTS("ftp://x", "m") is not True
    assert NODE_CLASS_MAPPINGS["OmniComprehension"].VALIDATE_INPUTS("http://x", "m", False, False) is not True
    assert NODE_CLASS_MAPPINGS["OmniTTS"].VALIDATE_INPUTS("http://x", "m") is True


def test_offline_throughput_benchmark_tiny():
    sys.path.insert(0, str(ROOT / "benchmarks" / "qwen3_omni"))
    try:
        import offline_throughput
    finally:
        sys.path.pop(0)
    rec = offline_throughput.main(["--tiny", "--num-prompts", "3", "--input-len", "6"])
    assert rec["requests"] == 3 and rec["text_tokens_per_s"] > 0 and rec["audio_seconds_per_s"] > 0


def test_ray_backend_reports_missing_dependency():
    from vllm_omni_b200.distributed import ray_utils
    assert ray_utils.stage_bundles([type("S", (), {"runtime": {"devices": "0,1"}})(),
                                    type("S", (), {"runtime": {}})()]) == [{"GPU": 2.0, "CPU": 1.0}, {"GPU": 1.0, "CPU": 1.0}]
    if not ray_utils.ray_available():
        with pytest.raises(RuntimeError, match="ray"):
            ray_utils.require_ray()


def test_serving_latency_benchmark_tiny():
    sys.path.insert(0, str(ROOT / "benchmarks" / "qwen3_omni"))
    try:
        import serving_latency
    finally:
        sys.path.pop(0)
    rec = serving_latency.main(["--tiny", "--num-prompts", "4", "--max-concurrency", "2", "--input-len", "8",
                                "--max-tokens", "5", "--codec-frames", "6", "--request-rate", "50"])
    assert rec["requests"] == 4 and rec["e2e_text_tokens_per_s"] > 0
    assert rec["ttft_s"]["p50"] is not None and rec["audio_ttfp_s"]["p50"] >= rec["ttft_s"]["p50"]


def test_ray_backend_with_a_fake_ray(monkeypatch, tmp_path):
    """The Ray worker backend end to end against a stand-in ``ray`` module whose actors are threads:
    placement group per stage, one actor per stage running the worker loop over "Ray" queues."""
    import queue
    import sys as _sys
    import threading
    import types

    ray = types.ModuleType("ray")
    state = {"actors": 0, "bundles": None, "killed": 0}
    ray.is_initialized = lambda: True
    ray.init = lambda **kw: None
    ray.get = lambda x: x
    ray.kill = lambda a: state.__setitem__("killed", state["killed"] + 1)

    def remote(cls):
        class Factory:
            @staticmethod
            def options(**kw):
                class Maker:
                    @staticmethod
                    def remote():
                        state["actors"] += 1
                        inst = cls()

                        class Handle:
                            class run:                                       # noqa: N801
                                @staticmethod
                                def remote(fn, a, kw):
                                    t = threading.Thread(target=fn, args=a, kwargs=kw, daemon=True)
                                    t.start()
                                    return t
                        Handle.inst = inst
                        return Handle
                return Maker
        return Factory
    ray.remote = remote
    util = types.ModuleType("ray.util")
    pgm = types.ModuleType("ray.util.placement_group")

    def placement_group(bundles, strategy="PACK"):
        state["bundles"] = bundles
        return types.SimpleNamespace(bundle_specs=bundles, ready=lambda: True)
    pgm.placement_group = placement_group
    qm = types.ModuleType("ray.util.queue")

    class Q(queue.Queue):
        def __init__(self, maxsize=0):
            super().__init__(maxsize)
    qm.Queue = Q
    sm = types.ModuleType("ray.util.scheduling_strategies")
    sm.PlacementGroupSchedulingStrategy = lambda **kw: kw
    for name, mod in (("ray", ray), ("ray.util", util), ("ray.util.placement_group", pgm), ("ray.util.queue", qm),
                      ("ray.util.scheduling_strategies", sm)):
        monkeypatch.setitem(_sys.modules, name, mod)

    from vllm_omni_b200.entrypoints.omni import Omni
    from vllm_omni_b200.inputs import SamplingParams
    y = tmp_path / "tts.yaml"
    y.write_text("""
stage_args:
  - stage_id: 0
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 2}
    engine_args: {model_stage: qwen3_tts, model_arch: Qwen3TTSForConditionalGeneration, worker_type: generation,
                  engine_output_type: audio, device: cpu, model_overrides: {tiny: true}}
    final_output: true
    final_output_type: audio
""")
    omni = Omni("qwen3-tts-tiny", stage_configs_path=str(y), worker_backend="ray")
    try:
        outs = omni.generate([{"prompt_token_ids": [5, 6, 7]}], [SamplingParams(temperature=0.0, max_tokens=4, seed=1)])
        assert outs and outs[0].final_output_type == "audio" and outs[0].multimodal_output["audio"].numel() > 0
        assert state["actors"] == 1 and state["bundles"] == [{"GPU": 1.0, "CPU": 1.0}]
    finally:
        omni.close()


def test_custom_pipeline_class_runs_behind_the_engine(tmp_path, monkeypatch):
    """``diffusion_load_format='custom_pipeline'``: the workers build the class named in
    ``custom_pipeline_args`` with the remaining keys as constructor arguments."""
    import sys

    import torch

    from vllm_omni_b200.entrypoints.omni import Omni
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    (tmp_path / "my_pipes.py").write_text(
        "from vllm_omni_b200.diffusion.models.tiny_mmdit.pipeline import TinyMMDiTPipeline\n"
        "class Doubled(TinyMMDiTPipeline):\n"
        "    def __init__(self, od_config, device=None, gain=1.0):\n"
        "        super().__init__(od_config, device=device)\n"
        "        self.gain = gain\n"
        "    def forward(self, req):\n"
        "        out = super().forward(req)\n"
        "        out.output = out.output * self.gain\n"
        "        return out\n")
    monkeypatch.syspath_prepend(str(tmp_path))
    monkeypatch.setenv("PYTHONPATH", str(tmp_path) + ":" + __import__("os").environ.get("PYTHONPATH", ""))
    sp = OmniDiffusionSamplingParams(height=32, width=32, num_inference_steps=2, seed=3, output_type="pt")

    def run(**kw):
        o = Omni("TinyMMDiTPipeline", dtype="float32", device="cpu", output_type="pt", **kw)
        try:
            return torch.as_tensor(o.generate(["x"], sp)[0].images[0]).float()
        finally:
            o.close()
    base = run(diffusion_load_format="dummy")
    got = run(diffusion_load_format="custom_pipeline", custom_pipeline_args={"pipeline_class": "my_pipes.Doubled", "gain": 0.0})
    assert base.abs().max() > 0 and got.shape == base.shape and got.abs().max() == 0      # the subclass's forward ran
    sys.modules.pop("my_pipes", None)
