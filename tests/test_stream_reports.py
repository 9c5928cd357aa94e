"""Progress reports of the AR engine: ``stream_interval`` (which steps report at all) and ``stream_mm_interval`` (which
reports carry the model's streamed tensors); nothing is lost in between, everything rides on a later report."""
import torch

from vllm_omni_b200.engine.llm_engine import LLMEngine
from vllm_omni_b200.inputs import SamplingParams
from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
from vllm_omni_b200.models.qwen3_omni.thinker import Qwen3OmniMoeThinker


def _engine():
    torch.manual_seed(0)
    cfg = Qwen3OmniConfig.tiny()
    th = Qwen3OmniMoeThinker(cfg, torch.float32, "cpu")
    return LLMEngine(th, None, "cpu", torch.float32, num_gpu_blocks=64, max_num_seqs=4), th


def _drain(eng):
    outs = []
    for _ in range(200):
        outs += eng.step()
        if not eng.has_unfinished_requests():
            break
    return outs


def test_stream_interval_selects_the_reporting_steps():
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True, detokenize=False)
    for every, want in ((1, list(range(1, 11))), (3, [3, 6, 9, 10]), (0, [10])):
        eng, _ = _engine()
        eng.stream_interval = every
        eng.add_request("r", {"prompt_token_ids": [5, 6, 7, 8]}, sp)
        outs = _drain(eng)
        assert [len(o.outputs[0].token_ids) for o in outs] == want, every
        assert outs[-1].finished and all(not o.finished for o in outs[:-1])


def test_streamed_tensors_ride_on_every_nth_report_and_add_up():
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True, detokenize=False)
    eng, th = _engine()
    th.stream_output_keys = th.chunk_stream_keys
    eng.stream_mm_interval = 4
    eng.add_request("r", {"prompt_token_ids": [5, 6, 7, 8]}, sp)
    outs = _drain(eng)
    rows, seen_tts = 0, 0
    for o in outs[:-1]:
        mm = o.outputs[0].multimodal_output or {}
        n = len(o.outputs[0].token_ids)
        if n % 4 == 0:
            assert "0" in mm and mm["0"].shape[0] > 0
            rows += mm["0"].shape[0]
            seen_tts += int("tts_bos_embed" in mm)
            assert rows == 4 + n - 1              # prompt rows + every fed reply token so far
        else:
            assert "0" not in mm
    final = outs[-1].outputs[0].multimodal_output
    assert outs[-1].finished and final["0"].shape[0] == 4 + 9 and seen_tts == 1      # the markers are sent once
