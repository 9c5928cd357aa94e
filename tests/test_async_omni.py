"""AsyncOmni: streaming, concurrent requests, abort, async-chunk audio streaming (CPU, tiny)."""
import asyncio
import textwrap

import pytest
import torch

from vllm_omni_b200.entrypoints.async_omni import AsyncOmni
from test_qwen3_omni_pipeline import YAML, _prompt


def _engine(tmp_path, async_chunk=False, talker_tokens=7):
    y = YAML.replace("async_chunk: false", f"async_chunk: {'true' if async_chunk else 'false'}")
    y = y.replace("max_tokens: 7", f"max_tokens: {talker_tokens}")
    # random weights may emit the stop code early; these tests want the whole utterance
    y = y.replace("stop_token_ids: [66]", "stop_token_ids: [], ignore_eos: true")
    p = tmp_path / "cfg.yaml"
    p.write_text(y)
    return AsyncOmni("qwen3-omni-tiny", stage_configs_path=str(p))


async def _collect(eng, prompt, rid):
    outs = []
    async for o in eng.generate(prompt, request_id=rid):
        outs.append(o)
    return outs


def test_concurrent_requests_stream_text_and_audio(tmp_path):
    eng = _engine(tmp_path)
    try:
        async def main():
            return await asyncio.gather(*[_collect(eng, _prompt(24 + 8 * i), f"r{i}") for i in range(3)])
        res = asyncio.run(main())
        for outs in res:
            texts = [o for o in outs if o.final_output_type == "text"]
            audio = [o for o in outs if o.final_output_type == "audio"]
            assert texts[-1].finished and len(texts[-1].outputs[0].token_ids) == 5
            assert len(texts) >= 2                      # streamed deltas before the final record
            assert len(audio) == 1 and audio[0].multimodal_output["audio"].numel() > 0
    finally:
        eng.close()


def test_abort_one_request_others_finish_and_id_reusable(tmp_path):
    eng = _engine(tmp_path)
    try:
        async def main():
            async def victim():
                n = 0
                async for _ in eng.generate(_prompt(), request_id="victim"):
                    n += 1
                    await eng.abort("victim")
                return n
            a, b, c = await asyncio.gather(victim(), _collect(eng, _prompt(), "ok1"), _collect(eng, _prompt(32), "ok2"))
            again = await _collect(eng, _prompt(), "victim")          # the aborted id can be reused
            return a, b, c, again
        a, b, c, again = asyncio.run(main())
        for outs in (b, c, again):
            assert any(o.final_output_type == "audio" for o in outs)
            assert [o for o in outs if o.final_output_type == "text"][-1].finished
    finally:
        eng.close()


def test_async_chunk_streams_audio_in_pieces(tmp_path):
    eng = _engine(tmp_path, async_chunk=True, talker_tokens=60)
    try:
        outs = asyncio.run(_collect(eng, _prompt(), "chunky"))
        audio = [o for o in outs if o.final_output_type == "audio"]
        text = [o for o in outs if o.final_output_type == "text"]
        assert text[-1].finished
        total = sum(a.multimodal_output["audio"].numel() for a in audio)
        # 60 talker steps (or fewer on the stop code) -> about frames x 16 samples (the decoder's
        # transposed convolutions drop a few samples at the end of every chunk), in >= 2 chunks of 25 frames
        assert len(audio) >= 2 and total >= 25 * 16 - 64
    finally:
        eng.close()


def test_async_chunk_talker_starts_from_the_running_thinker_and_matches_whole_request_hand_off(tmp_path):
    """Under ``async_chunk`` the talker is started once the thinker's prompt rows and first reply row exist and
    gets the later rows as updates; a decode step whose reply row has not arrived waits for it.  The codec
    frames and the text must equal the run in which the talker starts after the thinker has finished."""
    def run(async_chunk):
        y = YAML.replace("async_chunk: false", f"async_chunk: {'true' if async_chunk else 'false'}")
        y = y.replace("max_tokens: 7", "max_tokens: 40").replace("max_tokens: 5", "max_tokens: 30, ignore_eos: true")
        y = y.replace("stop_token_ids: [66]", "stop_token_ids: [], ignore_eos: true")
        p = tmp_path / f"cfg_{async_chunk}.yaml"
        p.write_text(y)
        eng = AsyncOmni("qwen3-omni-tiny", stage_configs_path=str(p))
        try:
            outs = asyncio.run(_collect(eng, _prompt(), "r"))
            text = [o for o in outs if o.final_output_type == "text"][-1].outputs[0].token_ids
            ro = eng.stage_list[1].engine_outputs[0]
            ro = getattr(ro, "request_output", None) or ro
            codes = ro.outputs[0].multimodal_output["codes"].clone()
            return list(text), codes, eng.stream_starts
        finally:
            eng.close()
    t0, c0, n0 = run(False)
    t1, c1, n1 = run(True)
    assert n0 == 0 and n1 == 1                      # the streamed start really happened
    assert t0 == t1 and len(t0) == 30
    assert c0.shape == c1.shape and c0.shape[0] == 40 and torch.equal(c0, c1)
