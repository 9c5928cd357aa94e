"""The talker fed by a thinker that is still generating: the request starts with the reply rows known so far, a
decode step whose row has not arrived is held back (``decode_blocked``), ``update_request`` delivers later rows and
the end of the reply; the codec frames equal those of a request that had the whole reply from the start."""
import torch

from vllm_omni_b200.engine.llm_engine import LLMEngine
from vllm_omni_b200.inputs import SamplingParams
from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
from vllm_omni_b200.models.qwen3_omni.talker import Qwen3OmniMoeTalker

PROMPT = [506, 509, 21, 500, 22, 507, 506, 510, 30]          # user turn with an audio placeholder, assistant header


def _info(emb, hid, e3, n_rows, stream):
    seq = PROMPT + list(range(40, 40 + 64))
    d = dict(thinker_embeddings=emb[:n_rows].clone(), thinker_hidden_states=hid[:n_rows].clone(),
             thinker_sequences=seq[:n_rows], thinker_input_ids=list(PROMPT), voice_type="Chelsie", **e3)
    if stream:
        d["thinker_stream"] = True
    return d


def _engine():
    torch.manual_seed(0)
    cfg = Qwen3OmniConfig.tiny()
    tk = Qwen3OmniMoeTalker(cfg, torch.float32, "cpu")
    return LLMEngine(tk, None, "cpu", torch.float32, num_gpu_blocks=64, max_num_seqs=4), cfg


def _run_to_end(eng, limit=400):
    frames = None
    for _ in range(limit):
        for ro in eng.step():
            if ro.finished:
                frames = ro.outputs[0].multimodal_output["codes"]
        if not eng.has_unfinished_requests():
            break
    return frames


def test_blocked_steps_wait_for_rows_and_frames_match_the_whole_reply():
    torch.manual_seed(1)
    n_reply = 9                                    # reply rows the thinker ends up producing (the last token has no row)
    L = len(PROMPT) + n_reply
    emb, hid = torch.randn(L, 64), torch.randn(L, 64)
    e3 = {k: torch.randn(1, 64) for k in ("tts_bos_embed", "tts_eos_embed", "tts_pad_embed")}
    sp = SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True, detokenize=False)

    eng, _ = _engine()
    eng.add_request("whole", {"prompt_token_ids": [0] * 11, "additional_information": _info(emb, hid, e3, L, False)}, sp)
    want = _run_to_end(eng)
    assert want.shape[0] == 14

    eng, _ = _engine()
    # the talker starts when only the first reply row exists
    req = eng.add_request("s", {"prompt_token_ids": [0] * 11,
                                "additional_information": _info(emb, hid, e3, len(PROMPT) + 1, True)}, sp)
    for _ in range(6):
        eng.step()
    assert req.decode_blocked and len(req.output_token_ids) == 1          # frame 0 done, frame 1 needs reply row 1
    assert not eng.scheduler.has_schedulable()
    # three more rows: steps 1..3 can run, then it waits again
    assert eng.update_request("s", {"thinker_embeddings": emb[len(PROMPT) + 1:len(PROMPT) + 4], "finished": False})
    assert not req.decode_blocked
    for _ in range(8):
        eng.step()
    assert req.decode_blocked and len(req.output_token_ids) == 4
    # an update without rows changes nothing; the rest of the reply and the end marker let it finish
    eng.update_request("s", {"thinker_embeddings": emb[:0], "finished": False})
    assert req.decode_blocked
    eng.update_request("s", {"thinker_embeddings": emb[len(PROMPT) + 4:], "finished": True})
    got = _run_to_end(eng)
    assert got.shape == want.shape and torch.equal(got, want)
    assert eng.update_request("s", {"finished": True}) is False           # finished requests ignore late updates
