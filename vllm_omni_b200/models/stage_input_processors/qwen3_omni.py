"""Stage-to-stage input builders for Qwen3-Omni
(vllm_omni/model_executor/stage_input_processors/qwen3_omni.py:86-313).

``thinker2talker``: packs the thinker's embeddings, layer-N hidden states, token ids and tts
special embeddings into the talker request's ``additional_information`` (tensors stay on
their device).  ``talker2code2wav``: turns the talker's codec frames into the code2wav
input.  The ``*_async_chunk`` variants emit the same payloads in pieces for streaming
(25 codec frames per chunk plus 25 frames of left context).
"""
from __future__ import annotations

import torch

from ...inputs.data import OmniTokensPrompt


def _outputs_of(stage_list, engine_input_source):
    if not engine_input_source:
        raise ValueError("engine_input_source is empty")
    src = stage_list[engine_input_source[0]].engine_outputs
    if not src:
        raise ValueError(f"stage {engine_input_source[0]} has no outputs yet")
    return [getattr(o, "request_output", None) or o for o in src]


def _hidden_key(mm: dict) -> str:
    for k in mm:
        if k.isdigit() and k != "0":
            return k
    raise KeyError("thinker output carries no captured hidden layer")


def thinker2talker(stage_list, engine_input_source, prompt=None, requires_multimodal_data=False):
    outs = []
    for ro in _outputs_of(stage_list, engine_input_source):
        o = ro.outputs[0]
        mm = o.multimodal_output
        info = {
            "thinker_embeddings": mm["0"].detach(),
            "thinker_hidden_states": mm[_hidden_key(mm)].detach(),
            "thinker_sequences": list(ro.prompt_token_ids) + list(o.token_ids),
            "thinker_input_ids": list(ro.prompt_token_ids),
            "tts_bos_embed": mm["tts_bos_embed"].detach(),
            "tts_eos_embed": mm["tts_eos_embed"].detach(),
            "tts_pad_embed": mm["tts_pad_embed"].detach(),
        }
        # the last generated token has no embedding row yet (it was never fed back)
        n_rows = info["thinker_embeddings"].shape[0]
        info["thinker_sequences"] = info["thinker_sequences"][:max(n_rows, len(info["thinker_input_ids"]))]
        outs.append(OmniTokensPrompt(prompt_token_ids=[0] * (len(info["thinker_input_ids"]) + 2),
                                     additional_information=info))
    return outs


def talker2code2wav(stage_list, engine_input_source, prompt=None, requires_multimodal_data=False):
    outs = []
    for ro in _outputs_of(stage_list, engine_input_source):
        codes = ro.outputs[0].multimodal_output.get("codes")
        if codes is None:
            codes = torch.zeros(0, 1, dtype=torch.long)
        codes = codes.long()
        # drop the frame that carries the end-of-speech code
        if codes.shape[0] and ro.outputs[0].finish_reason == "stop":
            codes = codes[:-1]
        outs.append(OmniTokensPrompt(prompt_token_ids=[0] * max(1, codes.shape[0]),
                                     additional_information={"codes": codes}))
    return outs


CHUNK_FRAMES = 25
LEFT_CONTEXT = 25


def talker2code2wav_async_chunk(codes_so_far: torch.Tensor, emitted_frames: int, finished: bool):
    """Next code2wav chunk for a growing frame list, or None when fewer than CHUNK_FRAMES new
    frames exist and the talker is still running.  Returns (payload, new_emitted_frames)."""
    total = codes_so_far.shape[0]
    avail = total - emitted_frames
    if avail <= 0 or (avail < CHUNK_FRAMES and not finished):
        return None, emitted_frames
    end = total if finished else emitted_frames + (avail // CHUNK_FRAMES) * CHUNK_FRAMES
    ctx = min(LEFT_CONTEXT, emitted_frames)
    payload = {"codes": codes_so_far[emitted_frames - ctx:end].long(), "left_context_frames": ctx,
               "last": bool(finished and end == total)}
    return payload, end


def thinker2talker_async_chunk(embeds: torch.Tensor, hidden: torch.Tensor, token_ids: list[int], emitted: int,
                               finished: bool, chunk_tokens: int = 16):
    """Streams the thinker's rows to the talker in chunks of ``chunk_tokens`` tokens."""
    total = embeds.shape[0]
    avail = total - emitted
    if avail <= 0 or (avail < chunk_tokens and not finished):
        return None, emitted
    end = total if finished else emitted + (avail // chunk_tokens) * chunk_tokens
    payload = {"thinker_embeddings": embeds[emitted:end], "thinker_hidden_states": hidden[emitted:end],
               "token_ids": token_ids[emitted:end], "last": bool(finished and end == total)}
    return payload, end
