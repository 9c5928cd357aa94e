"""Stage-to-stage input builders for Qwen2.5-Omni
(vllm_omni/model_executor/stage_input_processors/qwen2_5_omni.py).

``thinker2talker``: the thinker's per-token final hidden states, split into the prompt part and
the generated part, ride in ``additional_information`` (tensors stay on their device); the
talker prompt is codec BOS, one PAD per thinker prompt token, codec EOS.
``talker2code2wav``: the sampled codec tokens without the end marker.
"""
from __future__ import annotations

import torch

from ...inputs.data import OmniTokensPrompt
from .qwen3_omni import _outputs_of

TALKER_CODEC_PAD_TOKEN_ID = 8292
TALKER_CODEC_START_TOKEN_ID = 8293
TALKER_CODEC_END_TOKEN_ID = 8294


def thinker2talker(stage_list, engine_input_source, prompt=None, requires_multimodal_data=False):
    outs = []
    prompts = prompt if isinstance(prompt, list) else [prompt]
    for i, ro in enumerate(_outputs_of(stage_list, engine_input_source)):
        o = ro.outputs[0]
        latent = o.multimodal_output["latent"].detach()
        n_in = len(ro.prompt_token_ids)
        mmo = o.multimodal_output
        info = {
            "thinker_result": latent[n_in:],
            "prompt_embeds": latent[:n_in],
            **{k: mmo[k].detach() for k in ("tts_bos_embed", "tts_eos_embed", "tts_pad_embed") if k in mmo},
            "prompt_token_ids": list(ro.prompt_token_ids),
            "thinker_output_token_ids": list(o.token_ids),
        }
        mm = None
        if requires_multimodal_data and i < len(prompts) and isinstance(prompts[i], dict):
            mm = prompts[i].get("multi_modal_data")
        outs.append(OmniTokensPrompt(
            prompt_token_ids=[TALKER_CODEC_START_TOKEN_ID] + [TALKER_CODEC_PAD_TOKEN_ID] * n_in
            + [TALKER_CODEC_END_TOKEN_ID], additional_information=info, multi_modal_data=mm))
    return outs


def talker2code2wav(stage_list, engine_input_source, prompt=None, requires_multimodal_data=False):
    outs = []
    for ro in _outputs_of(stage_list, engine_input_source):
        o = ro.outputs[0]
        codes = o.multimodal_output.get("codes") if o.multimodal_output else None
        if codes is None:
            codes = torch.tensor(list(o.token_ids), dtype=torch.long)
        codes = codes.long().reshape(-1)
        if codes.numel() and o.finish_reason == "stop":
            codes = codes[:-1]                      # the end-of-speech token is not audio
        outs.append(OmniTokensPrompt(prompt_token_ids=[0] * max(1, codes.numel()),
                                     additional_information={"codes": codes}))
    return outs
