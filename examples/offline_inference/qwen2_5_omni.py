"""Qwen2.5-Omni end to end: thinker (text) -> talker (codec tokens) -> token2wav (flow-matching DiT +
BigVGAN), through the stage config shipped with the package.

    python examples/offline_inference/qwen2_5_omni.py --model Qwen/Qwen2.5-Omni-7B \
        --prompt "Describe the sound of rain." --voice Chelsie --out rain.wav
    python examples/offline_inference/qwen2_5_omni.py --text-only"""
import argparse
import os
import wave

import torch

import vllm_omni_b200
from vllm_omni_b200.entrypoints.omni import Omni


def save_wav(path, wav: torch.Tensor, rate: int):
    pcm = (wav.reshape(-1).clamp(-1, 1) * 32767).to(torch.int16).cpu().numpy().tobytes()
    with wave.open(path, "wb") as f:
        f.setnchannels(1)
        f.setsampwidth(2)
        f.setframerate(rate)
        f.writeframes(pcm)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen/Qwen2.5-Omni-7B")
    ap.add_argument("--stage-configs-path", default=os.path.join(os.path.dirname(vllm_omni_b200.__file__), "stage_configs",
                                                                 "qwen2_5_omni.yaml"))
    ap.add_argument("--prompt", default="Describe the sound of rain on a tin roof.")
    ap.add_argument("--voice", default=None, help="speaker name known to the checkpoint (e.g. Chelsie, Ethan)")
    ap.add_argument("--text-only", action="store_true", help="stop after the thinker: no speech")
    ap.add_argument("--out", default="reply.wav")
    a = ap.parse_args()
    omni = Omni(a.model, stage_configs_path=a.stage_configs_path)
    prompt = {"prompt": a.prompt}
    if a.voice:
        prompt["additional_information"] = {"voice": a.voice}
    if a.text_only:
        prompt["modalities"] = ["text"]
    outs = omni.generate([prompt], [s.default_sampling_params() for s in omni.stage_list])
    for o in outs:
        if o.final_output_type == "text":
            print(o.outputs[0].text)
        elif o.final_output_type == "audio":
            mm = o.multimodal_output
            save_wav(a.out, mm["audio"], int(mm.get("sample_rate", 24000)))
            print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
