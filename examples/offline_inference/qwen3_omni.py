"""Qwen3-Omni end to end: text (+ optional audio) in, text and speech out, through the three-stage
pipeline (thinker -> talker -> code2wav) described by a stage-config YAML.

    python examples/offline_inference/qwen3_omni.py --model Qwen/Qwen3-Omni-30B-A3B-Instruct \
        --prompt "Tell me a short story." --out story.wav
    python examples/offline_inference/qwen3_omni.py --stream      # AsyncOmni + async_chunk"""
import argparse
import asyncio
import wave

import torch

from vllm_omni_b200.entrypoints.async_omni import AsyncOmni
from vllm_omni_b200.entrypoints.omni import Omni


def save_wav(path, wav: torch.Tensor, rate: int):
    pcm = (wav.clamp(-1, 1) * 32767).to(torch.int16).cpu().numpy().tobytes()
    with wave.open(path, "wb") as f:
        f.setnchannels(1)
        f.setsampwidth(2)
        f.setframerate(rate)
        f.writeframes(pcm)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen/Qwen3-Omni-30B-A3B-Instruct")
    ap.add_argument("--stage-configs-path", default=None)
    ap.add_argument("--prompt", default="Tell me a short story about a lighthouse.")
    ap.add_argument("--stream", action="store_true")
    ap.add_argument("--out", default="reply.wav")
    a = ap.parse_args()
    if not a.stream:
        omni = Omni(a.model, stage_configs_path=a.stage_configs_path)
        outs = omni.generate([{"prompt": a.prompt}], [s.default_sampling_params() for s in omni.stage_list])
        for o in outs:
            if o.final_output_type == "text":
                print(o.outputs[0].text)
            elif o.final_output_type == "audio":
                mm = o.multimodal_output
                save_wav(a.out, mm["audio"], int(mm.get("sample_rate", 24000)))
                print("wrote", a.out)
        omni.close()
        return

    async def run():
        eng = AsyncOmni(a.model, stage_configs_path=a.stage_configs_path)
        parts, rate = [], 24000
        async for o in eng.generate({"prompt": a.prompt}):
            if o.final_output_type == "text" and o.outputs:
                print(o.outputs[0].text, end="\r", flush=True)
            elif o.final_output_type == "audio":
                parts.append(o.multimodal_output["audio"])
                rate = int(o.multimodal_output.get("sample_rate", rate))
        print()
        if parts:
            save_wav(a.out, torch.cat(parts), rate)
            print("wrote", a.out)
        eng.close()

    asyncio.run(run())


if __name__ == "__main__":
    main()
