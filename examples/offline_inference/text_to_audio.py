"""Stable Audio Open: text in, stereo 44.1 kHz clip out.

    python examples/offline_inference/text_to_audio.py --model stabilityai/stable-audio-open-1.0 \
        --prompt "The sound of a hammer hitting a wooden surface." --seconds 10 --out hammer.wav"""
import argparse
import struct

import numpy as np

from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def save_stereo_wav(path, audio, sample_rate):
    a = np.clip(np.asarray(audio, dtype=np.float32), -1.0, 1.0)
    a = a[None] if a.ndim == 1 else a                      # [channels, samples]
    pcm = (a.T * 32767.0).astype("<i2").tobytes()
    ch = a.shape[0]
    hdr = b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, ch, sample_rate,
                                                                                 sample_rate * 2 * ch, 2 * ch, 16)
    with open(path, "wb") as f:
        f.write(hdr + b"data" + struct.pack("<I", len(pcm)) + pcm)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="stabilityai/stable-audio-open-1.0")
    ap.add_argument("--prompt", default="The sound of a hammer hitting a wooden surface.")
    ap.add_argument("--negative-prompt", default="Low quality.")
    ap.add_argument("--seconds", type=float, default=10.0)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--guidance-scale", type=float, default=7.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="audio.wav")
    a = ap.parse_args()
    omni = Omni(a.model)
    sp = OmniDiffusionSamplingParams(num_inference_steps=a.steps, guidance_scale=a.guidance_scale, seed=a.seed,
                                     extra_args={"audio_start_in_s": 0.0, "audio_end_in_s": a.seconds})
    out = omni.generate([{"prompt": a.prompt, "negative_prompt": a.negative_prompt}], sp)[0]
    mm = out.multimodal_output
    save_stereo_wav(a.out, mm["audio"].float().cpu().numpy(), int(mm.get("sample_rate", 44100)))
    print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
