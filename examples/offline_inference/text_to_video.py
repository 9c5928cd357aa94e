"""Text to video (Wan 2.2 style dual-transformer pipeline, UniPC flow scheduler).

    python examples/offline_inference/text_to_video.py --model Wan-AI/Wan2.2-T2V-A14B-Diffusers \
        --prompt "a paper boat on a stream" --frames 81 --height 480 --width 832 --out boat"""
import argparse
import os

from vllm_omni_b200.diffusion.data import DiffusionParallelConfig
from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="WanPipeline")
    ap.add_argument("--prompt", default="a paper boat drifting down a stream")
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--guidance", type=float, default=4.0)
    ap.add_argument("--ulysses", type=int, default=1)
    ap.add_argument("--ring", type=int, default=1)
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--out", default="video_frames")
    a = ap.parse_args()
    kw = {"diffusion_load_format": "dummy"} if a.dummy else {}
    omni = Omni(a.model, dtype="bfloat16",
                parallel_config=DiffusionParallelConfig(ulysses_degree=a.ulysses, ring_degree=a.ring), **kw)
    sp = OmniDiffusionSamplingParams(height=a.height, width=a.width, num_frames=a.frames, num_inference_steps=a.steps,
                                     guidance_scale=a.guidance, seed=0)
    outs = omni.generate([{"prompt": a.prompt, "negative_prompt": ""}], sp)
    os.makedirs(a.out, exist_ok=True)
    frames = outs[0].images
    for i, f in enumerate(frames):
        f.save(os.path.join(a.out, f"{i:04d}.png"))
    print(f"wrote {len(frames)} frames to {a.out}/")
    omni.close()


if __name__ == "__main__":
    main()
