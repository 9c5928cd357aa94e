"""Image to video (Wan 2.2 I2V / TI2V): the first frame is given, the clip continues it.

    python examples/offline_inference/image_to_video.py --model Wan-AI/Wan2.2-I2V-A14B-Diffusers \
        --image first.png --prompt "the boat drifts away" --frames 81 --out clip

``--ti2v`` selects the 5B text+image pipeline (``Wan22TI2VPipeline``), which also runs without an image."""
import argparse
import os

from PIL import Image

from vllm_omni_b200.diffusion.data import DiffusionParallelConfig
from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--ti2v", action="store_true")
    ap.add_argument("--image", default=None)
    ap.add_argument("--prompt", default="the camera slowly pulls back")
    ap.add_argument("--negative-prompt", default="")
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--guidance", type=float, default=3.5)
    ap.add_argument("--fps", type=int, default=16)
    ap.add_argument("--ulysses", type=int, default=1)
    ap.add_argument("--ring", type=int, default=1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--out", default="video_frames")
    a = ap.parse_args()
    model = a.model or ("Wan22TI2VPipeline" if a.ti2v else "WanImageToVideoPipeline")
    kw = {"diffusion_load_format": "dummy"} if a.dummy else {}
    omni = Omni(model, dtype="bfloat16",
                parallel_config=DiffusionParallelConfig(ulysses_degree=a.ulysses, ring_degree=a.ring), **kw)
    prompt = {"prompt": a.prompt, "negative_prompt": a.negative_prompt}
    if a.image:
        prompt["multi_modal_data"] = {"image": Image.open(a.image).convert("RGB")}
    elif not a.ti2v:
        prompt["multi_modal_data"] = {"image": Image.new("RGB", (a.width, a.height), (96, 128, 160))}
    sp = OmniDiffusionSamplingParams(height=a.height, width=a.width, num_frames=a.frames, num_inference_steps=a.steps,
                                     guidance_scale=a.guidance, fps=a.fps, seed=a.seed)
    outs = omni.generate([prompt], sp)
    os.makedirs(a.out, exist_ok=True)
    frames = outs[0].images
    for i, f in enumerate(frames):
        f.save(os.path.join(a.out, f"{i:04d}.png"))
    print(f"wrote {len(frames)} frames to {a.out}/")
    omni.close()


if __name__ == "__main__":
    main()
