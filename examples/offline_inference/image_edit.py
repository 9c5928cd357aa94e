"""Image editing (Qwen-Image-Edit style): an input image plus an instruction.

    python examples/offline_inference/image_edit.py --model Qwen/Qwen-Image-Edit --image in.png \
        --prompt "make the sky purple" --out edited.png"""
import argparse

from PIL import Image

from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="QwenImageEditPipeline")
    ap.add_argument("--image", required=True)
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--cfg", type=float, default=4.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--out", default="edited.png")
    a = ap.parse_args()
    kw = {"diffusion_load_format": "dummy"} if a.dummy else {}
    omni = Omni(a.model, dtype="bfloat16", **kw)
    img = Image.open(a.image).convert("RGB")
    sp = OmniDiffusionSamplingParams(num_inference_steps=a.steps, true_cfg_scale=a.cfg, seed=a.seed)
    outs = omni.generate([{"prompt": a.prompt, "negative_prompt": " ", "multi_modal_data": {"image": img}}], sp)
    outs[0].images[0].save(a.out)
    print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
