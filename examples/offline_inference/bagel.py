"""BAGEL through one ``Omni`` object: text-to-image, image editing (a reference image conditions the
generation through its VAE latents and its vision-tower tokens) and the two-stage layout in which the
language-model stage hands its KV cache to the diffusion stage.

    python examples/offline_inference/bagel.py --model ByteDance-Seed/BAGEL-7B-MoT --prompt "a ceramic owl"
    python examples/offline_inference/bagel.py --model ... --image in.png --prompt "make it snow" \
        --cfg-text 4.0 --cfg-img 1.5
    python examples/offline_inference/bagel.py --model ... --stage-config vllm_omni_b200/stage_configs/bagel.yaml"""
import argparse

from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="BagelPipeline")
    ap.add_argument("--stage-config", default=None, help="YAML with the AR stage + DiT stage (KV hand-off)")
    ap.add_argument("--prompt", default="a ceramic owl on a bookshelf")
    ap.add_argument("--image", default=None, help="reference image: editing mode")
    ap.add_argument("--height", type=int, default=1024)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--cfg-text", type=float, default=4.0)
    ap.add_argument("--cfg-img", type=float, default=1.5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--out", default="bagel.png")
    a = ap.parse_args()
    kw = {"diffusion_load_format": "dummy"} if a.dummy else {}
    if a.stage_config:
        kw["stage_configs_path"] = a.stage_config
    omni = Omni(a.model, dtype="bfloat16", **kw)
    prompt = {"prompt": a.prompt}
    extra = {"cfg_text_scale": a.cfg_text}
    if a.image:
        from PIL import Image
        prompt["multi_modal_data"] = {"image": Image.open(a.image).convert("RGB")}
        extra["cfg_img_scale"] = a.cfg_img
    sp = OmniDiffusionSamplingParams(height=a.height, width=a.width, num_inference_steps=a.steps, seed=a.seed, extra_args=extra)
    out = omni.generate([prompt], sp)[0]
    out.images[0].save(a.out)
    print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
