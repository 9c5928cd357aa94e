"""A pipeline class of your own behind the engine: the workers build the default pipeline's config,
then ``re_init_pipeline`` swaps in the class named by ``custom_pipeline_args["pipeline_class"]``
(``diffusion_load_format="custom_pipeline"``), so schedulers, caches, parallel groups and the
request / output plumbing stay the engine's.

The class below reuses the Qwen-Image edit pipeline and blends the edited image with the input
(image-to-image strength), the way the reference's ``examples/offline_inference/custom_pipeline``
does.

    python examples/offline_inference/custom_pipeline.py --model Qwen/Qwen-Image-Edit --image in.png \
        --prompt "turn it into a watercolour" --blend 0.35"""
import argparse
import os
import sys

import torch

from vllm_omni_b200.diffusion.models.qwen_image.pipeline_edit import QwenImageEditPipeline
from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


class BlendedEditPipeline(QwenImageEditPipeline):
    """Edit, then mix ``blend`` of the input image back into the result."""

    def __init__(self, od_config, device=None, blend: float = 0.25, **kw):
        super().__init__(od_config, device=device, **kw)
        self.blend = float(blend)

    def forward(self, req):
        out = super().forward(req)
        src = ((req.prompts[0].get("multi_modal_data") or {}).get("image_tensor")
               if isinstance(req.prompts[0], dict) else None)
        img = getattr(out, "output", None)
        if self.blend > 0 and isinstance(src, torch.Tensor) and isinstance(img, torch.Tensor) and img.dim() == 4:
            s = torch.nn.functional.interpolate(src.to(img.device, img.dtype).reshape(-1, *src.shape[-3:]), size=img.shape[-2:],
                                                mode="bilinear", align_corners=False)
            out.output = (1 - self.blend) * img + self.blend * s[: img.shape[0]]
        return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="QwenImageEditPipeline")
    ap.add_argument("--image", required=True)
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--blend", type=float, default=0.25)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--out", default="custom.png")
    a = ap.parse_args()
    from PIL import Image
    # worker processes import the class by name: make this file importable as the module ``custom_pipeline``
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    os.environ["PYTHONPATH"] = here + os.pathsep + os.environ.get("PYTHONPATH", "")
    # (a registry name such as the default is accepted in place of a checkpoint folder: random weights)
    omni = Omni(a.model, dtype="bfloat16", diffusion_load_format="custom_pipeline",
                custom_pipeline_args={"pipeline_class": "custom_pipeline.BlendedEditPipeline", "blend": a.blend})
    sp = OmniDiffusionSamplingParams(num_inference_steps=a.steps, true_cfg_scale=4.0, seed=0)
    outs = omni.generate([{"prompt": a.prompt, "negative_prompt": " ",
                           "multi_modal_data": {"image": Image.open(a.image).convert("RGB")}}], sp)
    outs[0].images[0].save(a.out)
    print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
