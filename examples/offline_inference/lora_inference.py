"""Per-request LoRA adapters on a diffusion pipeline: the same prompt with and without an adapter, and
two adapters with different scales in one session (each is loaded once and cached; switching swaps the
low-rank deltas on the fused linear layers).

    python examples/offline_inference/lora_inference.py --model Qwen/Qwen-Image \
        --lora pixel=/adapters/pixel-art --lora ink=/adapters/ink-wash:0.7 --prompt "a harbour town"

An adapter is a PEFT folder (``adapter_config.json`` + ``adapter_model.safetensors``)."""
import argparse

from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import LoRARequest, OmniDiffusionSamplingParams


def parse_adapter(spec: str, idx: int) -> LoRARequest:
    name, _, rest = spec.partition("=")
    path, _, scale = rest.partition(":")
    return LoRARequest(lora_name=name, lora_int_id=idx + 1, lora_path=path, scale=float(scale) if scale else 1.0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="QwenImagePipeline")
    ap.add_argument("--lora", action="append", default=[], metavar="NAME=PATH[:SCALE]")
    ap.add_argument("--prompt", default="a harbour town at dusk")
    ap.add_argument("--height", type=int, default=1024)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--cfg", type=float, default=4.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dummy", action="store_true")
    a = ap.parse_args()
    kw = {"diffusion_load_format": "dummy"} if a.dummy else {}
    omni = Omni(a.model, dtype="bfloat16", **kw)
    prompt = {"prompt": a.prompt, "negative_prompt": " "}

    def run(tag, req):
        sp = OmniDiffusionSamplingParams(height=a.height, width=a.width, num_inference_steps=a.steps, true_cfg_scale=a.cfg,
                                         seed=a.seed, lora_request=req, lora_scale=req.scale if req else 1.0)
        out = omni.generate([prompt], sp)[0]
        out.images[0].save(f"lora_{tag}.png")
        print("wrote", f"lora_{tag}.png")
    run("base", None)
    for i, spec in enumerate(a.lora):
        req = parse_adapter(spec, i)
        run(req.lora_name, req)
    omni.close()


if __name__ == "__main__":
    main()
