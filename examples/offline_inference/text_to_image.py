"""Text to image through the ``Omni`` API.

    python examples/offline_inference/text_to_image.py --model Qwen/Qwen-Image --prompt "a red fox" \
        --height 1024 --width 1024 --steps 50 --cfg 4.0 --out fox.png
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/offline_inference/text_to_image.py \
        --model Qwen/Qwen-Image --cfg-parallel 2 --ulysses 4 ...

``--dummy`` builds the architecture with random weights (no checkpoint needed)."""
import argparse

from vllm_omni_b200.diffusion.data import DiffusionParallelConfig
from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="QwenImagePipeline")
    ap.add_argument("--prompt", default="a lighthouse at dawn, oil painting")
    ap.add_argument("--negative-prompt", default=" ")
    ap.add_argument("--height", type=int, default=1024)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--cfg", type=float, default=4.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ulysses", type=int, default=1)
    ap.add_argument("--ring", type=int, default=1)
    ap.add_argument("--cfg-parallel", type=int, default=1)
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--cache-backend", default=None, choices=[None, "tea_cache", "cache_dit"])
    ap.add_argument("--quantization", default=None, choices=[None, "fp8"])
    ap.add_argument("--lora-path", default=None)
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--layers", type=int, default=None, help="with --dummy: number of transformer blocks")
    ap.add_argument("--out", default="out.png")
    a = ap.parse_args()
    kw = {}
    if a.dummy:
        kw["diffusion_load_format"] = "dummy"
        if a.layers:
            kw["tf_model_config"] = {"num_layers": a.layers}
    if a.cache_backend:
        kw["cache_backend"] = a.cache_backend
    if a.quantization:
        kw["quantization"] = a.quantization
    if a.lora_path:
        kw["lora_path"] = a.lora_path
    par = DiffusionParallelConfig(ulysses_degree=a.ulysses, ring_degree=a.ring, cfg_parallel_size=a.cfg_parallel,
                                  tensor_parallel_size=a.tensor_parallel)
    omni = Omni(a.model, dtype="bfloat16", parallel_config=par, **kw)
    sp = OmniDiffusionSamplingParams(height=a.height, width=a.width, num_inference_steps=a.steps, true_cfg_scale=a.cfg,
                                     seed=a.seed)
    outs = omni.generate([{"prompt": a.prompt, "negative_prompt": a.negative_prompt}], sp)
    if outs and outs[0].images:
        outs[0].images[0].save(a.out)
        print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
