"""Image / video serving benchmark against a running server
(benchmarks/diffusion/diffusion_benchmark_serving.py in the reference).

    python benchmarks/diffusion/diffusion_benchmark_serving.py --base-url http://127.0.0.1:8000 \
        --model Qwen/Qwen-Image --num-prompts 32 --max-concurrency 4 --size 1024x1024 --num-inference-steps 50
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from vllm_omni_b200.benchmarks.serve_bench import main  # noqa: E402

if __name__ == "__main__":
    argv = sys.argv[1:]
    what = "video" if "--video" in argv else "image"
    argv = [a for a in argv if a != "--video"]
    sys.exit(main([what] + argv))
