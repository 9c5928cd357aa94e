"""BAGEL behind the OpenAI-compatible server: image generation and editing through the image endpoints,
understanding (image + question -> text) through chat completions.

    ./run_server.sh ByteDance-Seed/BAGEL-7B-MoT --stage-configs-path vllm_omni_b200/stage_configs/bagel.yaml
    python examples/online_serving/bagel_client.py generate --prompt "a ceramic owl"
    python examples/online_serving/bagel_client.py edit --image in.png --prompt "make it snow"
    python examples/online_serving/bagel_client.py ask --image in.png --prompt "What is on the shelf?\""""
import argparse
import base64

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("mode", choices=["generate", "edit", "ask"])
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="ByteDance-Seed/BAGEL-7B-MoT")
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--image", default=None)
    ap.add_argument("--size", default="1024x1024")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--out", default="bagel.png")
    a = ap.parse_args()
    if a.mode == "ask":
        content = [{"type": "text", "text": a.prompt}]
        if a.image:
            with open(a.image, "rb") as f:
                url = "data:image/png;base64," + base64.b64encode(f.read()).decode()
            content.insert(0, {"type": "image_url", "image_url": {"url": url}})
        r = requests.post(a.base_url + "/v1/chat/completions", timeout=600,
                          json={"model": a.model, "modalities": ["text"], "messages": [{"role": "user", "content": content}]})
        r.raise_for_status()
        print(r.json()["choices"][0]["message"]["content"])
        return
    if a.mode == "edit":
        if not a.image:
            ap.error("edit needs --image")
        with open(a.image, "rb") as f:
            r = requests.post(a.base_url + "/v1/images/edits", files={"image": f}, timeout=1800,
                              data={"model": a.model, "prompt": a.prompt, "num_inference_steps": a.steps})
    else:
        r = requests.post(a.base_url + "/v1/images/generations", timeout=1800,
                          json={"model": a.model, "prompt": a.prompt, "size": a.size, "num_inference_steps": a.steps, "seed": 0})
    r.raise_for_status()
    with open(a.out, "wb") as f:
        f.write(base64.b64decode(r.json()["data"][0]["b64_json"]))
    print("wrote", a.out)


if __name__ == "__main__":
    main()
