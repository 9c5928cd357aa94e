"""Per-request LoRA on the image endpoint: the request names an adapter folder on the server's disk, the
server loads it on first use (cached afterwards) and applies it with the given scale for this request only.

    ./run_server.sh Qwen/Qwen-Image
    python examples/online_serving/lora_client.py --lora-name pixel --lora-path /adapters/pixel-art --scale 0.8"""
import argparse
import base64

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--prompt", default="a harbour town at dusk")
    ap.add_argument("--size", default="1024x1024")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--lora-name", required=True)
    ap.add_argument("--lora-path", required=True, help="PEFT adapter folder, as seen by the server")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--out", default="lora.png")
    a = ap.parse_args()
    for tag, lora in (("base", None), (a.lora_name, {"name": a.lora_name, "path": a.lora_path, "scale": a.scale})):
        body = {"prompt": a.prompt, "size": a.size, "num_inference_steps": a.steps, "true_cfg_scale": 4.0, "seed": 0}
        if lora:
            body["lora"] = lora
        r = requests.post(a.base_url + "/v1/images/generations", json=body, timeout=1800)
        r.raise_for_status()
        path = a.out.replace(".png", f"_{tag}.png")
        with open(path, "wb") as f:
            f.write(base64.b64decode(r.json()["data"][0]["b64_json"]))
        print("wrote", path)


if __name__ == "__main__":
    main()
