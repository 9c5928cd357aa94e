"""``/v1/images/generations`` and ``/v1/images/edits`` clients."""
import argparse
import base64

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="Qwen/Qwen-Image")
    ap.add_argument("--prompt", default="a lighthouse at dawn")
    ap.add_argument("--size", default="1024x1024")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--edit-image", default=None, help="path of an image to edit instead of generating")
    ap.add_argument("--out", default="image.png")
    a = ap.parse_args()
    if a.edit_image:
        with open(a.edit_image, "rb") as f:
            r = requests.post(a.base_url + "/v1/images/edits", files={"image": f},
                              data={"model": a.model, "prompt": a.prompt, "num_inference_steps": a.steps}, timeout=1800)
    else:
        r = requests.post(a.base_url + "/v1/images/generations", timeout=1800,
                          json={"model": a.model, "prompt": a.prompt, "size": a.size, "num_inference_steps": a.steps,
                                "true_cfg_scale": 4.0, "seed": 0})
    r.raise_for_status()
    with open(a.out, "wb") as f:
        f.write(base64.b64decode(r.json()["data"][0]["b64_json"]))
    print("wrote", a.out)


if __name__ == "__main__":
    main()
