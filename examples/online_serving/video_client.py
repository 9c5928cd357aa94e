"""``POST /v1/videos``: text-to-video, or image-to-video when ``--image`` is given (Wan 2.2 pipelines).

    ./run_server.sh Wan-AI/Wan2.2-T2V-A14B-Diffusers --ulysses-degree 4 --ring-degree 2
    python examples/online_serving/video_client.py --prompt "a paper boat on a stream" --frames 81 --out boat.gif
    python examples/online_serving/video_client.py --image first.png --prompt "it starts to rain" --frames-dir clip"""
import argparse
import base64
import os

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default=None)
    ap.add_argument("--prompt", default="a paper boat drifting down a stream")
    ap.add_argument("--negative-prompt", default=None)
    ap.add_argument("--image", default=None, help="conditioning image (image-to-video)")
    ap.add_argument("--size", default="832x480")
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--fps", type=int, default=16)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--guidance", type=float, default=4.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--frames-dir", default=None, help="ask for PNG frames and write them here instead of one GIF")
    ap.add_argument("--out", default="video.gif")
    a = ap.parse_args()
    body = {"prompt": a.prompt, "size": a.size, "num_frames": a.frames, "fps": a.fps, "num_inference_steps": a.steps,
            "guidance_scale": a.guidance, "seed": a.seed, "response_format": "frames_b64" if a.frames_dir else "b64_json"}
    if a.model:
        body["model"] = a.model
    if a.negative_prompt is not None:
        body["negative_prompt"] = a.negative_prompt
    if a.image:
        with open(a.image, "rb") as f:
            body["image"] = base64.b64encode(f.read()).decode()
    r = requests.post(a.base_url + "/v1/videos", json=body, timeout=7200)
    r.raise_for_status()
    clip = r.json()["data"][0]
    if a.frames_dir:
        os.makedirs(a.frames_dir, exist_ok=True)
        for i, b in enumerate(clip["frames_b64"]):
            with open(os.path.join(a.frames_dir, f"{i:04d}.png"), "wb") as f:
                f.write(base64.b64decode(b))
        print(f"wrote {len(clip['frames_b64'])} frames to {a.frames_dir}/ ({clip['fps']} fps)")
    else:
        with open(a.out, "wb") as f:
            f.write(base64.b64decode(clip["b64_json"]))
        print("wrote", a.out)


if __name__ == "__main__":
    main()
