"""Streamed chat completion with text and audio deltas (``modalities: ["text", "audio"]``)."""
import argparse
import base64
import json

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="Qwen/Qwen3-Omni-30B-A3B-Instruct")
    ap.add_argument("--prompt", default="Say hello in one sentence.")
    ap.add_argument("--out", default="reply")
    a = ap.parse_args()
    body = {"model": a.model, "stream": True, "modalities": ["text", "audio"],
            "messages": [{"role": "user", "content": a.prompt}]}
    n_audio = 0
    with requests.post(a.base_url + "/v1/chat/completions", json=body, stream=True, timeout=600) as r:
        r.raise_for_status()
        for line in r.iter_lines():
            if not line or not line.startswith(b"data:"):
                continue
            data = line[5:].strip()
            if data == b"[DONE]":
                break
            for c in json.loads(data).get("choices", []):
                d = c.get("delta") or {}
                if d.get("content"):
                    print(d["content"], end="", flush=True)
                if d.get("audio", {}).get("data"):
                    with open(f"{a.out}_{n_audio:03d}.wav", "wb") as f:
                        f.write(base64.b64decode(d["audio"]["data"]))
                    n_audio += 1
    print(f"\n{n_audio} audio chunk(s) written")


if __name__ == "__main__":
    main()
