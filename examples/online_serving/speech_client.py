"""``/v1/audio/speech`` client (formats: wav, pcm, flac, mp3, aac, opus where the server has an encoder)."""
import argparse

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="Qwen/Qwen3-TTS")
    ap.add_argument("--text", default="Hello from the speech endpoint.")
    ap.add_argument("--voice", default="default")
    ap.add_argument("--format", default="wav")
    ap.add_argument("--out", default="speech.wav")
    a = ap.parse_args()
    print("voices:", requests.get(a.base_url + "/v1/audio/voices", timeout=30).json())
    r = requests.post(a.base_url + "/v1/audio/speech", timeout=600,
                      json={"model": a.model, "input": a.text, "voice": a.voice, "response_format": a.format})
    r.raise_for_status()
    with open(a.out, "wb") as f:
        f.write(r.content)
    print("wrote", a.out)


if __name__ == "__main__":
    main()
