"""Qwen3-TTS: one generation stage, text tokens in, waveform out.

    python examples/offline_inference/qwen3_tts.py --model Qwen/Qwen3-TTS --text "Hello there." --out hello.wav"""
import argparse

from qwen3_omni import save_wav

from vllm_omni_b200.entrypoints.omni import Omni


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen/Qwen3-TTS")
    ap.add_argument("--stage-configs-path", default=None)
    ap.add_argument("--text", default="Hello there.")
    ap.add_argument("--speaker", default="default")
    ap.add_argument("--language", default="auto")
    ap.add_argument("--out", default="speech.wav")
    a = ap.parse_args()
    omni = Omni(a.model, stage_configs_path=a.stage_configs_path)
    prompt = {"prompt": a.text, "additional_information": {"speaker": a.speaker, "language": a.language}}
    outs = omni.generate([prompt], [s.default_sampling_params() for s in omni.stage_list])
    mm = outs[0].multimodal_output
    save_wav(a.out, mm["audio"], int(mm.get("sample_rate", 24000)))
    print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
