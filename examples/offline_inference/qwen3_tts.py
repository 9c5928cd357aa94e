"""Qwen3-TTS: one generation stage, text in, waveform out.  Three request kinds, chosen by the
checkpoint (CustomVoice / VoiceDesign / Base) or by ``--task``:

    # a named voice of the checkpoint, optionally steered by an instruction
    python examples/offline_inference/qwen3_tts.py --model Qwen/Qwen3-TTS-12Hz-1.7B-CustomVoice \
        --text "Hello there." --speaker Vivian --language English --out hello.wav
    # a voice described in words
    python examples/offline_inference/qwen3_tts.py --model Qwen/Qwen3-TTS-12Hz-1.7B-VoiceDesign \
        --task VoiceDesign --instruct "A calm, low male voice." --text "Hello there."
    # a voice cloned from a reference clip (x-vector only; add --ref-text for in-context cloning when
    # the clip's codec frames are supplied by the caller)
    python examples/offline_inference/qwen3_tts.py --model Qwen/Qwen3-TTS-12Hz-1.7B-Base \
        --task Base --ref-audio ref.wav --x-vector-only --text "Hello there."
"""
import argparse

from qwen3_omni import save_wav

from vllm_omni_b200.entrypoints.omni import Omni


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen/Qwen3-TTS-12Hz-1.7B-CustomVoice")
    ap.add_argument("--stage-configs-path", default=None)
    ap.add_argument("--task", default=None, choices=["CustomVoice", "VoiceDesign", "Base"])
    ap.add_argument("--text", default="Hello there.")
    ap.add_argument("--speaker", default=None)
    ap.add_argument("--language", default="auto")
    ap.add_argument("--instruct", default=None)
    ap.add_argument("--ref-audio", default=None, help="WAV file of the voice to clone (task Base)")
    ap.add_argument("--ref-text", default=None)
    ap.add_argument("--x-vector-only", action="store_true")
    ap.add_argument("--out", default="speech.wav")
    a = ap.parse_args()
    omni = Omni(a.model, stage_configs_path=a.stage_configs_path)
    info = {"task_type": a.task, "speaker": a.speaker, "language": a.language, "instruct": a.instruct,
            "ref_audio": a.ref_audio, "ref_text": a.ref_text, "x_vector_only_mode": a.x_vector_only or None}
    prompt = {"prompt": a.text, "additional_information": {k: v for k, v in info.items() if v is not None}}
    outs = omni.generate([prompt], [s.default_sampling_params() for s in omni.stage_list])
    mm = outs[0].multimodal_output
    save_wav(a.out, mm["audio"], int(mm.get("sample_rate", 24000)))
    print("wrote", a.out)
    omni.close()


if __name__ == "__main__":
    main()
