"""Offline throughput of the three-stage Qwen3-Omni pipeline (benchmarks/qwen3-omni in the
reference): N requests through ``Omni.generate``; reports requests/s, text tokens/s, seconds of
audio per second and the stage breakdown from the orchestrator's metrics.

    python benchmarks/qwen3_omni/offline_throughput.py --model Qwen/Qwen3-Omni-30B-A3B-Instruct --num-prompts 64
    python benchmarks/qwen3_omni/offline_throughput.py --tiny --num-prompts 8        # CPU smoke
"""
import argparse
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

TINY_YAML = """
stage_args:
  - stage_id: 0
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 8}
    engine_args: {model_stage: thinker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                  engine_output_type: latent, device: DEVICE, num_gpu_blocks: 256, model_overrides: {tiny: true}}
    final_output: true
    final_output_type: text
    default_sampling_params: {temperature: 0.0, max_tokens: 8}
  - stage_id: 1
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 8}
    engine_args: {model_stage: talker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                  engine_output_type: latent, device: DEVICE, num_gpu_blocks: 256, model_overrides: {tiny: true}}
    engine_input_source: [0]
    custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.thinker2talker
    default_sampling_params: {temperature: 0.0, max_tokens: 12, detokenize: false, stop_token_ids: [66]}
  - stage_id: 2
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 8}
    engine_args: {model_stage: code2wav, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: generation,
                  engine_output_type: audio, device: DEVICE, model_overrides: {tiny: true}}
    engine_input_source: [1]
    custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.talker2code2wav
    final_output: true
    final_output_type: audio
"""


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen/Qwen3-Omni-30B-A3B-Instruct")
    ap.add_argument("--stage-configs-path", default=None)
    ap.add_argument("--num-prompts", type=int, default=32)
    ap.add_argument("--input-len", type=int, default=32)
    ap.add_argument("--tiny", action="store_true", help="random tiny weights (smoke run, CPU or GPU)")
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    from vllm_omni_b200.entrypoints.omni import Omni
    path = a.stage_configs_path
    if a.tiny:
        f = tempfile.NamedTemporaryFile("w", suffix=".yaml", delete=False)
        f.write(TINY_YAML.replace("DEVICE", a.device))
        f.close()
        path = f.name
    omni = Omni(a.model, stage_configs_path=path)
    prompts = [{"prompt_token_ids": [(7 * i + j) % 400 + 10 for j in range(a.input_len)]} for i in range(a.num_prompts)]
    sps = [s.default_sampling_params() for s in omni.stage_list]
    t0 = time.perf_counter()
    outs = omni.generate(prompts, sps)
    wall = time.perf_counter() - t0
    toks = sum(len(o.outputs[0].token_ids) for o in outs if o.final_output_type == "text")
    audio_s = 0.0
    for o in outs:
        if o.final_output_type == "audio":
            mm = o.multimodal_output
            audio_s += mm["audio"].numel() / float(mm.get("sample_rate", 24000))
    rec = {"requests": a.num_prompts, "wall_s": round(wall, 4), "requests_per_s": round(a.num_prompts / wall, 3),
           "text_tokens_per_s": round(toks / wall, 2), "audio_seconds_per_s": round(audio_s / wall, 3),
           "summary": omni.metrics.build_summary().get("overall", {})}
    print(json.dumps(rec))
    omni.close()
    return rec


if __name__ == "__main__":
    main()
