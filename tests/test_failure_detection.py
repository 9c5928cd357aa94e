"""Failure detection of the multi-process diffusion executor, with the failures made on the host:
a worker process that is killed, one that is frozen (SIGSTOP) and a call that overruns its
time limit.  The worker runs the tiny pipeline on the CPU; no GPU is involved."""
import os
import signal
import time

import pytest
import torch

from vllm_omni_b200.diffusion.data import OmniDiffusionConfig
from vllm_omni_b200.diffusion.executor import MultiprocDiffusionExecutor, WorkerDeadError


def _config():
    return OmniDiffusionConfig.from_kwargs(model="TinyMMDiTPipeline", model_class_name="TinyMMDiTPipeline",
                                           dtype=torch.float32, device="cpu", distributed_executor_backend="mp")


@pytest.fixture()
def executor():
    ex = MultiprocDiffusionExecutor(_config(), init_timeout=120, heartbeat_stall_s=1.5)
    yield ex
    for p in list(ex.procs):
        if p.is_alive():
            try:
                os.kill(p.pid, signal.SIGCONT)
            except OSError:
                pass
    ex.shutdown()


def test_rpc_roundtrip_then_killed_worker_is_reported(executor):
    assert executor.check_health()
    assert executor.collective_rpc("list_loras", timeout=30) == []
    os.kill(executor.procs[0].pid, signal.SIGKILL)
    executor.procs[0].join(10)
    assert not executor.check_health()
    with pytest.raises(WorkerDeadError, match="died"):
        executor.collective_rpc("list_loras", timeout=30)


def test_frozen_worker_is_detected_by_missing_heartbeats(executor):
    assert executor.collective_rpc("check_health", timeout=30) is True
    os.kill(executor.procs[0].pid, signal.SIGSTOP)          # alive for the OS, but makes no progress
    t0 = time.monotonic()
    with pytest.raises(WorkerDeadError, match="stopped responding"):
        executor.collective_rpc("list_loras", timeout=60)
    assert time.monotonic() - t0 < 10
    assert executor.check_health()                           # process exists: only the heartbeat tells
    os.kill(executor.procs[0].pid, signal.SIGCONT)


def test_rpc_time_limit(executor):
    executor.heartbeat_stall_s = 60.0                        # the call's own limit must fire first
    os.kill(executor.procs[0].pid, signal.SIGSTOP)
    with pytest.raises(TimeoutError):
        executor.collective_rpc("list_loras", timeout=1.0)
    os.kill(executor.procs[0].pid, signal.SIGCONT)
    # the late reply of the timed-out call must not be taken for the next call's answer
    assert executor.collective_rpc("check_health", timeout=30) is True


TTS_PROC_YAML = """
stage_args:
  - stage_id: 0
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 2, process: true}
    engine_args: {model_stage: qwen3_tts, model_arch: Qwen3TTSForConditionalGeneration, worker_type: generation,
                  engine_output_type: audio, device: cpu, model_overrides: {tiny: true}}
    final_output: true
    final_output_type: audio
"""


def test_dead_stage_fails_inflight_requests_and_is_restarted(tmp_path):
    """A stage process is killed while a request is inside it: the request fails with a typed error,
    the stage is started again and the next request is served."""
    import asyncio

    from vllm_omni_b200.entrypoints.async_omni import AsyncOmni
    from vllm_omni_b200.entrypoints.orchestrator import StageError
    from vllm_omni_b200.inputs import SamplingParams
    y = tmp_path / "tts_proc.yaml"
    y.write_text(TTS_PROC_YAML)

    async def run():
        eng = AsyncOmni("qwen3-tts-tiny", stage_configs_path=str(y), auto_restart_stages=True)
        try:
            sp = [SamplingParams(temperature=0.0, max_tokens=4, seed=1)]
            outs = [o async for o in eng.generate({"prompt_token_ids": [5, 6, 7]}, sampling_params_list=sp)]
            assert outs and outs[-1].final_output_type == "audio"
            first_pid = eng.stage_list[0]._worker.pid

            async def doomed():
                got = []
                with pytest.raises(StageError, match="died"):
                    async for o in eng.generate({"prompt_token_ids": [8, 9]}, request_id="doomed",
                                                sampling_params_list=[SamplingParams(temperature=0.0, max_tokens=60, seed=1)]):
                        got.append(o)
                return got

            task = asyncio.create_task(doomed())
            await asyncio.sleep(0.05)
            os.kill(first_pid, signal.SIGKILL)
            await asyncio.wait_for(task, 60)
            # the router restarts the stage; wait until the new worker is in place
            for _ in range(600):
                if eng.stage_list[0]._worker.pid != first_pid and eng.stage_list[0].check_health():
                    break
                await asyncio.sleep(0.1)
            assert eng.stage_list[0]._worker.pid != first_pid and not eng.errored
            outs = [o async for o in eng.generate({"prompt_token_ids": [5, 6, 7]}, sampling_params_list=sp)]
            assert outs and outs[-1].multimodal_output["audio"].numel() > 0
        finally:
            eng.close()

    asyncio.run(run())


FAULTY_EDGE_YAML = """
async_chunk: false
stage_args:
  - stage_id: 0
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 4}
    engine_args: {model_stage: thinker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                  engine_output_type: latent, device: cpu, num_gpu_blocks: 64, max_num_batched_tokens: 64,
                  model_overrides: {tiny: true}}
    final_output: true
    final_output_type: text
    default_sampling_params: {temperature: 0.0, max_tokens: 4}
  - stage_id: 1
    stage_type: llm
    runtime: {devices: "0", max_batch_size: 4, process: true}
    engine_args: {model_stage: talker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                  engine_output_type: latent, device: cpu, num_gpu_blocks: 64, model_overrides: {tiny: true}}
    engine_input_source: [0]
    custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.thinker2talker
    final_output: true
    final_output_type: latent
    default_sampling_params: {temperature: 0.0, max_tokens: 3, detokenize: false, stop_token_ids: [66]}
runtime:
  connectors:
    flaky:
      name: FaultInjectionConnector
      extra:
        inner: {name: SharedMemoryConnector, extra: {shm_threshold_bytes: 64, get_retries: 2, get_retry_interval_s: 0.01}}
        schedule: [corrupt]
  edges:
    - {from: 0, to: 1, connector: flaky}
"""


def test_corrupted_stage_payload_fails_one_request_and_the_pipeline_keeps_serving(tmp_path):
    """The thinker -> talker edge of a process-separated pipeline corrupts the first payload: that
    request ends with a checksum error from the receiving stage, the next one goes through."""
    from vllm_omni_b200.entrypoints.omni import Omni
    y = tmp_path / "faulty_edge.yaml"
    y.write_text(FAULTY_EDGE_YAML)
    o = Omni("qwen3-omni-tiny", stage_configs_path=str(y))
    try:
        prompt = {"prompt_token_ids": [506, 509, 11, 12, 507, 506, 510, 13]}
        from vllm_omni_b200.entrypoints.orchestrator import StageError
        with pytest.raises(StageError, match="checksum"):
            o.generate([prompt])
        second = o.generate([prompt])
        assert not [x.error for x in second if x.error]
        assert any(x.stage_id == 1 for x in second)
    finally:
        o.close()
