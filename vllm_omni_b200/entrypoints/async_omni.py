"""``AsyncOmni``: asyncio front-end over the staged pipeline.

``generate`` is an async generator per request (vllm_omni/entrypoints/async_omni.py:235-361).
One background thread polls every stage's result queue and routes results: outputs of final
stages go to the request's asyncio queue (text deltas stream while the stage is still
running), finished outputs of a stage become the inputs of its consumers (sequential mode,
async_omni.py:408-473).  With ``async_chunk`` enabled both edges of the omni pipeline stream: the
talker starts from a thinker that is still generating (its rows follow as update tasks), and codec
frames of a running talker are forwarded to the vocoder stage in chunks of 25 frames (+25 frames of
left context), so audio starts shortly after the first text tokens
(async_omni.py:363-406, chunk_transfer_adapter.py, stage_input_processors/qwen3_omni.py:86-141).
``abort`` reaches every stage; ``pause_generation`` / ``resume_generation`` gate new work.
"""
from __future__ import annotations

import asyncio
import threading
import time
import uuid
from typing import Any, AsyncGenerator, Sequence

import torch

from ..logger import init_logger
from ..outputs import CompletionOutput, OmniRequestOutput, RequestOutput
from .omni_base import OmniBase
from .orchestrator import StageError, send_downstream, wrap_stage_output
from .stage_utils import OmniStageTaskType

logger = init_logger(__name__)

_DONE = object()


class _ReqState:
    def __init__(self, rid, prompt, sps, loop, modalities):
        self.rid, self.prompt, self.sps, self.loop = rid, prompt, sps, loop
        self.queue: asyncio.Queue = asyncio.Queue()
        self.done_stages: set[int] = set()
        self.modalities = modalities
        self.t0 = time.time()
        self.emitted_frames = 0          # async-chunk bookkeeping (talker -> code2wav)
        self.chunk_idx = 0
        self.audio_chunks_expected = None
        self.audio_chunks_seen = 0
        self.first_output_ts: dict[str, float] = {}
        self.codes_parts: list = []
        self.row_parts: list = []        # async-chunk bookkeeping (thinker -> talker): rows not yet forwarded
        self.hid_parts: list = []
        self.tts_rows: dict = {}
        self.talker_started = False
        self.rows_sent = 0
        self.hid_key = None


class AsyncOmni(OmniBase):
    def __init__(self, model: str | None = None, **kwargs):
        # auto_restart_stages: when a stage worker dies, fail the requests in flight with a typed
        # error, start a fresh worker for that stage and keep serving (instead of declaring the whole
        # engine dead)
        self.auto_restart = bool(kwargs.pop("auto_restart_stages", False))
        super().__init__(model, **kwargs)
        self.async_chunk = bool(self.stage_configs.async_chunk)
        self.stream_starts = 0            # requests whose talker was started from a thinker that was still running
        self._states: dict[str, _ReqState] = {}
        self._lock = threading.Lock()
        self._paused = asyncio.Event() if False else None
        self._pause_flag = threading.Event()
        self._pause_flag.set()                     # set = running
        self._stop = threading.Event()
        self.consumers = {s.stage_id: [d for d in self.stage_list if s.stage_id in d.engine_input_source]
                          for s in self.stage_list}
        self.final_stages = [s.stage_id for s in self.stage_list if s.final_output] or [self.stage_list[-1].stage_id]
        self.must_finish = set(self.final_stages) | {s.stage_id for s in self.stage_list
                                                     if not self.consumers[s.stage_id]}
        self._errored = None
        self._thread = threading.Thread(target=self._output_handler, name="omni-output-handler", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ public API
    async def generate(self, prompt, request_id: str | None = None, sampling_params_list: Any = None,
                       output_modalities: Sequence[str] | None = None) -> AsyncGenerator[OmniRequestOutput, None]:
        while not self._pause_flag.is_set():
            await asyncio.sleep(0.005)
        if self._errored is not None:
            raise RuntimeError(f"engine is dead: {self._errored}")
        rid = request_id or f"req-{uuid.uuid4().hex[:10]}"
        if sampling_params_list is None:
            sampling_params_list = [s.default_sampling_params() for s in self.stage_list]
        elif not isinstance(sampling_params_list, (list, tuple)):
            sampling_params_list = [sampling_params_list]
        if len(sampling_params_list) < self.num_stages:
            sampling_params_list = list(sampling_params_list) + [
                s.default_sampling_params() for s in self.stage_list[len(sampling_params_list):]]
        st = _ReqState(rid, prompt, list(sampling_params_list), asyncio.get_running_loop(), output_modalities)
        with self._lock:
            if rid in self._states:
                raise ValueError(f"request id {rid!r} is already in flight")
            self._states[rid] = st
        self.metrics.on_request_start(rid, st.t0)
        self.stage_list[0].submit({"type": OmniStageTaskType.GENERATE, "request_id": rid, "engine_inputs": prompt,
                                   "sampling_params": st.sps[0]})
        try:
            while True:
                item = await st.queue.get()
                if item is _DONE:
                    break
                if isinstance(item, Exception):
                    raise item
                yield item
        except (asyncio.CancelledError, GeneratorExit):
            await self.abort(rid)
            raise
        finally:
            with self._lock:
                self._states.pop(rid, None)

    async def abort(self, request_id: str | Sequence[str]) -> None:
        ids = [request_id] if isinstance(request_id, str) else list(request_id)
        for s in self.stage_list:
            s.abort(ids)
        with self._lock:
            for rid in ids:
                st = self._states.pop(rid, None)
                if st is not None:
                    st.loop.call_soon_threadsafe(st.queue.put_nowait, _DONE)

    async def pause_generation(self, wait_for_inflight: bool = True) -> None:
        self._pause_flag.clear()
        for s in self.stage_list:
            s.pause()
        if wait_for_inflight:
            while self._states:
                await asyncio.sleep(0.005)

    async def resume_generation(self) -> None:
        for s in self.stage_list:
            s.resume()
        self._pause_flag.set()

    @property
    def is_paused(self) -> bool:
        return not self._pause_flag.is_set()

    @property
    def is_running(self) -> bool:
        return self._errored is None and self._thread.is_alive()

    @property
    def errored(self) -> bool:
        return self._errored is not None

    async def check_health(self) -> None:
        if self._errored is not None:
            raise RuntimeError(f"engine is dead: {self._errored}")
        for s in self.stage_list:
            if not s.check_health():
                raise RuntimeError(f"stage {s.stage_id} worker is not alive")

    # EngineClient-style shims kept for API parity with serving layers
    async def get_model_config(self):
        return {"model": self.model, "num_stages": self.num_stages}

    async def is_sleeping(self) -> bool:
        return False

    async def sleep(self, level: int = 1) -> None:
        for s in self.stage_list:
            s.submit({"type": OmniStageTaskType.PAUSE})

    async def wake_up(self, tags=None) -> None:
        for s in self.stage_list:
            s.submit({"type": OmniStageTaskType.RESUME})

    async def add_lora(self, lora_request) -> bool:
        return False

    # ------------------------------------------------------------------ router thread
    def _post(self, st: _ReqState, item) -> None:
        st.loop.call_soon_threadsafe(st.queue.put_nowait, item)

    def _output_handler(self) -> None:
        while not self._stop.is_set():
            progressed = False
            for stage in self.stage_list:
                res = stage.try_collect()
                if res is None:
                    continue
                progressed = True
                try:
                    self._route(stage, res)
                except Exception as e:   # noqa: BLE001
                    logger.exception("routing failed")
                    rid = res.get("request_id")
                    st = self._states.get(rid)
                    if st is not None:
                        self._post(st, e)
                        self._post(st, _DONE)
            if not progressed:
                for s in list(self.stage_list):
                    if not s.check_health() and not self._stop.is_set():
                        why = f"stage {s.stage_id} worker died"
                        with self._lock:
                            lost = list(self._states)
                            for st in self._states.values():
                                self._post(st, StageError(s.stage_id, st.rid, why, ""))
                                self._post(st, _DONE)
                            self._states.clear()
                        if self.auto_restart:
                            for other in self.stage_list:          # drop what the lost requests left behind
                                if other is not s and other.check_health() and lost:
                                    other.abort(lost)
                            try:
                                self.restart_stage(s.stage_id)
                                self._rewire()
                                continue
                            except Exception as e:   # noqa: BLE001
                                why = f"{why}; restart failed: {e}"
                        self._errored = why
                        return
                time.sleep(0.0005)

    def _rewire(self) -> None:
        """Consumer lists hold stage objects: rebuild them after a stage was replaced."""
        self.consumers = {s.stage_id: [d for d in self.stage_list if s.stage_id in d.engine_input_source]
                          for s in self.stage_list}

    def _route(self, stage, res: dict) -> None:
        if res.get("type") in ("profile", "stage_stopped", "stage_ready"):
            return
        rid = res.get("request_id")
        st = self._states.get(rid)
        if st is None:
            return
        if "error" in res:
            self._post(st, StageError(stage.stage_id, rid, res["error"], res.get("error_tb", "")))
            self._post(st, _DONE)
            for s in self.stage_list:
                s.abort([rid])
            return
        outs = res.get("engine_outputs")
        outs = outs if isinstance(outs, list) else [outs]
        finished = res.get("finished", True)
        sid = stage.stage_id
        if sid in self.final_stages:
            for o in outs:
                w = wrap_stage_output(stage, o)
                w.request_id = w.request_id or rid
                if w.is_pipeline_output:
                    w.final_output_type = stage.final_output_type
                w.finished = bool(finished)
                if st.modalities is None or w.final_output_type in st.modalities or w.final_output_type == "text":
                    st.first_output_ts.setdefault(w.final_output_type, time.time())
                    self._post(st, w)
        if self.async_chunk and not finished:
            self._forward_chunks(stage, st, outs, finished=False)
            self._stream_rows(stage, st, outs, finished=False)
        if not finished:
            return
        stage.set_engine_outputs(outs)
        if "metrics" in res:
            self.metrics.on_stage_metrics(sid, rid, res["metrics"])
        if self.async_chunk and self._chunk_consumers(stage):
            self._forward_chunks(stage, st, outs, finished=True)
            plain = [d for d in self.consumers[sid] if d not in self._chunk_consumers(stage)]
        else:
            plain = self.consumers[sid]
        if self.async_chunk and self._stream_rows(stage, st, outs, finished=True):
            plain = [d for d in plain if d not in self._row_consumers(stage)]      # they were started from the stream
        if self._is_chunk_sink(stage):
            # the vocoder finishes once per chunk; the stage is done for this request only when
            # the talker has finished and every chunk it produced has come back
            st.audio_chunks_seen += 1
            if st.audio_chunks_expected is None or st.audio_chunks_seen < st.audio_chunks_expected:
                return
        for dst in plain:
            send_downstream(self, stage, dst, rid, st.prompt, st.sps[dst.stage_id])
        st.done_stages.add(sid)
        if st.audio_chunks_expected is not None and st.audio_chunks_seen >= st.audio_chunks_expected:
            st.done_stages.update(d.stage_id for d in self._chunk_consumers(stage))
        if self.must_finish <= st.done_stages:
            self.metrics.on_finalize_request(rid)
            self._post(st, _DONE)

    # ------------------------------------------------------------------ async chunk (thinker -> talker)
    def _row_consumers(self, stage):
        """Consumers that can start from a thinker that is still generating."""
        if stage.model_stage != "thinker":
            return []
        return [d for d in self.consumers[stage.stage_id] if d.model_stage == "talker"]

    def _stream_rows(self, stage, st: _ReqState, outs, finished: bool) -> bool:
        """The thinker's progress reports carry its new rows every few tokens.  The talker is started as soon as
        the prompt rows and the first reply row exist (marked ``thinker_stream``); later rows, and the news that
        the thinker has finished, follow as UPDATE tasks.  Returns True when the talker runs from the stream
        (the whole-request hand-off is then skipped)."""
        dsts = self._row_consumers(stage)
        if not dsts:
            return False
        ro = getattr(outs[0], "request_output", None) or outs[0]
        comp = ro.outputs[0] if getattr(ro, "outputs", None) else None
        mm = (comp.multimodal_output if comp is not None else None) or {}
        if finished:
            if not st.talker_started:
                return False
            full = mm.get("0")
            new = full[st.rows_sent:] if full is not None else None
            for dst in dsts:
                dst.submit({"type": OmniStageTaskType.UPDATE, "request_id": st.rid,
                            "payload": {"thinker_embeddings": new, "finished": True}})
            return True
        hk = next((k for k in mm if k != "0" and str(k).isdigit()), None)
        if mm.get("0") is not None and mm["0"].shape[0]:
            st.row_parts.append(mm["0"])
            if hk is not None:
                st.hid_parts.append(mm[hk])
                st.hid_key = hk
        for k in ("tts_bos_embed", "tts_eos_embed", "tts_pad_embed"):
            if k in mm:
                st.tts_rows[k] = mm[k]
        if not st.row_parts:
            return st.talker_started
        rows = torch.cat(st.row_parts, 0)
        if not st.talker_started:
            n_prompt = len(ro.prompt_token_ids or [])
            if rows.shape[0] < n_prompt + 1 or len(st.tts_rows) < 3 or st.hid_key is None:
                return False
            import copy
            comp2 = copy.copy(comp)
            comp2.multimodal_output = {"0": rows, st.hid_key: torch.cat(st.hid_parts, 0), **st.tts_rows}
            comp2.token_ids = list(comp.token_ids)
            syn = copy.copy(ro)
            syn.outputs, syn.multimodal_output, syn.finished = [comp2], comp2.multimodal_output, False
            stage.set_engine_outputs([syn])
            for dst in dsts:
                send_downstream(self, stage, dst, st.rid, st.prompt, st.sps[dst.stage_id], mark={"thinker_stream": True})
            st.talker_started = True
            self.stream_starts += 1
        else:
            for dst in dsts:
                dst.submit({"type": OmniStageTaskType.UPDATE, "request_id": st.rid,
                            "payload": {"thinker_embeddings": rows, "finished": False}})
        st.rows_sent += rows.shape[0]
        st.row_parts, st.hid_parts = [], []
        return True

    # ------------------------------------------------------------------ async chunk (talker -> code2wav)
    def _chunk_consumers(self, stage):
        """Consumers that take this stage's codec frames as a stream."""
        if stage.model_stage != "talker":
            return []
        return [d for d in self.consumers[stage.stage_id] if d.model_stage == "code2wav"]

    def _is_chunk_sink(self, stage) -> bool:
        return self.async_chunk and stage.model_stage == "code2wav"

    def _forward_chunks(self, stage, st: _ReqState, outs, finished: bool) -> None:
        dsts = self._chunk_consumers(stage)
        if not dsts:
            return
        from ..models.stage_input_processors.qwen3_omni import talker2code2wav_async_chunk
        ro = getattr(outs[0], "request_output", None) or outs[0]
        mm = ro.outputs[0].multimodal_output if ro.outputs else {}
        if finished:
            codes = mm.get("codes")                      # the final output carries every frame
        else:
            part = mm.get("codes")                       # streaming outputs carry only the new frames
            if part is not None and part.numel():
                st.codes_parts.append(part)
            codes = torch.cat(st.codes_parts, 0) if st.codes_parts else None
        if codes is None:
            return
        if finished and ro.outputs and ro.outputs[0].finish_reason == "stop":
            codes = codes[:-1]
        payload, new_emitted = talker2code2wav_async_chunk(codes, st.emitted_frames, finished)
        if finished:
            st.audio_chunks_expected = st.chunk_idx + (1 if payload is not None else 0)
            if st.audio_chunks_expected == 0:          # nothing to vocode at all
                st.audio_chunks_expected = None
                st.done_stages.update(d.stage_id for d in dsts)
        if payload is None:
            return
        st.emitted_frames = new_emitted
        for dst in dsts:
            dst.submit({"type": OmniStageTaskType.GENERATE, "request_id": st.rid,
                        "engine_inputs": {"prompt_token_ids": [0] * payload["codes"].shape[0],
                                          "additional_information": payload},
                        "sampling_params": st.sps[dst.stage_id], "chunk_index": st.chunk_idx})
        st.chunk_idx += 1

    # ------------------------------------------------------------------ shutdown
    def close(self):
        self._stop.set()
        if hasattr(self, "_thread") and self._thread.is_alive() and threading.current_thread() is not self._thread:
            self._thread.join(timeout=2)
        super().close()

    shutdown = close
