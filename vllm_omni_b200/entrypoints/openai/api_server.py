"""OpenAI-compatible HTTP server over ``AsyncOmni`` / ``AsyncOmniDiffusion``.

Routes (vllm_omni/entrypoints/openai/api_server.py:729-1589): ``GET /health``,
``GET /v1/models``, ``GET /metrics`` (Prometheus text), ``POST /v1/chat/completions``
(text, streamed text, audio output, image output for diffusion-as-chat),
``POST /v1/images/generations``, ``POST /v1/images/edits``, ``POST /v1/videos``,
``POST /v1/audio/speech``, ``GET /v1/audio/voices``.

``build_app(engine, model_name, kind)`` takes any object with the ``AsyncOmni`` interface, so
the API tests run against a mocked engine.
"""
from __future__ import annotations

import asyncio
import base64
import json
import time
import uuid
from typing import Any

from fastapi import FastAPI, File, Form, HTTPException, Request, UploadFile
from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse

from ...inputs.data import LoRARequest, OmniDiffusionSamplingParams, SamplingParams
from ...logger import init_logger
from . import media_utils as mu
from .protocol import (ChatChoice, ChatChoiceMessage, ChatCompletionAudio, ChatCompletionRequest,
                       ChatCompletionResponse, ImageData, ImageGenerationRequest, ImageGenerationResponse,
                       OpenAICreateSpeechRequest, Usage, VideoData, VideoGenerationRequest, VideoGenerationResponse)

logger = init_logger(__name__)

DEFAULT_VOICES = ["Vivian", "Ethan", "Chelsie", "Serena"]


def _err(status: int, msg: str, typ: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"error": {"message": msg, "type": typ, "code": status}}, status_code=status)


def _parse_lora_request(lora: dict | None) -> tuple[LoRARequest | None, float]:
    """{"name": ..., "path": ..., "scale": ...} -> LoRARequest with a stable integer id."""
    if not lora:
        return None, 1.0
    name, path = lora.get("name") or lora.get("lora_name"), lora.get("path") or lora.get("lora_path")
    if not name or not path:
        raise ValueError("lora needs 'name' and 'path'")
    import hashlib
    lid = int.from_bytes(hashlib.sha256(f"{name}:{path}".encode()).digest()[:4], "little") & 0x7FFFFFFF
    return LoRARequest(name, lid or 1, path, float(lora.get("scale", 1.0))), float(lora.get("scale", 1.0))


def _flatten_content(content, placeholders: bool = False, style: str | None = None) -> tuple[str, dict]:
    """OpenAI message content -> (text, raw multimodal items).  Items: ``image`` PIL images, ``audio`` (waveform,
    rate) pairs, ``video`` frame lists.  With ``placeholders`` the text carries one placeholder group per item at
    the item's position in the message (the omni thinker expands it to the item's feature length)."""
    if content is None:
        return "", {}
    if isinstance(content, str):
        return content, {}
    from ...inputs import omni_processor as op
    text, mm = [], {}
    marks = op.placeholders_for(style)

    def _url(part, key):
        v = part.get(key)
        return v.get("url") if isinstance(v, dict) else v

    for part in content:
        t = part.get("type")
        if t == "text":
            text.append(part.get("text", ""))
        elif t == "image_url":
            url = _url(part, "image_url")
            if isinstance(url, str) and (url.startswith("data:") or len(url) > 256):
                mm.setdefault("image", []).append(mu.decode_image_base64(url))
                if placeholders:
                    text.append(marks["image"])
        elif t in ("input_audio", "audio_url"):
            src = part.get("input_audio") if t == "input_audio" else _url(part, "audio_url")
            data = src.get("data") if isinstance(src, dict) else src
            if not isinstance(data, str) or data.startswith(("http://", "https://")):
                raise ValueError("audio input must be inline (base64 or a data: URL); remote URLs are not fetched")
            mm.setdefault("audio", []).append(op.decode_audio_bytes(op.decode_data_url(data)))
            if placeholders:
                text.append(marks["audio"])
        elif t == "video_url":
            url = _url(part, "video_url")
            if not isinstance(url, str) or url.startswith(("http://", "https://")):
                raise ValueError("video input must be inline (a data: URL of an animated GIF); remote URLs are not fetched")
            mm.setdefault("video", []).append(op.gif_frames(op.decode_data_url(url)))
            if placeholders:
                text.append(marks["video"])
        elif t == "video_frames":
            fr = (part.get("video_frames") or {}).get("frames") or []
            mm.setdefault("video", []).append([mu.decode_image_base64(f) for f in fr])
            if placeholders:
                text.append(marks["video"])
    return "".join(text), mm


def build_app(engine, model_name: str = "omni", kind: str = "omni", default_stage_params=None) -> FastAPI:
    """kind: "omni" (multi-stage AR pipeline) or "diffusion" (image / video generation)."""
    app = FastAPI(title="vllm_omni_b200", version="0.1")
    app.state.engine, app.state.model_name, app.state.kind = engine, model_name, kind
    app.state.started = time.time()

    # ------------------------------------------------------------------ basics
    @app.get("/health")
    async def health():
        try:
            await engine.check_health()
        except Exception as e:   # noqa: BLE001
            return _err(503, f"unhealthy: {e}", "service_unavailable")
        return Response(status_code=200)

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": int(app.state.started),
                                             "owned_by": "vllm_omni_b200"}]}

    @app.get("/metrics")
    async def metrics():
        agg = getattr(engine, "metrics", None)
        return PlainTextResponse(agg.render_prometheus() if agg is not None else "")

    # ------------------------------------------------------------------ images
    async def _generate_image(prompt_obj, sp: OmniDiffusionSamplingParams, rid: str):
        outs = []
        async for o in _iter_generate(prompt_obj, rid, [sp], ["image"]):
            outs.append(o)
        imgs = [im for o in outs for im in (o.images or [])]
        if not imgs:
            raise HTTPException(500, "generation produced no image")
        return imgs

    async def _iter_generate(prompt, rid, sps, modalities):
        gen = engine.generate(prompt, request_id=rid, sampling_params_list=sps, output_modalities=modalities) \
            if kind == "omni" or hasattr(engine, "stage_list") else None
        if gen is not None:
            async for o in gen:
                yield o
        else:                                  # AsyncOmniDiffusion: one coroutine per request
            yield await engine.generate(prompt, sps[0], rid)

    @app.post("/v1/images/generations")
    async def images_generations(req: ImageGenerationRequest):
        try:
            w, h = mu.parse_size(req.size)
            lora, lscale = _parse_lora_request(req.lora)
        except ValueError as e:
            return _err(400, str(e))
        if req.response_format.value == "url":
            return _err(400, "response_format=url is not supported; use b64_json")
        if w % 16 or h % 16:
            return _err(400, "width and height must be multiples of 16")
        sp = OmniDiffusionSamplingParams(height=h, width=w, num_outputs_per_prompt=req.n, seed=req.seed,
                                         generator_device=req.generator_device, lora_request=lora, lora_scale=lscale)
        if req.num_inference_steps is not None:
            sp.num_inference_steps = req.num_inference_steps
        if req.guidance_scale is not None:
            sp.guidance_scale = req.guidance_scale
        if req.true_cfg_scale is not None:
            sp.true_cfg_scale = req.true_cfg_scale
        prompt: Any = req.prompt
        if req.negative_prompt is not None:
            prompt = {"prompt": req.prompt, "negative_prompt": req.negative_prompt}
        try:
            imgs = await _generate_image(prompt, sp, f"img-{uuid.uuid4().hex[:10]}")
        except HTTPException:
            raise
        except Exception as e:   # noqa: BLE001
            logger.exception("image generation failed")
            return _err(500, f"generation failed: {e}", "internal_error")
        return ImageGenerationResponse(data=[ImageData(b64_json=mu.encode_image_base64(im)) for im in imgs],
                                       size=f"{w}x{h}")

    @app.post("/v1/images/edits")
    async def images_edits(image: list[UploadFile] = File(...), prompt: str = Form(...), size: str | None = Form(None),
                           n: int = Form(1), negative_prompt: str | None = Form(None),
                           num_inference_steps: int | None = Form(None), true_cfg_scale: float | None = Form(None),
                           seed: int | None = Form(None)):
        from PIL import Image
        import io
        try:
            w, h = mu.parse_size(size, default=(0, 0))
            pil = [Image.open(io.BytesIO(await f.read())).convert("RGB") for f in image]
        except Exception as e:   # noqa: BLE001
            return _err(400, f"bad input: {e}")
        if w == 0:
            w, h = pil[0].size
            w, h = w // 16 * 16, h // 16 * 16
        sp = OmniDiffusionSamplingParams(height=h, width=w, num_outputs_per_prompt=n, seed=seed)
        if num_inference_steps is not None:
            sp.num_inference_steps = num_inference_steps
        if true_cfg_scale is not None:
            sp.true_cfg_scale = true_cfg_scale
        p = {"prompt": prompt, "multi_modal_data": {"image": pil if len(pil) > 1 else pil[0]}}
        if negative_prompt is not None:
            p["negative_prompt"] = negative_prompt
        try:
            imgs = await _generate_image(p, sp, f"edit-{uuid.uuid4().hex[:10]}")
        except HTTPException:
            raise
        except Exception as e:   # noqa: BLE001
            return _err(500, f"generation failed: {e}", "internal_error")
        return ImageGenerationResponse(data=[ImageData(b64_json=mu.encode_image_base64(im)) for im in imgs],
                                       size=f"{w}x{h}")

    # ------------------------------------------------------------------ videos
    @app.post("/v1/videos")
    async def videos(req: VideoGenerationRequest):
        try:
            w, h = mu.parse_size(req.size, default=(832, 480))
        except ValueError as e:
            return _err(400, str(e))
        sp = OmniDiffusionSamplingParams(height=h, width=w, seed=req.seed, num_frames=req.num_frames or 17,
                                         fps=req.fps or 16)
        if req.num_inference_steps is not None:
            sp.num_inference_steps = req.num_inference_steps
        if req.guidance_scale is not None:
            sp.guidance_scale = req.guidance_scale
        prompt: Any = {"prompt": req.prompt}
        if req.negative_prompt is not None:
            prompt["negative_prompt"] = req.negative_prompt
        if req.image:
            prompt["multi_modal_data"] = {"image": mu.decode_image_base64(req.image)}
        try:
            outs = [o async for o in _iter_generate(prompt, f"vid-{uuid.uuid4().hex[:10]}", [sp], ["video"])]
        except Exception as e:   # noqa: BLE001
            return _err(500, f"generation failed: {e}", "internal_error")
        data = []
        for o in outs:
            v = (o.multimodal_output or {}).get("video")
            if v is None:
                continue
            for clip in (v if isinstance(v, list) else [v]):
                if req.response_format == "frames_b64":
                    from PIL import Image
                    data.append(VideoData(frames_b64=[mu.encode_image_base64(Image.fromarray(f)) for f in clip],
                                          format="png", fps=sp.fps))
                else:
                    data.append(VideoData(b64_json=base64.b64encode(mu.frames_to_gif_bytes(clip, sp.fps)).decode(),
                                          format="gif", fps=sp.fps))
        if not data:
            return _err(500, "generation produced no video", "internal_error")
        return VideoGenerationResponse(data=data)

    # ------------------------------------------------------------------ speech
    def _known_voices():
        from ..utils import voices_of_checkpoint
        return (getattr(engine, "voices", None) or voices_of_checkpoint(getattr(engine, "model", None)) or DEFAULT_VOICES)

    @app.get("/v1/audio/voices")
    async def voices():
        return {"voices": _known_voices()}

    @app.post("/v1/audio/speech")
    async def speech(req: OpenAICreateSpeechRequest):
        if not req.input or not req.input.strip():
            return _err(400, "input must not be empty")
        if req.response_format not in ("wav", "pcm", "flac"):
            return _err(400, f"response_format {req.response_format!r} is not available in this build; use wav, pcm or flac")
        task = req.task_type or ("Base" if req.ref_audio else "CustomVoice")
        known = _known_voices()
        voice = req.voice
        if task == "CustomVoice":                        # a named voice; the other tasks describe or clone one
            voice = voice or known[0]
            if voice.lower() not in {k.lower() for k in known}:
                return _err(400, f"unknown voice {voice!r}; available: {known}")
        elif task == "Base" and not (req.ref_audio or voice):
            return _err(400, "voice cloning (task_type Base) needs ref_audio (a WAV file as base64 or a data: URL)")
        elif task == "VoiceDesign" and not req.instructions:
            return _err(400, "voice design (task_type VoiceDesign) needs instructions that describe the voice")
        info = {"voice": voice, "instructions": req.instructions, "language": req.language, "task_type": task,
                "ref_text": req.ref_text, "ref_audio": req.ref_audio, "x_vector_only_mode": req.x_vector_only_mode}
        prompt = {"prompt": req.input, "additional_information": {k: v for k, v in info.items() if v is not None}}
        sps = None
        if req.max_new_tokens:
            sps = [s.default_sampling_params() for s in getattr(engine, "stage_list", [])]
            for s in sps:
                if isinstance(s, SamplingParams):
                    s.max_tokens = req.max_new_tokens
        rid = f"tts-{uuid.uuid4().hex[:10]}"
        chunks, sr = [], 24000
        try:
            async for o in engine.generate(prompt, request_id=rid, sampling_params_list=sps,
                                           output_modalities=["audio"]):
                if o.final_output_type == "audio":
                    mm = o.multimodal_output
                    chunks.append(mm["audio"])
                    sr = int(mm.get("sample_rate", sr))
        except Exception as e:   # noqa: BLE001
            return _err(500, f"generation failed: {e}", "internal_error")
        if not chunks:
            return _err(500, "generation produced no audio", "internal_error")
        import torch
        wav = torch.cat([c.reshape(-1).float().cpu() for c in chunks])
        data, media = mu.encode_audio(wav, sr, req.response_format, req.speed or 1.0)
        return Response(content=data, media_type=media)

    # ------------------------------------------------------------------ chat
    def _stage_params_from_request(req: ChatCompletionRequest):
        stages = getattr(engine, "stage_list", None)
        if not stages:
            return None
        sps = [s.default_sampling_params() for s in stages]
        if req.sampling_params_list:
            if len(req.sampling_params_list) != len(sps):
                raise ValueError(f"sampling_params_list needs {len(sps)} entries (one per stage)")
            for sp, d in zip(sps, req.sampling_params_list):
                for k, v in d.items():
                    if hasattr(sp, k):
                        setattr(sp, k, v)
        first = sps[0]
        if isinstance(first, SamplingParams):
            mt = req.max_completion_tokens or req.max_tokens
            if mt is not None:
                first.max_tokens = mt
            for k in ("temperature", "top_p", "top_k", "seed"):
                v = getattr(req, k)
                if v is not None:
                    setattr(first, k, v)
            if req.stop:
                first.stop = [req.stop] if isinstance(req.stop, str) else list(req.stop)
        return sps

    async def _diffusion_chat(req: ChatCompletionRequest, rid: str):
        text, mm = _flatten_content(req.messages[-1].content)
        eb = req.extra_body or {}
        w, h = mu.parse_size(req.size or eb.get("size"))
        sp = OmniDiffusionSamplingParams(height=h, width=w, seed=req.seed if req.seed is not None else eb.get("seed"))
        for k in ("num_inference_steps", "guidance_scale", "true_cfg_scale"):
            v = getattr(req, k) if getattr(req, k) is not None else eb.get(k)
            if v is not None:
                setattr(sp, k, v)
        prompt: Any = {"prompt": text}
        neg = req.negative_prompt or eb.get("negative_prompt")
        if neg is not None:
            prompt["negative_prompt"] = neg
        if mm.get("image"):
            prompt["multi_modal_data"] = {"image": mm["image"][0] if len(mm["image"]) == 1 else mm["image"]}
        imgs = await _generate_image(prompt, sp, rid)
        content = [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + mu.encode_image_base64(im)}}
                   for im in imgs]
        return ChatCompletionResponse(id=rid, model=model_name, choices=[ChatChoice(message=ChatChoiceMessage(
            content=content))])

    @app.post("/v1/chat/completions")
    async def chat(req: ChatCompletionRequest, raw: Request):
        rid = f"chatcmpl-{uuid.uuid4().hex[:12]}"
        if not req.messages:
            return _err(400, "messages must not be empty")
        if kind == "diffusion":
            try:
                return await _diffusion_chat(req, rid)
            except ValueError as e:
                return _err(400, str(e))
            except HTTPException:
                raise
            except Exception as e:   # noqa: BLE001
                return _err(500, f"generation failed: {e}", "internal_error")
        try:
            sps = _stage_params_from_request(req)
        except ValueError as e:
            return _err(400, str(e))
        modalities = req.modalities or ["text"]
        tok = getattr(engine, "tokenizer", None)
        msgs = []
        mm_all: dict = {}
        try:
            for m in req.messages:
                t, mm = _flatten_content(m.content, placeholders=True,
                                         style=(getattr(engine, "mm_processor_kwargs", None) or {}).get("style"))
                msgs.append({"role": m.role, "content": t})
                for k, v in mm.items():
                    mm_all.setdefault(k, []).extend(v)
            if mm_all:
                # raw items -> the tensors the thinker's towers take (pixels, frames, log-mel features)
                from ...inputs.omni_processor import thinker_inputs
                mm_all = thinker_inputs(mm_all, **(getattr(engine, "mm_processor_kwargs", None) or {}))
        except ValueError as e:
            return _err(400, str(e))
        if tok is not None and hasattr(tok, "apply_chat_template"):
            text = tok.apply_chat_template(msgs, add_generation_prompt=True, tokenize=False)
        else:
            text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in msgs) + "<|im_start|>assistant\n"
        prompt: Any = {"prompt": text}
        if mm_all:
            prompt["multi_modal_data"] = mm_all
        if req.audio and req.audio.get("voice"):
            prompt["additional_information"] = {"voice": req.audio["voice"]}

        if req.stream:
            async def sse():
                sent = 0
                first = True
                try:
                    async for o in engine.generate(prompt, request_id=rid, sampling_params_list=sps,
                                                   output_modalities=modalities):
                        if await raw.is_disconnected():
                            await engine.abort(rid)
                            return
                        delta: dict = {}
                        if o.final_output_type == "text" and o.outputs:
                            full = o.outputs[0].text
                            if len(full) > sent:
                                delta["content"] = full[sent:]
                                sent = len(full)
                            elif not o.finished:
                                continue
                        elif o.final_output_type == "audio" and "audio" in modalities:
                            mm = o.multimodal_output
                            wav = mu.wav_bytes(mm["audio"], int(mm.get("sample_rate", 24000)))
                            delta["audio"] = {"id": f"audio-{rid}", "data": base64.b64encode(wav).decode()}
                        else:
                            continue
                        if first:
                            delta["role"] = "assistant"
                            first = False
                        fin = "stop" if (o.finished and o.final_output_type == "text") else None
                        chunk = {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()),
                                 "model": model_name, "modality": o.final_output_type,
                                 "choices": [{"index": 0, "delta": delta, "finish_reason": fin}]}
                        yield f"data: {json.dumps(chunk)}\n\n"
                except Exception as e:   # noqa: BLE001
                    yield f"data: {json.dumps({'error': {'message': str(e), 'type': 'internal_error'}})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")

        text_out, audio_parts, sr, usage, finish = "", [], 24000, Usage(), "stop"
        try:
            async for o in engine.generate(prompt, request_id=rid, sampling_params_list=sps,
                                           output_modalities=modalities):
                if o.final_output_type == "text" and o.outputs:
                    text_out = o.outputs[0].text
                    if o.finished:
                        finish = o.outputs[0].finish_reason or "stop"
                        usage = Usage(prompt_tokens=len(o.prompt_token_ids or []),
                                      completion_tokens=len(o.outputs[0].token_ids),
                                      total_tokens=len(o.prompt_token_ids or []) + len(o.outputs[0].token_ids))
                elif o.final_output_type == "audio":
                    mm = o.multimodal_output
                    audio_parts.append(mm["audio"])
                    sr = int(mm.get("sample_rate", sr))
        except Exception as e:   # noqa: BLE001
            logger.exception("chat failed")
            return _err(500, f"generation failed: {e}", "internal_error")
        msg = ChatChoiceMessage(content=text_out)
        if audio_parts and "audio" in modalities:
            import torch
            wav = torch.cat([a.reshape(-1).float().cpu() for a in audio_parts])
            msg.audio = ChatCompletionAudio(id=f"audio-{rid}", data=base64.b64encode(mu.wav_bytes(wav, sr)).decode(),
                                            expires_at=int(time.time()) + 3600, transcript=text_out)
        agg = getattr(engine, "metrics", None)
        return ChatCompletionResponse(id=rid, model=model_name, choices=[ChatChoice(message=msg, finish_reason=finish)],
                                      usage=usage, metrics=agg.build_summary()["overall"] if agg is not None else None)

    return app


def omni_run_server(model: str, host: str = "0.0.0.0", port: int = 8000, **kwargs):
    """Build the engine for ``model`` and serve it (blocking)."""
    import uvicorn
    from ..async_omni import AsyncOmni
    engine = AsyncOmni(model, **kwargs)
    kind = "diffusion" if all(s.stage_type == "diffusion" for s in engine.stage_list) else "omni"
    app = build_app(engine, model_name=kwargs.get("served_model_name") or model, kind=kind)
    try:
        uvicorn.run(app, host=host, port=port, log_level="info")
    finally:
        engine.close()
