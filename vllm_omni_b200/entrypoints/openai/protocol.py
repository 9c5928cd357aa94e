"""Request / response schemas of the OpenAI-compatible server
(vllm_omni/entrypoints/openai/protocol/{images,videos,audio,chat_completion}.py)."""
from __future__ import annotations

import time
from enum import Enum
from typing import Any, Literal

from pydantic import BaseModel, Field


class ResponseFormat(str, Enum):
    B64_JSON = "b64_json"
    URL = "url"


class ImageGenerationRequest(BaseModel):
    prompt: str = Field(..., description="Text description of the desired image(s)")
    model: str | None = None
    n: int = Field(default=1, ge=1, le=10)
    size: str | None = Field(default=None, description="WIDTHxHEIGHT, e.g. 1024x1024")
    response_format: ResponseFormat = ResponseFormat.B64_JSON
    user: str | None = None
    negative_prompt: str | None = None
    num_inference_steps: int | None = Field(default=None, ge=1, le=200)
    guidance_scale: float | None = Field(default=None, ge=0.0, le=20.0)
    true_cfg_scale: float | None = Field(default=None, ge=0.0, le=20.0)
    seed: int | None = None
    generator_device: str | None = None
    lora: dict[str, Any] | None = None
    vae_use_slicing: bool | None = False
    vae_use_tiling: bool | None = False


class ImageData(BaseModel):
    b64_json: str | None = None
    url: str | None = None
    revised_prompt: str | None = None


class ImageGenerationResponse(BaseModel):
    created: int = Field(default_factory=lambda: int(time.time()))
    data: list[ImageData]
    output_format: str | None = "png"
    size: str | None = None


class VideoGenerationRequest(BaseModel):
    prompt: str
    model: str | None = None
    size: str | None = None
    num_frames: int | None = Field(default=None, ge=1, le=257)
    fps: int | None = Field(default=None, ge=1, le=60)
    negative_prompt: str | None = None
    num_inference_steps: int | None = Field(default=None, ge=1, le=200)
    guidance_scale: float | None = None
    seed: int | None = None
    response_format: Literal["b64_json", "frames_b64"] = "b64_json"
    image: str | None = Field(default=None, description="base64 conditioning image (image-to-video)")


class VideoData(BaseModel):
    b64_json: str | None = None
    frames_b64: list[str] | None = None
    format: str = "gif"
    fps: int = 16


class VideoGenerationResponse(BaseModel):
    created: int = Field(default_factory=lambda: int(time.time()))
    data: list[VideoData]


class OpenAICreateSpeechRequest(BaseModel):
    input: str
    model: str | None = None
    voice: str | None = None
    instructions: str | None = None
    response_format: Literal["wav", "pcm", "flac", "mp3", "aac", "opus"] = "wav"
    speed: float | None = Field(default=1.0, ge=0.25, le=4.0)
    stream_format: Literal["sse", "audio"] | None = "audio"
    task_type: Literal["CustomVoice", "VoiceDesign", "Base"] | None = None
    language: str | None = None
    ref_audio: str | None = None
    ref_text: str | None = None
    x_vector_only_mode: bool | None = None
    max_new_tokens: int | None = None


class ChatMessage(BaseModel):
    role: str
    content: Any = None
    audio: dict[str, Any] | None = None


class ChatCompletionRequest(BaseModel):
    model: str | None = None
    messages: list[ChatMessage]
    stream: bool = False
    max_tokens: int | None = None
    max_completion_tokens: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    seed: int | None = None
    stop: list[str] | str | None = None
    n: int = 1
    modalities: list[str] | None = None              # ["text"], ["text", "audio"], ["image"]
    audio: dict[str, Any] | None = None              # {"format": "wav", "voice": ...}
    sampling_params_list: list[dict[str, Any]] | None = None   # one dict per stage
    extra_body: dict[str, Any] | None = None
    user: str | None = None
    # diffusion-as-chat extras
    size: str | None = None
    num_inference_steps: int | None = None
    guidance_scale: float | None = None
    true_cfg_scale: float | None = None
    negative_prompt: str | None = None


class ChatCompletionAudio(BaseModel):
    id: str
    data: str                 # base64 wav
    expires_at: int
    transcript: str | None = None


class ChatChoiceMessage(BaseModel):
    role: str = "assistant"
    content: Any = None
    audio: ChatCompletionAudio | None = None


class ChatChoice(BaseModel):
    index: int = 0
    message: ChatChoiceMessage
    finish_reason: str | None = "stop"


class Usage(BaseModel):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0


class ChatCompletionResponse(BaseModel):
    id: str
    object: str = "chat.completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str | None = None
    choices: list[ChatChoice]
    usage: Usage = Field(default_factory=Usage)
    metrics: dict[str, Any] | None = None


class ErrorResponse(BaseModel):
    error: dict[str, Any]
