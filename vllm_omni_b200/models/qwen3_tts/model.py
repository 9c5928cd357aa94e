"""Qwen3-TTS: text (plus an optional instruction / voice) to speech inside ONE generation stage
(vllm_omni/model_executor/models/qwen3_tts/qwen3_tts.py, modeling_qwen3_tts.py,
stage_configs/qwen3_tts.yaml).

Per request: text embeddings are projected into the talker's width and prefilled together with a
language / speaker prefix; the talker then emits one 12 Hz codec frame per step — code 0 from its
own head, codes 1..G-1 from the code predictor — until the codec EOS id or ``max_tokens``; the
frames are decoded by the speech tokenizer's decoder (the same causal conv / transformer stack as
Qwen3-Omni's code2wav) in chunks with left context.  The inner loop runs on a private paged KV
cache (``LocalDecodeSession``) instead of the reference's cache-less HF loop.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ...ops.sampler import RowParams, sample
from ..base import StageModel
from ..local_decode import LocalDecodeSession
from ..qwen3_omni.code2wav import Qwen3OmniCode2Wav
from ..qwen3_omni.config import Code2WavConfig, CodePredictorConfig, Qwen3OmniConfig
from ..qwen3_omni.talker import CodePredictor
from ..qwen_decoder import DecoderConfig, QwenDecoderModel


@dataclass
class Qwen3TTSConfig:
    text_vocab_size: int = 151936
    text_hidden_size: int = 2048
    talker: DecoderConfig = field(default_factory=lambda: DecoderConfig(
        vocab_size=3072, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
        head_dim=128, intermediate_size=3072, rope_theta=1e6))
    code_predictor: CodePredictorConfig = field(default_factory=CodePredictorConfig)
    tokenizer_decoder: Code2WavConfig = field(default_factory=lambda: Code2WavConfig(upsample_rates=(8, 5, 4, 3),
                                                                                    upsampling_ratios=(2, 2)))
    codec_bos_id: int = 2149
    codec_eos_id: int = 2150
    codec_pad_id: int = 2148
    num_speakers: int = 32
    num_languages: int = 16
    max_frames: int = 4096

    @classmethod
    def tiny(cls) -> "Qwen3TTSConfig":
        return cls(text_vocab_size=512, text_hidden_size=48,
                   talker=DecoderConfig(vocab_size=96, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                                        num_key_value_heads=2, head_dim=16, intermediate_size=64),
                   code_predictor=CodePredictorConfig(hidden_size=32, num_hidden_layers=1, num_attention_heads=2,
                                                      num_key_value_heads=2, head_dim=16, intermediate_size=64,
                                                      vocab_size=64, num_code_groups=4),
                   tokenizer_decoder=Code2WavConfig(codebook_size=64, num_quantizers=4, hidden_size=32,
                                                    num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2,
                                                    intermediate_size=64, decoder_dim=32, upsample_rates=(4, 2),
                                                    upsampling_ratios=(2,), chunk_size=12, left_context=3),
                   codec_bos_id=65, codec_eos_id=66, codec_pad_id=64, num_speakers=4, num_languages=2, max_frames=64)

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen3TTSConfig":
        c = cls()
        tk = d.get("talker_config") or {}
        if tk:
            c.talker = DecoderConfig.from_dict(tk)
            for k in ("codec_bos_id", "codec_eos_id", "codec_pad_id"):
                if k in tk:
                    setattr(c, k, tk[k])
            if "text_hidden_size" in tk:
                c.text_hidden_size = tk["text_hidden_size"]
            if "text_vocab_size" in tk:
                c.text_vocab_size = tk["text_vocab_size"]
        return c


class Qwen3TTSModel(StageModel):
    engine_output_type = "audio"
    is_generation_model = True

    def __init__(self, cfg: Qwen3TTSConfig, dtype=torch.bfloat16, device=None):
        super().__init__(None, dtype, device)
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        Dt = cfg.talker.hidden_size
        self.text_embedding = nn.Parameter(torch.empty(cfg.text_vocab_size, cfg.text_hidden_size, **kw).normal_(0, 0.02),
                                           requires_grad=False)
        self.text_projection = FusedLinear(cfg.text_hidden_size, Dt, **kw)
        self.speaker_embedding = nn.Parameter(torch.empty(cfg.num_speakers, Dt, **kw).normal_(0, 0.02), requires_grad=False)
        self.language_embedding = nn.Parameter(torch.empty(cfg.num_languages, Dt, **kw).normal_(0, 0.02), requires_grad=False)
        self.talker = QwenDecoderModel(cfg.talker, dtype, device, with_lm_head=False)
        self.codec_head = FusedLinear(Dt, cfg.talker.vocab_size, bias=False, **kw)
        self.code_predictor = CodePredictor(cfg.code_predictor, Dt, dtype, device)
        oc = Qwen3OmniConfig.tiny()
        oc.code2wav = cfg.tokenizer_decoder
        self.decoder = Qwen3OmniCode2Wav(oc, dtype, device)          # speech tokenizer decoder
        self.speakers: dict[str, int] = {"default": 0}
        self.languages: dict[str, int] = {"auto": 0}
        self._session = None

    def _session_for(self, n_tokens: int) -> LocalDecodeSession:
        if self._session is None or self._session.max_len < n_tokens:
            self._session = LocalDecodeSession(self.talker, max(n_tokens, 256))
        self._session.reset()
        return self._session

    @torch.no_grad()
    def synthesize(self, text_ids, instruct_ids=None, speaker: str | int = "default", language: str | int = "auto",
                   temperature: float = 0.9, top_k: int = 50, seed: int = 0, max_frames: int | None = None):
        """Returns (codes [T, G] int64, waveform [T * up] fp32)."""
        cfg = self.cfg
        dev = self.text_embedding.device
        V = self.talker.embed_tokens.shape[0]
        codec = self.talker.embed_tokens
        ids = list(instruct_ids or []) + list(text_ids)
        tok = torch.tensor(ids, dtype=torch.long, device=dev).clamp(0, cfg.text_vocab_size - 1)
        text = self.text_projection(self.text_embedding[tok].contiguous())
        spk = self.speakers.get(speaker, 0) if isinstance(speaker, str) else int(speaker)
        lang = self.languages.get(language, 0) if isinstance(language, str) else int(language)
        prefix = torch.stack([self.language_embedding[lang % cfg.num_languages],
                              self.speaker_embedding[spk % cfg.num_speakers]], 0)
        head = torch.cat([prefix, text + codec[cfg.codec_pad_id % V][None], codec[cfg.codec_bos_id % V][None]], 0)
        max_frames = min(max_frames or cfg.max_frames, cfg.max_frames)
        sess = self._session_for(head.shape[0] + max_frames + 1)
        hidden = sess.prefill(embeds=head.to(self.dtype_))[-1:]
        frames = []
        for k in range(max_frames):
            logits = self.codec_head(hidden).float()
            if temperature <= 0:
                c0 = logits.argmax(-1)
            else:
                c0, _ = sample(logits, [RowParams(temperature=temperature, top_k=top_k, seed=seed, step=k)])
                c0 = c0.long()
            if int(c0) == cfg.codec_eos_id:
                break
            e0 = codec[c0.clamp(0, V - 1)]
            rest, summed = self.code_predictor.generate(hidden.to(self.dtype_), e0, temperature=temperature,
                                                        seed=seed, step=k)
            frames.append(torch.cat([c0[:, None], rest], 1))
            hidden = sess.step(embed=(e0 + summed).to(self.dtype_))
        G = cfg.code_predictor.num_code_groups
        codes = torch.cat(frames, 0) if frames else torch.zeros(0, G, dtype=torch.long, device=dev)
        wav = self.decoder.chunked_decode(codes.t()[None].contiguous())[0] if frames else torch.zeros(0, device=dev)
        return codes, wav.float()

    def generate_for(self, req, start, n):
        info = req.additional_information or {}
        sp = req.sampling_params
        codes, wav = self.synthesize(
            req.prompt_token_ids[start:start + n], instruct_ids=info.get("instruct_token_ids"),
            speaker=info.get("speaker", info.get("voice", "default")), language=info.get("language", "auto"),
            temperature=sp.temperature, top_k=sp.top_k if sp.top_k and sp.top_k > 0 else 50, seed=sp.seed or 0,
            max_frames=sp.max_tokens)
        return {"audio": wav, "codes": codes, "sample_rate": self.cfg.tokenizer_decoder.sample_rate}

    def load_weights(self, weights):
        ws = list(weights)
        loaded = set(self.talker.load_weights(((n[len("talker."):], w) for n, w in ws if n.startswith("talker."))))
        return {"talker." + n for n in loaded}


def build_qwen3_tts_stage(model_stage, hf_config: dict, dtype, device, **kw):
    if kw.get("tiny") or (hf_config or {}).get("tiny"):
        cfg = Qwen3TTSConfig.tiny()
    elif hf_config:
        cfg = Qwen3TTSConfig.from_hf(hf_config)
    else:
        cfg = Qwen3TTSConfig()
    return Qwen3TTSModel(cfg, dtype, device)
