"""Qwen3-TTS: text (plus an optional instruction, a named voice, or a cloned voice) to speech inside
ONE generation stage (vllm_omni/model_executor/models/qwen3_tts/qwen3_tts.py:65-150,
modeling_qwen3_tts.py:1406-2316, stage_configs/qwen3_tts.yaml).

Module tree and checkpoint names follow the published model: ``talker.model.{text_embedding,
codec_embedding, layers, norm}``, ``talker.text_projection.linear_fc1/2`` (Linear, SiLU, Linear with
biases), ``talker.codec_head``, ``talker.code_predictor.{model.*, lm_head.N, small_to_mtp_projection}``,
``speaker_encoder.*``; the 12 Hz speech tokenizer lives in the checkpoint's ``speech_tokenizer/``
folder.

Prompt rows (talker width), for the ChatML text ``<|im_start|>assistant\\n TEXT <|im_end|>\\n
<|im_start|>assistant\\n``:

    [instruction rows: projected text embeddings of ``<|im_start|>user\\n INSTRUCT <|im_end|>\\n``]
    3 role rows        projected text embeddings of ``<|im_start|> assistant \\n``
    codec prefix rows  codec embeddings of [nothink, think_bos, think_eos] (language "auto") or
                       [think, think_bos, LANGUAGE, think_eos], then the speaker row (a named voice's
                       codec token or a cloned voice's x-vector) if any, then codec_pad; each added to
                       the projected ``tts_pad`` text embedding, the last one to ``tts_bos``
    first text row     projected first text token + codec_bos

Every later step feeds the sum of the previous frame's G code embeddings plus the next text token's
projection (then ``tts_eos``, then ``tts_pad`` for as long as speech continues).  In-context voice
cloning prepends the reference text to the text and the reference frames to the codec stream.
Code 0 of a frame comes from the talker's head (ids of the last 1024 vocabulary slots other than EOS
are suppressed, EOS is not allowed in the first two frames, repetition penalty 1.05), codes 1..G-1
from the code predictor.  The inner loop runs on a private paged KV cache
(``LocalDecodeSession``) instead of the reference's HF ``generate`` loop.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import torch
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ...ops.sampler import RowParams, sample
from ..base import StageModel
from ..local_decode import LocalDecodeSession
from ..qwen3_omni.config import CodePredictorConfig
from ..qwen3_omni.talker import CodePredictor, ResizeMLP
from ..qwen_decoder import DecoderConfig, QwenDecoderModel
from .speaker import Qwen3TTSSpeakerEncoder, SpeakerEncoderConfig
from .tokenizer_12hz import Qwen3TTSTokenizerDecoder, TokenizerDecoderConfig


@dataclass
class Qwen3TTSConfig:
    text_vocab_size: int = 151936
    text_hidden_size: int = 2048
    talker: DecoderConfig = field(default_factory=lambda: DecoderConfig(
        vocab_size=3072, hidden_size=1024, num_hidden_layers=20, num_attention_heads=16, num_key_value_heads=2,
        head_dim=64, intermediate_size=2048, rope_theta=1e4))
    code_predictor: CodePredictorConfig = field(default_factory=lambda: CodePredictorConfig(num_code_groups=32, rope_theta=1e4))
    tokenizer_decoder: TokenizerDecoderConfig = field(default_factory=TokenizerDecoderConfig)
    speaker_encoder: SpeakerEncoderConfig | None = None
    tts_model_type: str = "custom_voice"            # custom_voice | voice_design | base (voice cloning)
    codec_eos_id: int = 4198
    codec_think_id: int = 4202
    codec_nothink_id: int = 4203
    codec_think_bos_id: int = 4204
    codec_think_eos_id: int = 4205
    codec_pad_id: int = 4196
    codec_bos_id: int = 4197
    spk_id: dict = field(default_factory=dict)              # voice name -> codec token id
    spk_is_dialect: dict = field(default_factory=dict)      # voice name -> False | dialect name
    codec_language_id: dict = field(default_factory=dict)   # language name -> codec token id
    im_start_token_id: int = 151644
    im_end_token_id: int = 151645
    assistant_token_id: int = 77091
    user_token_id: int = 872
    newline_token_id: int = 198
    tts_pad_token_id: int = 151671
    tts_bos_token_id: int = 151672
    tts_eos_token_id: int = 151673
    suppress_tail: int = 1024                       # trailing vocabulary slots never sampled (EOS excepted)
    repetition_penalty: float = 1.05
    max_frames: int = 4096

    @classmethod
    def tiny(cls) -> "Qwen3TTSConfig":
        return cls(text_vocab_size=512, text_hidden_size=48,
                   talker=DecoderConfig(vocab_size=96, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                                        num_key_value_heads=2, head_dim=16, intermediate_size=64, rope_theta=1e4),
                   code_predictor=CodePredictorConfig(hidden_size=24, num_hidden_layers=1, num_attention_heads=2,
                                                      num_key_value_heads=2, head_dim=12, intermediate_size=48,
                                                      vocab_size=64, num_code_groups=4, rope_theta=1e4),
                   tokenizer_decoder=TokenizerDecoderConfig(codebook_size=64, num_quantizers=4, hidden_size=32,
                                                            num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2,
                                                            intermediate_size=64, decoder_dim=32, upsample_rates=(4, 2),
                                                            upsampling_ratios=(2,), chunk_size=12, left_context=3,
                                                            codebook_dim=16, latent_dim=24, sliding_window=8),
                   speaker_encoder=SpeakerEncoderConfig(mel_dim=16, enc_dim=32, enc_channels=(8, 8, 8, 8, 24),
                                                        enc_attention_channels=4, enc_res2net_scale=2, enc_se_channels=4),
                   tts_model_type="base",
                   codec_eos_id=66, codec_think_id=70, codec_nothink_id=71, codec_think_bos_id=72, codec_think_eos_id=73,
                   codec_pad_id=64, codec_bos_id=65, spk_id={"vivian": 80, "uncle_fu": 81}, spk_is_dialect={"vivian": False,
                                                                                                           "uncle_fu": "beijing"},
                   codec_language_id={"english": 75, "chinese": 76, "beijing": 77},
                   im_start_token_id=506, im_end_token_id=507, assistant_token_id=510, user_token_id=509, newline_token_id=11,
                   tts_pad_token_id=503, tts_bos_token_id=504, tts_eos_token_id=505, suppress_tail=16, max_frames=64)

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen3TTSConfig":
        c = cls()
        tk = dict(d.get("talker_config") or {})
        if tk:
            if "head_dim" not in tk and "hidden_size" in tk and "num_attention_heads" in tk:
                tk["head_dim"] = tk["hidden_size"] // tk["num_attention_heads"]
            tk.setdefault("rope_theta", 10000.0)
            tk.pop("mrope_section", None)                # all three position axes are equal for speech rows
            tk["rope_scaling"] = None
            c.talker = DecoderConfig.from_dict(tk)
            c.talker.mrope_section = None
            for ours, theirs in (("codec_eos_id", "codec_eos_token_id"), ("codec_think_id",) * 2, ("codec_nothink_id",) * 2,
                                 ("codec_think_bos_id",) * 2, ("codec_think_eos_id",) * 2, ("codec_pad_id",) * 2,
                                 ("codec_bos_id",) * 2, ("text_hidden_size",) * 2, ("text_vocab_size",) * 2):
                if tk.get(theirs) is not None:
                    setattr(c, ours, tk[theirs])
            for k in ("spk_id", "spk_is_dialect", "codec_language_id"):
                if tk.get(k):
                    setattr(c, k, {str(a).lower(): b for a, b in tk[k].items()})
            cp = dict(tk.get("code_predictor_config") or {})
            cp.setdefault("num_code_groups", tk.get("num_code_groups", 32))
            cp.setdefault("rope_theta", 10000.0)
            keys = set(CodePredictorConfig.__dataclass_fields__)
            c.code_predictor = CodePredictorConfig(**{k: v for k, v in cp.items() if k in keys})
        if d.get("speaker_encoder_config") is not None and (d.get("tts_model_type") or "base") == "base":
            c.speaker_encoder = SpeakerEncoderConfig.from_dict(d["speaker_encoder_config"])
        for k in ("im_start_token_id", "im_end_token_id", "tts_pad_token_id", "tts_bos_token_id", "tts_eos_token_id",
                  "tts_model_type"):
            if d.get(k) is not None:
                setattr(c, k, d[k])
        tok_cfg = os.path.join(d.get("_model_dir") or "", "speech_tokenizer", "config.json")
        if d.get("_model_dir") and os.path.exists(tok_cfg):
            with open(tok_cfg) as f:
                c.tokenizer_decoder = TokenizerDecoderConfig.from_dict(json.load(f).get("decoder_config") or {})
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
        self.text_projection = ResizeMLP(cfg.text_hidden_size, cfg.text_hidden_size, Dt, dtype, device)
        self.talker = QwenDecoderModel(cfg.talker, dtype, device, with_lm_head=False)     # embed_tokens = codec embedding
        self.codec_head = FusedLinear(Dt, cfg.talker.vocab_size, bias=False, **kw)
        self.code_predictor = CodePredictor(cfg.code_predictor, Dt, dtype, device)
        self.speaker_encoder = Qwen3TTSSpeakerEncoder(cfg.speaker_encoder, device) if cfg.speaker_encoder else None
        self.decoder = Qwen3TTSTokenizerDecoder(cfg.tokenizer_decoder, dtype, device)     # speech tokenizer decoder
        self.tokenizer_encoder = None                   # speech tokenizer encoder, built when the checkpoint ships one
        self.tokenizer_25hz = None                      # the single-codebook 25 Hz tokenizer, when the checkpoint names it
        self.voices: dict[str, dict] = {}               # registered cloned voices
        self.text_tokenizer = None                      # set by the engine; turns instruction / transcript strings into ids
        self._session = None

    # ------------------------------------------------------------------ prompt pieces
    def _text(self, ids) -> torch.Tensor:
        tok = torch.as_tensor(list(ids), dtype=torch.long, device=self.text_embedding.device)
        if tok.numel() == 0:
            return torch.zeros(0, self.cfg.talker.hidden_size, dtype=self.text_embedding.dtype, device=tok.device)
        return self.text_projection(self.text_embedding[tok.clamp(0, self.cfg.text_vocab_size - 1)].contiguous())

    def _codec(self, ids) -> torch.Tensor:
        tok = torch.as_tensor(list(ids), dtype=torch.long, device=self.text_embedding.device)
        return self.talker.embed_tokens[tok]

    def wrap_text(self, ids) -> list[int]:
        """``<|im_start|>assistant\\n`` IDS ``<|im_end|>\\n<|im_start|>assistant\\n`` unless already wrapped."""
        c = self.cfg
        ids = [int(i) for i in ids]
        head = [c.im_start_token_id, c.assistant_token_id, c.newline_token_id]
        if ids[:3] == head:
            return ids
        return head + ids + [c.im_end_token_id, c.newline_token_id] + head

    def wrap_instruct(self, ids) -> list[int]:
        c = self.cfg
        ids = [int(i) for i in ids]
        if ids[:1] == [c.im_start_token_id]:
            return ids
        return [c.im_start_token_id, c.user_token_id, c.newline_token_id] + ids + [c.im_end_token_id, c.newline_token_id]

    def wrap_ref_text(self, ids) -> list[int]:
        c = self.cfg
        ids = [int(i) for i in ids]
        if ids[:1] == [c.im_start_token_id]:
            return ids
        return [c.im_start_token_id, c.assistant_token_id, c.newline_token_id] + ids + [c.im_end_token_id, c.newline_token_id]

    def _language_id(self, language, speaker):
        c = self.cfg
        lang = (language or "auto").lower() if isinstance(language, str) else language
        lid = None
        if isinstance(lang, int):
            lid = lang
        elif lang != "auto":
            if lang not in c.codec_language_id:
                raise ValueError(f"language {language!r} is not supported; known: {sorted(c.codec_language_id)}")
            lid = c.codec_language_id[lang]
        if lang in ("chinese", "auto") and isinstance(speaker, str) and speaker:
            dialect = c.spk_is_dialect.get(speaker.lower(), False)
            if dialect:
                lid = c.codec_language_id[dialect]
        return lid

    def _speaker_row(self, speaker, voice):
        """One row of talker width, or None (voice-design requests and x-vector-less cloning)."""
        if voice is not None:
            if voice.get("x_vector_only_mode") or voice.get("icl_mode"):
                return voice["ref_spk_embedding"].to(self.talker.embed_tokens).reshape(1, -1)
            return None
        if speaker is None or speaker == "":
            return None
        if isinstance(speaker, int):
            return self._codec([speaker])
        key = speaker.lower()
        if key not in self.cfg.spk_id:
            raise ValueError(f"speaker {speaker!r} is not supported; known: {sorted(self.cfg.spk_id)}")
        return self._codec([self.cfg.spk_id[key]])

    @torch.no_grad()
    def build_prompt(self, input_ids, instruct_ids=None, speaker=None, language="auto", voice=None, ref_ids=None,
                     non_streaming_mode=False):
        """Returns (prefill rows [L, D], trailing text rows [K, D], tts_pad row [1, D])."""
        c = self.cfg
        ids = self.wrap_text(input_ids)
        pad_bos_eos = self._text([c.tts_pad_token_id, c.tts_bos_token_id, c.tts_eos_token_id])
        tts_pad, tts_bos, tts_eos = pad_bos_eos[0:1], pad_bos_eos[1:2], pad_bos_eos[2:3]
        lid = self._language_id(language, speaker)
        prefix = [c.codec_nothink_id, c.codec_think_bos_id, c.codec_think_eos_id] if lid is None else \
            [c.codec_think_id, c.codec_think_bos_id, lid, c.codec_think_eos_id]
        rows = [self._codec(prefix)]
        spk = self._speaker_row(speaker, voice)
        if spk is not None:
            rows.append(spk)
        rows.append(self._codec([c.codec_pad_id, c.codec_bos_id]))
        codec_in = torch.cat(rows, 0)                                       # [n, D], last row = codec_bos
        n = codec_in.shape[0]
        parts = []
        if instruct_ids is not None and len(instruct_ids):
            parts.append(self._text(self.wrap_instruct(instruct_ids)))
        parts.append(self._text(ids[:3]))
        parts.append(torch.cat([tts_pad.expand(n - 2, -1), tts_bos], 0) + codec_in[:-1])
        icl = voice is not None and voice.get("ref_code") is not None and voice.get("icl_mode")
        if icl:
            ref = self.wrap_ref_text(ref_ids if ref_ids is not None else voice.get("ref_ids", []))
            text = torch.cat([self._text(ref[3:-2] + ids[3:-5]), tts_eos], 0)
            code = torch.as_tensor(voice["ref_code"], dtype=torch.long, device=tts_pad.device)      # [T, G]
            emb = self.talker.embed_tokens[code[:, 0]]
            for g in range(1, code.shape[1]):
                emb = emb + self.code_predictor.codec_embedding[g - 1][code[:, g]]
            codec = torch.cat([self._codec([c.codec_bos_id]), emb], 0)
            Lt, Lc = text.shape[0], codec.shape[0]
            if non_streaming_mode:
                parts.append(text + self._codec([c.codec_pad_id]))
                parts.append(codec + tts_pad)
                trailing = tts_pad
            elif Lt > Lc:
                parts.append(text[:Lc] + codec)
                trailing = text[Lc:]
            else:
                parts.append(torch.cat([text, tts_pad.expand(Lc - Lt, -1)], 0) + codec)
                trailing = tts_pad
        elif non_streaming_mode:
            body = torch.cat([self._text(ids[3:-5]), tts_eos], 0)
            parts.append(body + self._codec([c.codec_pad_id]))
            parts.append(tts_pad + codec_in[-1:])
            trailing = tts_pad
        else:
            parts.append(self._text(ids[3:4]) + codec_in[-1:])
            trailing = torch.cat([self._text(ids[4:-5]), tts_eos], 0)
        return torch.cat(parts, 0), trailing, tts_pad

    # ------------------------------------------------------------------ generation
    def _session_for(self, n_tokens: int) -> LocalDecodeSession:
        if self._session is None or self._session.max_len < n_tokens:
            self._session = LocalDecodeSession(self.talker, max(n_tokens, 256))
        self._session.reset()
        return self._session

    def _filter_logits(self, logits: torch.Tensor, history: list, step: int) -> torch.Tensor:
        c = self.cfg
        V = logits.shape[-1]
        logits = logits.clone()
        if history and c.repetition_penalty != 1.0:
            idx = torch.tensor(sorted(set(history)), dtype=torch.long, device=logits.device)
            v = logits[0, idx]
            logits[0, idx] = torch.where(v < 0, v * c.repetition_penalty, v / c.repetition_penalty)
        eos = logits[0, c.codec_eos_id].clone() if c.codec_eos_id < V else None
        logits[0, max(0, V - c.suppress_tail):] = float("-inf")
        if eos is not None:
            logits[0, c.codec_eos_id] = eos if step >= 2 else float("-inf")
        return logits

    @torch.no_grad()
    def synthesize(self, text_ids, instruct_ids=None, speaker=None, language="auto", voice=None, ref_ids=None,
                   non_streaming_mode=False, temperature: float = 0.9, top_k: int = 50, top_p: float = 1.0,
                   subtalker_temperature: float | None = None, seed: int = 0, max_frames: int | None = None):
        """Returns (codes [T, G] int64, waveform fp32).  ``voice``: a dict from ``create_voice_clone_prompt``
        or the name of a registered one."""
        cfg = self.cfg
        dev = self.text_embedding.device
        if isinstance(voice, str):
            voice = self.voices[voice]
        head, trailing, tts_pad = self.build_prompt(text_ids, instruct_ids, speaker, language, voice, ref_ids, non_streaming_mode)
        max_frames = min(max_frames or cfg.max_frames, cfg.max_frames)
        sess = self._session_for(head.shape[0] + max_frames + 1)
        hidden = sess.prefill(embeds=head.to(self.dtype_))[-1:]
        sub_t = temperature if subtalker_temperature is None else subtalker_temperature
        frames, history = [], []
        for k in range(max_frames):
            logits = self._filter_logits(self.codec_head(hidden).float(), history, k)
            if temperature <= 0:
                c0 = logits.argmax(-1)
            else:
                c0, _ = sample(logits, [RowParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed, step=k)])
                c0 = c0.long()
            if int(c0) == cfg.codec_eos_id:
                break
            history.append(int(c0))
            e0 = self.talker.embed_tokens[c0]
            rest, summed = self.code_predictor.generate(hidden.to(self.dtype_), e0, temperature=sub_t, seed=seed, step=k)
            frames.append(torch.cat([c0[:, None], rest], 1))
            nxt = e0 + summed + (trailing[k:k + 1] if k < trailing.shape[0] else tts_pad)
            hidden = sess.step(embed=nxt.to(self.dtype_))
        G = cfg.code_predictor.num_code_groups
        codes = torch.cat(frames, 0) if frames else torch.zeros(0, G, dtype=torch.long, device=dev)
        wav = self.decode_codes(codes, voice)
        return codes, wav

    @torch.no_grad()
    def decode_codes(self, codes: torch.Tensor, voice=None) -> torch.Tensor:
        """[T, G] frames -> waveform.  With in-context cloning the reference frames are decoded in front
        (their context shapes the first samples) and the matching share of the output is cut."""
        if codes.shape[0] == 0:
            return torch.zeros(0, device=codes.device)
        if self.tokenizer_25hz is not None:
            # one codebook; the voice carries the tokenizer's own x-vector and reference mel
            tk, v = self.tokenizer_25hz, voice or {}
            row = codes.reshape(codes.shape[0], -1)[:, 0][None]
            xv = v.get("tokenizer_xvector")
            mel = v.get("ref_mel")
            return tk.decode(row, None if xv is None else torch.as_tensor(xv)[None],
                             None if mel is None else torch.as_tensor(mel)[None])[0].float()
        ref = None
        if voice is not None and voice.get("icl_mode") and voice.get("ref_code") is not None:
            ref = torch.as_tensor(voice["ref_code"], dtype=torch.long, device=codes.device)
        full = codes if ref is None else torch.cat([ref, codes], 0)
        full = full[:, :self.decoder.c.num_quantizers]
        wav = self.decoder.chunked_decode(full.t()[None].contiguous())[0].float()
        if ref is not None:
            wav = wav[int(ref.shape[0] / full.shape[0] * wav.shape[0]):]
        return wav

    # ------------------------------------------------------------------ voice cloning
    @torch.no_grad()
    def create_voice_clone_prompt(self, ref_audio: torch.Tensor, sr: int, ref_ids=None, ref_code=None,
                                  x_vector_only_mode: bool = False, name: str | None = None) -> dict:
        """Reference clip -> {"ref_spk_embedding", "ref_code", "x_vector_only_mode", "icl_mode", "ref_ids"}.
        In-context mode needs the clip's codec frames ``ref_code`` [T, G] — given, or computed by the
        speech tokenizer's encoder when the checkpoint ships it — and its transcript ``ref_ids``; without
        frames only the x-vector is used."""
        if self.speaker_encoder is None:
            raise ValueError("this checkpoint has no speaker encoder: voice cloning needs the 'base' model type")
        ref_audio = torch.as_tensor(ref_audio, dtype=torch.float32)
        xvec = self.speaker_encoder.embed_audio(ref_audio, sr)
        if ref_code is None and not x_vector_only_mode and self.tokenizer_encoder is not None:
            from .speaker import resample_sinc
            clip = resample_sinc(ref_audio.reshape(1, -1), int(sr), self.tokenizer_encoder.cfg.sampling_rate)[0]
            ref_code = self.tokenizer_encoder.encode(clip)
        extra = {}
        if self.tokenizer_25hz is not None and self.tokenizer_25hz.encoder is not None:
            c25, xv25, mel25 = self.tokenizer_25hz.encode([ref_audio.reshape(-1)], int(sr))
            extra = {"tokenizer_xvector": xv25[0], "ref_mel": mel25[0]}
            if ref_code is None and not x_vector_only_mode:
                ref_code = c25[0][:, None]
        icl = (not x_vector_only_mode) and ref_code is not None
        if icl and not ref_ids:
            raise ValueError("in-context voice cloning needs the reference transcript (ref_ids)")
        v = {"ref_spk_embedding": xvec, "ref_code": torch.as_tensor(ref_code).long() if icl else None,
             "x_vector_only_mode": not icl, "icl_mode": icl, "ref_ids": list(ref_ids or []), **extra}
        if name:
            self.voices[name] = v
        return v

    # ------------------------------------------------------------------ stage interface
    def _ids_of(self, info: dict, ids_key: str, *text_keys):
        """Token ids of a request field given either as ids or as a string."""
        if info.get(ids_key) is not None:
            return list(info[ids_key])
        for k in text_keys:
            if isinstance(info.get(k), str) and info[k] and self.text_tokenizer is not None:
                return list(self.text_tokenizer.encode(info[k]))
        return None

    @property
    def voice_names(self) -> list[str]:
        return sorted(self.cfg.spk_id) + sorted(self.voices)

    def generate_for(self, req, start, n):
        info = dict(req.additional_information or {})
        sp = req.sampling_params
        instruct_ids = self._ids_of(info, "instruct_token_ids", "instruct", "instructions")
        ref_ids = self._ids_of(info, "ref_token_ids", "ref_text")
        task = str(info.get("task_type") or {"custom_voice": "CustomVoice", "voice_design": "VoiceDesign",
                                             "base": "Base"}.get(self.cfg.tts_model_type, "CustomVoice"))
        speaker = info.get("speaker", info.get("voice"))
        voice = None
        if task == "VoiceDesign":
            speaker = None
        elif task == "Base":
            voice, speaker = info.get("voice_clone_prompt") or (speaker if isinstance(speaker, str) and speaker in self.voices
                                                                else None), None
            if voice is None and info.get("ref_audio") is not None:
                audio, sr = load_reference_audio(info["ref_audio"], info.get("ref_sr"))
                voice = self.create_voice_clone_prompt(audio, sr, ref_ids=ref_ids, ref_code=info.get("ref_code"),
                                                       x_vector_only_mode=bool(info.get("x_vector_only_mode", False)))
            if voice is None:
                speaker = info.get("speaker")          # plain id / name on a checkpoint that has named voices
        elif speaker == "default":
            speaker = next(iter(self.cfg.spk_id), None)
        codes, wav = self.synthesize(
            req.prompt_token_ids[start:start + n], instruct_ids=instruct_ids, speaker=speaker,
            language=info.get("language") or "auto", voice=voice, ref_ids=ref_ids,
            non_streaming_mode=bool(info.get("non_streaming_mode", False)), temperature=sp.temperature,
            top_k=sp.top_k if sp.top_k and sp.top_k > 0 else 50, top_p=sp.top_p or 1.0, seed=sp.seed or 0,
            max_frames=sp.max_tokens)
        return {"audio": wav, "codes": codes, "sample_rate": self.cfg.tokenizer_decoder.sample_rate}

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, weights):
        groups = {"talker.model.": [], "talker.text_projection.": [], "talker.code_predictor.": [], "speaker_encoder.": [],
                  "speech_tokenizer.decoder.": []}
        loaded = set()
        for n, w in weights:
            if n == "talker.codec_head.weight":
                self.codec_head.weight.copy_(w.to(self.codec_head.weight.dtype))
                loaded.add(n)
            elif n == "talker.model.text_embedding.weight":
                self.text_embedding.copy_(w.to(self.text_embedding.dtype))
                loaded.add(n)
            else:
                for pre, lst in groups.items():
                    if n.startswith(pre):
                        lst.append((n[len(pre):], w))
                        break
        subs = {"talker.model.": self.talker, "talker.text_projection.": self.text_projection,
                "talker.code_predictor.": self.code_predictor, "speaker_encoder.": self.speaker_encoder,
                "speech_tokenizer.decoder.": self.decoder}
        for pre, lst in groups.items():
            if lst and subs[pre] is not None:
                loaded |= {pre + n for n in subs[pre].load_weights(lst)}
        return loaded

    @torch.no_grad()
    def load_auxiliary(self, model_dir: str) -> int:
        """The speech tokenizer sits in ``speech_tokenizer/`` beside the main checkpoint: its decoder is
        rebuilt from that folder's config when it differs from the default geometry, then loaded."""
        folder = os.path.join(model_dir, "speech_tokenizer")
        if not os.path.isdir(folder):
            return 0
        from ...diffusion.loader import _shard_files, safetensors_weights_iterator
        cfg_path = os.path.join(folder, "config.json")
        tok_cfg = {}
        if os.path.exists(cfg_path):
            with open(cfg_path) as f:
                tok_cfg = json.load(f)
            if tok_cfg.get("model_type") == "qwen3_tts_tokenizer_25hz":
                from .tokenizer_25hz import build_speech_tokenizer
                self.tokenizer_25hz = build_speech_tokenizer(tok_cfg, self.text_embedding.device,
                                                             with_encoder=self.speaker_encoder is not None)
                files = _shard_files(folder)
                return len(self.tokenizer_25hz.load_weights(safetensors_weights_iterator(files))) if files else 0
            dc = TokenizerDecoderConfig.from_dict(tok_cfg.get("decoder_config") or {})
            if dc != self.cfg.tokenizer_decoder:
                self.cfg.tokenizer_decoder = dc
                self.decoder = Qwen3TTSTokenizerDecoder(dc, self.dtype_, self.text_embedding.device)
        files = _shard_files(folder)
        if not files:
            return 0
        ws = list(safetensors_weights_iterator(files))
        n = len(self.decoder.load_weights((k[len("decoder."):], w) for k, w in ws if k.startswith("decoder.")))
        enc = [(k[len("encoder."):], w) for k, w in ws if k.startswith("encoder.")]
        if self.speaker_encoder is not None and tok_cfg.get("encoder_config") and len(enc) > 1:
            from .tokenizer_12hz_encoder import MimiEncoderConfig, Qwen3TTSTokenizerEncoder
            self.tokenizer_encoder = Qwen3TTSTokenizerEncoder(MimiEncoderConfig.from_dict(tok_cfg["encoder_config"]),
                                                              int(tok_cfg.get("encoder_valid_num_quantizers", 16)),
                                                              self.text_embedding.device)
            n += len(self.tokenizer_encoder.load_weights(enc))
        return n


def load_reference_audio(ref, sr=None):
    """A reference clip given as samples (with ``sr``), a path to a 16-bit / float WAV file, or base64
    of such a file (optionally as a ``data:`` URL) -> (mono float32 tensor, sample rate)."""
    if not isinstance(ref, (str, bytes)):
        return torch.as_tensor(ref, dtype=torch.float32).reshape(-1), int(sr or 24000)
    import base64
    import io
    import wave

    import numpy as np
    if isinstance(ref, str) and os.path.exists(ref):
        with open(ref, "rb") as f:
            raw = f.read()
    else:
        text = ref.decode() if isinstance(ref, bytes) else ref
        raw = base64.b64decode(text.split(",", 1)[1] if text.startswith("data:") else text)
    with wave.open(io.BytesIO(raw)) as w:
        ch, width, rate, frames = w.getnchannels(), w.getsampwidth(), w.getframerate(), w.readframes(w.getnframes())
    if width == 2:
        x = np.frombuffer(frames, dtype="<i2").astype(np.float32) / 32768.0
    elif width == 4:
        x = np.frombuffer(frames, dtype="<i4").astype(np.float32) / 2147483648.0
    elif width == 1:
        x = (np.frombuffer(frames, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    else:
        raise ValueError(f"unsupported WAV sample width {width}")
    x = x.reshape(-1, ch).mean(1) if ch > 1 else x
    return torch.from_numpy(np.ascontiguousarray(x)), int(rate)


def build_qwen3_tts_stage(model_stage, hf_config: dict, dtype, device, **kw):
    if kw.get("tiny") or (hf_config or {}).get("tiny"):
        cfg = Qwen3TTSConfig.tiny()
    elif hf_config:
        cfg = Qwen3TTSConfig.from_hf(hf_config)
    else:
        cfg = Qwen3TTSConfig()
    for k, v in kw.items():                              # stage-config overrides of single fields
        if k in Qwen3TTSConfig.__dataclass_fields__ and not isinstance(getattr(cfg, k), (DecoderConfig, CodePredictorConfig,
                                                                                          TokenizerDecoderConfig)):
            setattr(cfg, k, v)
    return Qwen3TTSModel(cfg, dtype, device)
