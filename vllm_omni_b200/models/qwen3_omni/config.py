"""Configuration of the Qwen3-Omni-MoE three-stage model (thinker / talker / code2wav).
Defaults are the 30B-A3B geometry; ``tiny()`` is the CPU test geometry.  ``from_hf`` reads the
``thinker_config`` / ``talker_config`` / ``code2wav_config`` sub-dicts of an HF config.json
(the reference selects them with ``hf_config_name``, vllm_omni/config/model.py)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..qwen_decoder import DecoderConfig


@dataclass
class AudioEncoderConfig:
    num_mel_bins: int = 128
    d_model: int = 1280
    encoder_layers: int = 32
    encoder_attention_heads: int = 20
    encoder_ffn_dim: int = 5120
    downsample_hidden_size: int = 480
    output_dim: int = 2048
    n_window: int = 50                 # a chunk of the conv stem is 2 * n_window mel frames
    n_window_infer: int = 400          # mel frames covered by one attention window
    activation_function: str = "gelu"


@dataclass
class VisionEncoderConfig:
    depth: int = 27
    hidden_size: int = 1152
    num_heads: int = 16
    intermediate_size: int = 4304
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 2048
    num_position_embeddings: int = 2304            # learned G x G position grid, G = 48
    deepstack_visual_indexes: tuple = (8, 16, 24)  # blocks whose output also feeds decoder layers 0, 1, 2
    hidden_act: str = "gelu_pytorch_tanh"


@dataclass
class CodePredictorConfig:
    hidden_size: int = 1024
    num_hidden_layers: int = 5
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    vocab_size: int = 2048
    num_code_groups: int = 16
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6


@dataclass
class Code2WavConfig:
    codebook_size: int = 2048
    num_quantizers: int = 16
    hidden_size: int = 1024
    num_hidden_layers: int = 8
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    intermediate_size: int = 3072
    sliding_window: int = 72
    head_dim: int | None = None        # None: hidden_size / num_attention_heads
    attention_bias: bool = False
    layer_scale_initial_scale: float = 0.01
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    decoder_dim: int = 1536
    upsample_rates: tuple = (8, 5, 4, 3)
    upsampling_ratios: tuple = (2, 2)
    sample_rate: int = 24000
    chunk_size: int = 300
    left_context: int = 25

    @property
    def total_upsample(self) -> int:
        n = 1
        for r in tuple(self.upsample_rates) + tuple(self.upsampling_ratios):
            n *= r
        return n


@dataclass
class Qwen3OmniConfig:
    thinker: DecoderConfig = field(default_factory=lambda: DecoderConfig(
        vocab_size=151936, hidden_size=2048, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
        head_dim=128, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, rope_theta=1e6,
        mrope_section=(24, 20, 20), mrope_interleaved=True))
    talker: DecoderConfig = field(default_factory=lambda: DecoderConfig(
        vocab_size=3072, hidden_size=1024, num_hidden_layers=20, num_attention_heads=16, num_key_value_heads=2,
        head_dim=128, intermediate_size=2048, num_experts=128, num_experts_per_tok=6, moe_intermediate_size=384,
        shared_expert_intermediate_size=768, rope_theta=1e6,
        mrope_section=(24, 20, 20), mrope_interleaved=True))
    audio: AudioEncoderConfig = field(default_factory=AudioEncoderConfig)
    vision: VisionEncoderConfig = field(default_factory=VisionEncoderConfig)
    code_predictor: CodePredictorConfig = field(default_factory=CodePredictorConfig)
    code2wav: Code2WavConfig = field(default_factory=Code2WavConfig)
    accept_hidden_layer: int = 24
    audio_token_id: int = 151675
    image_token_id: int = 151655
    video_token_id: int = 151656
    tts_bos_token_id: int = 151672
    tts_eos_token_id: int = 151673
    tts_pad_token_id: int = 151671
    im_start_token_id: int = 151644
    im_end_token_id: int = 151645
    codec_bos_id: int = 2149
    codec_eos_id: int = 2150
    codec_pad_id: int = 2148
    codec_nothink_id: int = 2155
    codec_think_bos_id: int = 2156
    codec_think_eos_id: int = 2157
    system_token_id: int = 8948         # role tokens that follow <|im_start|>
    user_token_id: int = 872
    assistant_token_id: int = 77091
    audio_start_token_id: int = 151669  # stands in for the speaker token when the checkpoint lists no voices
    speaker_ids: dict = field(default_factory=dict)      # voice name (lower case) -> codec token id

    @classmethod
    def tiny(cls) -> "Qwen3OmniConfig":
        th = DecoderConfig(vocab_size=512, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, num_experts=4, num_experts_per_tok=2,
                           moe_intermediate_size=32, mrope_section=(4, 2, 2), mrope_interleaved=True)
        tk = DecoderConfig(vocab_size=96, hidden_size=48, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, intermediate_size=64, num_experts=4,
                           num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=24,
                           mrope_section=(4, 2, 2), mrope_interleaved=True)
        return cls(thinker=th, talker=tk,
                   audio=AudioEncoderConfig(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=2,
                                            encoder_ffn_dim=64, downsample_hidden_size=8, output_dim=64, n_window=8,
                                            n_window_infer=32),
                   vision=VisionEncoderConfig(depth=1, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4,
                                              temporal_patch_size=1, spatial_merge_size=2, out_hidden_size=64,
                                              num_position_embeddings=16, deepstack_visual_indexes=(0,)),
                   code_predictor=CodePredictorConfig(hidden_size=48, num_hidden_layers=1, num_attention_heads=4,
                                                      num_key_value_heads=2, head_dim=16, intermediate_size=64,
                                                      vocab_size=64, num_code_groups=4),
                   code2wav=Code2WavConfig(codebook_size=64, num_quantizers=4, hidden_size=32, num_hidden_layers=1,
                                           num_attention_heads=2, num_key_value_heads=2, intermediate_size=64,
                                           decoder_dim=32, upsample_rates=(4, 2), upsampling_ratios=(2,),
                                           chunk_size=12, left_context=3),
                   accept_hidden_layer=2, audio_token_id=500, image_token_id=501, video_token_id=502,
                   tts_bos_token_id=503, tts_eos_token_id=504, tts_pad_token_id=505, im_start_token_id=506,
                   im_end_token_id=507, codec_bos_id=65, codec_eos_id=66, codec_pad_id=64, codec_nothink_id=67,
                   codec_think_bos_id=68, codec_think_eos_id=69, system_token_id=508, user_token_id=509,
                   assistant_token_id=510, audio_start_token_id=71, speaker_ids={"ethan": 70, "chelsie": 72})

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen3OmniConfig":
        c = cls()
        th = d.get("thinker_config", {})
        if th.get("text_config"):
            c.thinker = DecoderConfig.from_dict(th["text_config"])
        tk = d.get("talker_config", {})
        if tk.get("text_config"):
            c.talker = DecoderConfig.from_dict(tk["text_config"])
        cp = tk.get("code_predictor_config")
        if cp:
            keys = set(CodePredictorConfig.__dataclass_fields__)
            cp = dict(cp)
            if cp.get("rope_theta") is None:
                cp["rope_theta"] = float((cp.get("rope_parameters") or {}).get("rope_theta", 1e6))
            c.code_predictor = CodePredictorConfig(**{k: v for k, v in cp.items() if k in keys})
        cw = d.get("code2wav_config")
        if cw:
            keys = set(Code2WavConfig.__dataclass_fields__)
            cw = dict(cw)
            if cw.get("rope_theta") is None:
                cw["rope_theta"] = float((cw.get("rope_parameters") or {}).get("rope_theta", 10000.0))
            c.code2wav = Code2WavConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in cw.items() if k in keys})
        if isinstance(tk.get("speaker_id"), dict):
            c.speaker_ids = {str(k).lower(): int(v) for k, v in tk["speaker_id"].items()}
        for src, dst in (("codec_think_bos_id", "codec_think_bos_id"), ("codec_think_eos_id", "codec_think_eos_id"),
                         ("audio_start_token_id", "audio_start_token_id"), ("codec_eos_token_id", "codec_eos_id"), ("codec_bos_id", "codec_bos_id"),
                         ("codec_pad_id", "codec_pad_id"), ("codec_nothink_id", "codec_nothink_id")):
            if src in tk:
                setattr(c, dst, tk[src])
        for key, klass, attr in (("audio_config", AudioEncoderConfig, "audio"), ("vision_config", VisionEncoderConfig, "vision")):
            sub = th.get(key)
            if sub:
                keys = set(klass.__dataclass_fields__)
                setattr(c, attr, klass(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in sub.items() if k in keys}))
        for k in ("audio_token_id", "image_token_id", "video_token_id"):
            if k in th:
                setattr(c, k, th[k])
        for k in ("tts_bos_token_id", "tts_eos_token_id", "tts_pad_token_id", "im_start_token_id", "im_end_token_id",
                  "system_token_id", "user_token_id", "assistant_token_id"):
            if k in d:
                setattr(c, k, d[k])
        if "accept_hidden_layer" in tk:
            c.accept_hidden_layer = tk["accept_hidden_layer"]
        return c
