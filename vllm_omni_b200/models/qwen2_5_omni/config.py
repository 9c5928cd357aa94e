"""Configuration of the three Qwen2.5-Omni stages (thinker, talker, token2wav); defaults are
the 7B model's shapes (vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni.py:58-140)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..qwen2_5_vl_vision import Qwen25VisionConfig
from .audio import Qwen25AudioConfig
from ..qwen_decoder import DecoderConfig


@dataclass
class DiTConfig:
    """Flow-matching transformer: codec tokens -> mel spectrogram."""
    hidden_size: int = 1024
    num_hidden_layers: int = 22
    num_attention_heads: int = 16
    head_dim: int = 64
    ff_mult: int = 2
    mel_dim: int = 80
    num_embeds: int = 8193              # codec vocabulary + 1 "dropped" id
    emb_dim: int = 512
    repeats: int = 2                    # mel frames per codec token
    block_size: int = 24                # attention is restricted to neighbouring blocks of this many frames
    look_ahead_layers: tuple = (10,)    # layers that also see the next block
    look_backward_layers: tuple = (0, 20)   # layers that also see the previous block
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    enc_emb_dim: int = 192              # speaker x-vector width
    enc_dim: int = 128                  # output of the reference-mel speaker encoder
    enc_channels: tuple = (256, 256, 256, 256, 768)
    enc_kernel_sizes: tuple = (5, 3, 3, 3, 1)
    enc_dilations: tuple = (1, 2, 3, 4, 1)
    enc_attention_channels: int = 64
    enc_res2net_scale: int = 2
    enc_se_channels: int = 64
    num_steps: int = 10
    guidance_scale: float = 0.5
    sway_coefficient: float = -1.0

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        if d.get("rope_theta") is None:
            d["rope_theta"] = float((d.get("rope_parameters") or {}).get("rope_theta", 10000.0))
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


@dataclass
class BigVGANConfig:
    mel_dim: int = 80
    upsample_initial_channel: int = 1536
    upsample_rates: tuple = (5, 3, 2, 2, 2, 2)
    upsample_kernel_sizes: tuple = (11, 7, 4, 4, 4, 4)
    resblock_kernel_sizes: tuple = (3, 7, 11)
    resblock_dilation_sizes: tuple = ((1, 3, 5), (1, 3, 5), (1, 3, 5))
    sample_rate: int = 24000

    @property
    def total_upsample(self) -> int:
        n = 1
        for r in self.upsample_rates:
            n *= r
        return n

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        tup = lambda v: tuple(tup(x) for x in v) if isinstance(v, (list, tuple)) else v
        return cls(**{k: tup(v) for k, v in d.items() if k in keys})


@dataclass
class Qwen25OmniConfig:
    thinker: DecoderConfig = field(default_factory=lambda: DecoderConfig(
        vocab_size=152064, hidden_size=3584, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
        head_dim=128, intermediate_size=18944, qk_norm=False, attention_bias=True, rope_theta=1e6,
        mrope_section=(16, 24, 24)))
    talker: DecoderConfig = field(default_factory=lambda: DecoderConfig(
        vocab_size=8448, hidden_size=896, num_hidden_layers=24, num_attention_heads=12, num_key_value_heads=4,
        head_dim=128, intermediate_size=18944, qk_norm=False, attention_bias=True, rope_theta=1e6,
        mrope_section=(16, 24, 24)))
    audio: Qwen25AudioConfig = field(default_factory=Qwen25AudioConfig)
    talker_embedding_size: int = 3584     # width of the talker's codec embedding table (= thinker width)
    vision: Qwen25VisionConfig = field(default_factory=Qwen25VisionConfig)
    dit: DiTConfig = field(default_factory=DiTConfig)
    bigvgan: BigVGANConfig = field(default_factory=BigVGANConfig)
    audio_token_id: int = 151646
    image_token_id: int = 151655
    video_token_id: int = 151656
    im_end_token_id: int = 151645
    codec_pad_id: int = 8292
    codec_bos_id: int = 8293
    codec_eos_id: int = 8294
    tts_text_bos_id: int = 151860       # thinker-vocabulary tokens whose embeddings frame the spoken text
    tts_text_eos_id: int = 151861
    tts_text_pad_id: int = 151859

    @classmethod
    def tiny(cls) -> "Qwen25OmniConfig":
        th = DecoderConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, intermediate_size=96, qk_norm=False,
                           attention_bias=True, mrope_section=(4, 2, 2))
        tk = DecoderConfig(vocab_size=96, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                           num_key_value_heads=2, head_dim=16, intermediate_size=64, qk_norm=False,
                           attention_bias=True, mrope_section=(4, 2, 2))
        return cls(thinker=th, talker=tk,
                   audio=Qwen25AudioConfig(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=2,
                                           encoder_ffn_dim=64, output_dim=64, n_window=8),
                   talker_embedding_size=64,
                   vision=Qwen25VisionConfig(depth=2, hidden_size=32, num_heads=2, intermediate_size=48, patch_size=4,
                                             temporal_patch_size=1, spatial_merge_size=2, out_hidden_size=64,
                                             window_size=16, fullatt_block_indexes=(1,)),
                   dit=DiTConfig(hidden_size=32, num_hidden_layers=3, num_attention_heads=2, head_dim=16, mel_dim=8,
                                 num_embeds=97, emb_dim=16, block_size=4, look_ahead_layers=(1,), look_backward_layers=(0, 2),
                                 enc_emb_dim=8, enc_dim=8, enc_channels=(8, 8, 8, 8, 24), enc_kernel_sizes=(5, 3, 3, 3, 1),
                                 enc_dilations=(1, 2, 3, 4, 1), enc_attention_channels=4, enc_res2net_scale=2,
                                 enc_se_channels=4, num_steps=3),
                   bigvgan=BigVGANConfig(mel_dim=8, upsample_initial_channel=16, upsample_rates=(2, 2),
                                         upsample_kernel_sizes=(4, 4), resblock_kernel_sizes=(3,),
                                         resblock_dilation_sizes=((1, 3),)),
                   audio_token_id=500, image_token_id=501, video_token_id=502, im_end_token_id=507,
                   codec_pad_id=92, codec_bos_id=93, codec_eos_id=94, tts_text_bos_id=503, tts_text_eos_id=504,
                   tts_text_pad_id=505)

    @classmethod
    def from_hf(cls, d: dict) -> "Qwen25OmniConfig":
        c = cls()
        th = d.get("thinker_config", {})
        if th.get("text_config"):
            # the thinker checkpoint always carries its own ``lm_head.weight``, whatever the tie flag says
            c.thinker = DecoderConfig.from_dict({**th["text_config"], "qk_norm": False, "attention_bias": True,
                                                 "tie_word_embeddings": False})
        if th.get("audio_config"):
            c.audio = Qwen25AudioConfig.from_dict(th["audio_config"])
        if th.get("vision_config"):
            c.vision = Qwen25VisionConfig.from_dict(th["vision_config"])
        tk = d.get("talker_config", {})
        if tk:
            c.talker = DecoderConfig.from_dict({**tk, "qk_norm": False, "attention_bias": True})
            c.talker_embedding_size = int(tk.get("embedding_size", c.thinker.hidden_size))
        tw = d.get("token2wav_config", {})
        if tw.get("dit_config"):
            c.dit = DiTConfig.from_dict(tw["dit_config"])
        if tw.get("bigvgan_config"):
            c.bigvgan = BigVGANConfig.from_dict(tw["bigvgan_config"])
        for k, src in (("audio_token_id", "audio_token_index"), ("image_token_id", "image_token_index"),
                       ("video_token_id", "video_token_index")):
            if src in th:
                setattr(c, k, th[src])
        for k, src in (("codec_pad_id", "tts_codec_pad_token_id"), ("codec_bos_id", "tts_codec_start_token_id"),
                       ("codec_eos_id", "tts_codec_end_token_id"), ("tts_text_bos_id", "tts_text_start_token_id"),
                       ("tts_text_eos_id", "tts_text_end_token_id"), ("tts_text_pad_id", "tts_text_pad_token_id")):
            if src in tk:
                setattr(c, k, tk[src])
        return c
