"""Stable-Audio text-to-audio pipeline (vllm_omni/diffusion/models/stable_audio/): a 1-D
diffusion transformer with cross attention to the text states over a latent sequence, followed
by a convolutional decoder (transposed-conv up-sampling with Snake activations) to stereo audio.
The engine reports the result as ``final_output_type='audio'``."""
from __future__ import annotations

import torch
from torch import nn

from ....models.qwen3_omni.code2wav import DecoderBlock as UpBlock
from ...data import DiffusionOutput, OmniDiffusionConfig
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..qwen_image.pipeline import HashTextEncoder
from ..wan.transformer import WanTransformer3DModel, WanTransformerConfig


class AudioDecoder(nn.Module):
    def __init__(self, latent_ch=64, dim=128, rates=(8, 8, 4, 4, 2), dtype=torch.float32, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.conv_in = nn.Conv1d(latent_ch, dim, 7, padding=3, **kw)
        ups, c = [], dim
        for r in rates:
            ups.append(UpBlock(c, max(c // 2, 8), r, dtype, device))
            c = max(c // 2, 8)
        self.ups = nn.ModuleList(ups)
        self.conv_out = nn.Conv1d(c, 2, 7, padding=3, **kw)
        self.total = 1
        for r in rates:
            self.total *= r

    def forward(self, z):
        x = self.conv_in(z)
        for u in self.ups:
            x = u(x)
        return torch.tanh(self.conv_out(x).float())


class StableAudioPipeline(nn.Module):
    sample_rate = 44100

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        p = self.od_config.tf_model_config.to_dict()
        tc = transformer_config or WanTransformerConfig.from_dict({**dict(patch_size=(1, 1, 1), num_attention_heads=24,
                                                                          attention_head_dim=64, in_channels=64,
                                                                          out_channels=64, text_dim=768, ffn_dim=6144,
                                                                          num_layers=24), **p})
        tc.patch_size = (1, 1, 1)
        self.transformer = WanTransformer3DModel(tc, dtype=dtype, device=self.device_)
        rates = tuple(p.get("decoder_rates", (8, 8, 4, 4, 2)))
        self.decoder = AudioDecoder(tc.out_channels, int(p.get("decoder_dim", 128)), rates,
                                    torch.float32 if self.device_.type == "cpu" else dtype, self.device_)
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=1.0)
        self.text_encoder = HashTextEncoder(tc.text_dim, max_len=128)

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        B = len(texts)
        seconds = float(sp.extra_args.get("audio_seconds", 1.0)) if sp.extra_args else 1.0
        T = max(4, int(seconds * self.sample_rate / self.decoder.total))
        C = self.transformer.cfg.in_channels
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        lat = torch.randn(B, C, T, 1, 1, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = lat.to(self.device_, torch.float32)
        pe, _ = self.text_encoder(texts, self.device_, self.od_config.dtype)
        ts = self.scheduler.set_timesteps(sp.num_inference_steps, device=self.device_)
        for i, t in enumerate(ts):
            v = self.transformer(lat.to(self.od_config.dtype), t.expand(B), pe).float()
            lat = lat + self.scheduler.dt(i) * v
        wav = self.decoder(lat[:, :, :, 0, 0].to(self.decoder.conv_in.weight.dtype))
        return DiffusionOutput(output=[w for w in wav])
