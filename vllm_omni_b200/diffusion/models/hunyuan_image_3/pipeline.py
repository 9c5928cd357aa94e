"""HunyuanImage-3 pipeline (vllm_omni/diffusion/models/hunyuan_image_3/): a multimodal LLM with
mixture-of-experts MLPs that denoises image tokens.  Image latents are patch-embedded into the
LLM width, run through the MoE decoder together with the text tokens (full attention over image
tokens, the grouped tcgen05 MoE kernel for the experts) and projected back to velocities; the
timestep enters as an extra token embedding.  TP shards heads and experts (MoE partial sums are
added across ranks)."""
from __future__ import annotations

import torch
from torch import nn

from ....models.qwen_decoder import DecoderConfig, ModelBatch, PrefillSeg, QwenDecoderModel
from ....ops import fused
from ...data import DiffusionOutput, OmniDiffusionConfig
from ...layers.linear import FusedLinear
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..qwen_image.pipeline import HashTextEncoder, pack_latents, unpack_latents
from ..qwen_image.transformer import TimestepEmbedder
from ..vae.autoencoder_kl_qwenimage import AutoencoderKLQwenImage2d, QwenImageVAEConfig


class HunyuanImage3Pipeline(nn.Module):
    def __init__(self, od_config: OmniDiffusionConfig | None = None, decoder_config: DecoderConfig | None = None,
                 vae_config=None, device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        p = self.od_config.tf_model_config.to_dict()
        dc = decoder_config or DecoderConfig.from_dict({**dict(vocab_size=1024, hidden_size=4096, num_hidden_layers=32,
                                                               num_attention_heads=32, num_key_value_heads=8,
                                                               head_dim=128, num_experts=64, num_experts_per_tok=8,
                                                               moe_intermediate_size=3072), **p})
        self.llm = QwenDecoderModel(dc, dtype, self.device_, with_lm_head=False)
        D = dc.hidden_size
        self.patch_in = FusedLinear(64, D, dtype=dtype, device=self.device_)
        self.patch_out = FusedLinear(D, 64, dtype=dtype, device=self.device_)
        self.time_embed = TimestepEmbedder(D, dtype, self.device_)
        self.text_encoder = HashTextEncoder(D, max_len=128)
        self.vae = AutoencoderKLQwenImage2d(vae_config or QwenImageVAEConfig()).to(device=self.device_, dtype=dtype)
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=3.0)
        self.transformer = self.llm            # what caches / LoRA / quantisation attach to
        self.vae_decode = None

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        H, W = sp.height or 1024, sp.width or 1024
        h, w = 2 * (H // 16), 2 * (W // 16)
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        outs = []
        ts = None
        for text in texts:                      # one sequence per prompt (the LLM batch is flat)
            pe, mask = self.text_encoder([text], self.device_, self.od_config.dtype)
            n_txt = int(mask.sum())
            z = torch.randn(1, 16, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
            lat = pack_latents(z.to(self.device_, torch.float32))
            ts = self.scheduler.set_timesteps(sp.num_inference_steps, device=self.device_)
            S = lat.shape[1]
            T = n_txt + 1 + S
            pos = torch.arange(T, device=self.device_)
            for i in range(len(ts)):
                sig = float(self.scheduler.sigmas[i])
                temb = self.time_embed(torch.tensor([sig], device=self.device_), self.od_config.dtype)
                x = torch.cat([pe[0, :n_txt], temb, self.patch_in(lat[0].to(self.od_config.dtype))], dim=0)
                batch = ModelBatch(torch.zeros(T, dtype=torch.long, device=self.device_), pos,
                                   torch.full((T,), -1, dtype=torch.int32, device=self.device_),
                                   [PrefillSeg(0, T, 0, None)], input_embeds=x, embeds_mask=None)
                hdn, _ = self.llm(batch, None)
                v = self.patch_out(hdn[n_txt + 1:].contiguous())[None]
                fused.cfg_euler_step_(v.contiguous(), None, lat, 1.0, self.scheduler.dt(i), False, None)
            outs.append(lat)
        lat = torch.cat(outs, 0)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(unpack_latents(lat, h, w)))

    def load_weights(self, weights) -> set:
        return self.llm.load_weights(weights)
