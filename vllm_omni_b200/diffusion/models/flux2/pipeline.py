"""FLUX.2-klein text-to-image and reference-image editing pipeline
(vllm_omni/diffusion/models/flux2_klein/pipeline_flux2_klein.py:164-993).

Latents: 32 VAE channels in 2x2 pixel-shuffled form (128 channels at half resolution), one token per
position, normalised by the running statistics of the autoencoder's batch norm (``vae.bn``); the
decode path undoes the normalisation, un-shuffles and runs the KL decoder without a scaling factor.
Tokens carry 4-axis position ids (t, y, x, l): the noise grid has t = 0, reference image i has
t = 10 (i + 1), text token l has (0, 0, 0, l).  Reference latents are appended to the image rows of
every step's input and their rows of the output are dropped.  The schedule is the flow-match Euler
schedule with an empirically fitted dynamic shift ``mu(sequence length, steps)``; guidance is plain
classifier-free guidance against the empty prompt when the scale exceeds 1 (the distilled klein
checkpoints run without it).
"""
from __future__ import annotations

import os

import numpy as np
import torch
from torch import nn

from ....ops import fused
from ...data import DiffusionOutput, OmniDiffusionConfig
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..qwen_image.pipeline import HashTextEncoder
from ..vae import build_vae
from .transformer import Flux2Transformer2DModel, Flux2TransformerConfig, image_ids, text_ids

KLEIN_SCHEDULER = dict(num_train_timesteps=1000, shift=3.0, use_dynamic_shifting=True, time_shift_type="exponential")


def compute_empirical_mu(image_seq_len: int, num_steps: int) -> float:
    """Dynamic shift fitted on (sequence length, step count): linear in the length at 10 and at 200 steps,
    interpolated linearly in the step count; long sequences use the 200-step line alone."""
    a1, b1 = 8.73809524e-05, 1.89833333
    a2, b2 = 0.00016927, 0.45666666
    if image_seq_len > 4300:
        return float(a2 * image_seq_len + b2)
    m200, m10 = a2 * image_seq_len + b2, a1 * image_seq_len + b1
    a = (m200 - m10) / 190.0
    return float(a * num_steps + (m200 - 200.0 * a))


def patchify(z: torch.Tensor) -> torch.Tensor:
    """[B, C, H, W] -> [B, 4C, H/2, W/2], channel order (c, dy, dx)."""
    B, C, H, W = z.shape
    return z.view(B, C, H // 2, 2, W // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(B, C * 4, H // 2, W // 2)


def unpatchify(z: torch.Tensor) -> torch.Tensor:
    B, C4, H, W = z.shape
    return z.reshape(B, C4 // 4, 2, 2, H, W).permute(0, 1, 4, 2, 5, 3).reshape(B, C4 // 4, H * 2, W * 2)


class Flux2KleinPipeline(nn.Module):
    vae_scale_factor = 8
    default_guidance = 1.0
    max_text_len = 512
    max_condition_images = 4

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None, device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        tcfg = transformer_config or Flux2TransformerConfig.from_dict(self.od_config.tf_model_config.to_dict())
        self.transformer = Flux2Transformer2DModel(tcfg, dtype=dtype, device=self.device_)
        vc = dict(vae_config or self.od_config.vae_config or {})
        vc["_class_name"] = "AutoencoderKL"
        vc.setdefault("latent_channels", tcfg.in_channels // 4)
        vc.setdefault("scaling_factor", 1.0)
        vc.setdefault("shift_factor", None)
        vc.setdefault("use_quant_conv", True)
        vc.setdefault("use_post_quant_conv", True)
        self.bn_eps = float(vc.get("batch_norm_eps", 1e-4))
        self.vae = build_vae(vc, "kl", with_encoder=True).to(device=self.device_, dtype=dtype)
        self.vae.use_tiling = self.od_config.vae_use_tiling
        self.register_buffer("bn_mean", torch.zeros(tcfg.in_channels, device=self.device_))
        self.register_buffer("bn_var", torch.ones(tcfg.in_channels, device=self.device_))
        self.scheduler = FlowMatchEulerDiscreteScheduler(**KLEIN_SCHEDULER)
        self.text_encoder = HashTextEncoder(tcfg.joint_attention_dim, max_len=self.max_text_len)
        self.vae_decode = None
        self.cfg_exchange = None        # set by CFG-parallel: rank 0 runs the prompt branch, rank 1 the empty-prompt branch

    def attach_text_encoder(self, model_path: str) -> bool:
        if not (os.path.isfile(os.path.join(model_path, "text_encoder", "config.json")) and
                os.path.isdir(os.path.join(model_path, "tokenizer"))):
            return False
        from .text_encoder import Flux2PromptEncoder
        self.text_encoder = Flux2PromptEncoder.from_pretrained(model_path, self.od_config.dtype, self.device_,
                                                               max_length=self.max_text_len)
        return True

    def load_weights(self, weights) -> set:
        groups = {"transformer": [], "vae": [], "text_encoder": []}
        loaded = set()
        for n, w in weights:
            comp, _, rest = n.partition(".")
            if n == "vae.bn.running_mean":
                self.bn_mean.copy_(w.to(self.bn_mean))
                loaded.add(n)
            elif n == "vae.bn.running_var":
                self.bn_var.copy_(w.to(self.bn_var))
                loaded.add(n)
            elif comp in groups:
                groups[comp].append((rest, w))
        loaded |= {"transformer." + n for n in self.transformer.load_weights(groups["transformer"])}
        if groups["vae"]:
            loaded |= {"vae." + n for n in self.vae.load_weights(groups["vae"])}
        if groups["text_encoder"] and hasattr(self.text_encoder, "load_weights"):
            loaded |= {"text_encoder." + n for n in self.text_encoder.load_weights(groups["text_encoder"])}
        return loaded

    # ------------------------------------------------------------------ latents
    def _bn(self):
        return self.bn_mean.view(1, -1, 1, 1).float(), torch.sqrt(self.bn_var.view(1, -1, 1, 1).float() + self.bn_eps)

    def _reference_latents(self, prompt):
        """Reference images -> (tokens [1, N, C], ids [N, 4]) or (None, None)."""
        mm = (prompt.get("multi_modal_data") or {}) if isinstance(prompt, dict) else {}
        imgs = (mm.get("image_tensor") or [])[: self.max_condition_images]
        if not imgs:
            return None, None
        mean, std = self._bn()
        toks, ids = [], []
        for i, im in enumerate(imgs):
            x = im.to(self.device_, torch.float32)[None]
            H, W = x.shape[-2:]
            if H * W > 1024 * 1024:                          # cap the reference at one megapixel
                s = (1024 * 1024 / (H * W)) ** 0.5
                H, W = int(H * s), int(W * s)
            H, W = (H // 16) * 16, (W // 16) * 16
            x = torch.nn.functional.interpolate(x, size=(H, W), mode="bilinear", align_corners=False)
            z = patchify(self.vae.encode(x.to(self.od_config.dtype)).float())
            z = (z - mean) / std
            toks.append(z.flatten(2).transpose(1, 2))
            ids.append(image_ids(z.shape[2], z.shape[3], t=10 * (i + 1)))
        return torch.cat(toks, dim=1), torch.cat(ids, dim=0)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        dt_model = self.od_config.dtype
        tf = self.transformer
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        n = sp.num_outputs_per_prompt
        H, W = sp.height or 1024, sp.width or 1024
        h, w = H // 16, W // 16                                   # token grid (VAE / 8, pixel shuffle / 2)
        scale = float(sp.guidance_scale) if sp.guidance_scale_provided else self.default_guidance
        do_cfg = scale > 1.0
        pes = [p.get("prompt_embeds") if isinstance(p, dict) else None for p in req.prompts]
        if all(e is not None for e in pes):
            pe = torch.stack([e.reshape(-1, e.shape[-1]) for e in pes]).to(self.device_, dt_model)
        else:
            pe, _ = self.text_encoder(texts, self.device_, dt_model, sp.max_sequence_length)
        ne = None
        if do_cfg:
            ne, _ = self.text_encoder([""] * len(texts), self.device_, dt_model, sp.max_sequence_length)
        if n > 1:
            pe = pe.repeat_interleave(n, 0)
            ne = ne.repeat_interleave(n, 0) if ne is not None else None
        B = pe.shape[0]
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        C = tf.cfg.in_channels
        z = torch.randn(B, C, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = z.to(self.device_, torch.float32).flatten(2).transpose(1, 2).contiguous()          # [B, h*w, C]
        ids_img = image_ids(h, w)
        ref, ref_ids = self._reference_latents(req.prompts[0])
        if ref is not None:
            ids_img = torch.cat([ids_img, ref_ids], dim=0)
            ref = ref.expand(B, -1, -1).to(dt_model)
        ids_txt = text_ids(pe.shape[1])
        S = lat.shape[1]
        sig = np.linspace(1.0, 1 / sp.num_inference_steps, sp.num_inference_steps) if sp.sigmas is None else sp.sigmas
        ts = self.scheduler.set_timesteps(sigmas=sig, mu=compute_empirical_mu(S, sp.num_inference_steps), device=self.device_)
        lat_in = lat.to(dt_model)
        tv = torch.empty(B, device=self.device_)
        for i in range(len(ts)):
            tv.fill_(float(self.scheduler.sigmas[i]))
            x = lat_in if ref is None else torch.cat([lat_in, ref], dim=1)
            if do_cfg and self.cfg_exchange is not None:     # one branch per rank, velocities exchanged inside the step kernel
                mine = ne if self.cfg_exchange.is_negative_rank else pe
                v = tf(x, mine, tv, ids_img, ids_txt)[:, :S].contiguous()
                self.cfg_exchange.step(v, lat, scale, self.scheduler.dt(i), False, lat_in)
                continue
            v = tf(x, pe, tv, ids_img, ids_txt)[:, :S]
            vn = tf(x, ne, tv, ids_img, ids_txt, branch=1)[:, :S] if do_cfg else None
            fused.cfg_euler_step_(v.contiguous(), vn.contiguous() if vn is not None else None, lat, scale if do_cfg else 1.0,
                                  self.scheduler.dt(i), False, lat_in)
        z = lat.transpose(1, 2).reshape(B, C, h, w)
        mean, std = self._bn()
        z = unpatchify(z * std + mean)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=z)
        img = (self.vae_decode or self.vae.decode)(z)
        return DiffusionOutput(output=img, metrics={"num_steps": len(ts), "batch": B})
